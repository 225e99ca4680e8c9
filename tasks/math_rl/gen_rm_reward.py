"""Generative-reward-model plug-ins of the math recipe (``bt_rm.reward_model_info[*].py_path`` / ``fn_name``): how a
sample becomes a grading prompt and how the grader's text becomes a score (the role of the reference's
tasks/math_rl_v4/gen_rm_reward.py).  The grader model is another rollout engine; ``gen_reward_repeat_n`` verdicts per
sample are averaged by the caller."""
import re

GRADER_TEMPLATE = ("You are grading a solution to a math problem.\n\nProblem:\n{question}\n\nReference answer: {answer}\n\n"
                  "Solution:\n{response}\n\nIs the final answer of the solution equal to the reference answer? "
                  "Reply with 'Verdict: correct' or 'Verdict: wrong'.")
_VERDICT = re.compile(r"verdict\s*:\s*(correct|wrong)", re.IGNORECASE)


def build_grader_prompt(sample: dict, tokenizer=None) -> str:
    """Text the grader model completes.  ``sample`` carries ``prompt_text`` / ``response_text`` (or token ids that the
    tokenizer decodes) and the dataset's ``answer``."""
    def text(key_text, key_ids):
        if sample.get(key_text) is not None:
            return sample[key_text]
        ids = sample.get(key_ids)
        return tokenizer.decode(list(ids)) if (tokenizer is not None and ids is not None) else ""
    return GRADER_TEMPLATE.format(question=text("prompt_text", "prompt_ids"), answer=sample.get("answer", ""),
                                 response=text("response_text", "response_ids"))


def parse_verdict(grader_text: str) -> float:
    """1.0 for a 'correct' verdict, 0.0 for 'wrong'; a reply without a verdict scores 0 (the last verdict counts when
    the grader changes its mind)."""
    hits = _VERDICT.findall(grader_text or "")
    return 1.0 if hits and hits[-1].lower() == "correct" else 0.0
