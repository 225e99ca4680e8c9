"""Rule reward of the math recipe: 1.0 when the \\boxed{...} answer of the response equals the reference answer
(after whitespace / trailing-period normalisation), else 0.0; responses without a boxed answer get 0.0
(tasks/math_rl_v4/bt_reward.py and math_external_reward.py in the reference)."""
import torch

from gcore_b200.reward.rewards import boxed_answer


def _norm(a):
    return None if a is None else a.strip().rstrip(".").replace(" ", "")


def math_reward(samples, tokenizer=None, **_):
    out = []
    for s in samples:
        text = s.get("response_text")
        if text is None and tokenizer is not None:
            text = tokenizer.decode(torch.as_tensor(s["tokens"][s["prompt_length"]:]).tolist())
        got, want = _norm(boxed_answer(text or "")), _norm(str(s.get("answer", "")))
        out.append(1.0 if got is not None and got == want else 0.0)
    return torch.tensor(out)
