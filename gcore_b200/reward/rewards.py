"""Reward composition: rule-only, reward-model-only and mixed (``RewardFactory``, gpatch_v4/reward/*.py).

A reward function maps a list of samples to ``(reward [N], per_token_reward | None, metrics: {name: [N]})``; the rule
plug-in contract is the reference's (``fn(batched_data, tokenizer, actor_tokenizer)``, tasks/math_rl_v4/bt_reward.py:
82-152).  Reward models are ``TrainingEngine``s with a value head scoring the last token (BT-RM) or rollout engines
prompted to judge (generative RM, tasks/math_rl_v4/gen_rm_reward.py:30-131); several sources mix by ``reward_weight``.
"""
from __future__ import annotations

import re
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..configs.base import import_from_path


def boxed_answer(text: str) -> Optional[str]:
    """Last ``\\boxed{...}`` of a string (brace-balanced), the math recipes' answer extractor."""
    i = text.rfind("\\boxed{")
    if i < 0:
        return None
    depth, out = 0, []
    for ch in text[i + 7:]:
        if ch == "{":
            depth += 1
        elif ch == "}":
            if depth == 0:
                return "".join(out).strip()
            depth -= 1
        out.append(ch)
    return None


def math_rule_reward(samples: Sequence[dict], tokenizer=None, actor_tokenizer=None):
    """1.0 when the boxed answer of the decoded response equals ``gt_label`` (string compare after whitespace strip)."""
    tok = actor_tokenizer or tokenizer
    r, fmt = [], []
    for s in samples:
        resp = s.get("response_text")
        if resp is None and tok is not None:
            resp = tok.decode(s["tokens"][s["prompt_length"]:].tolist())
        ans = boxed_answer(resp or "")
        fmt.append(1.0 if ans is not None else 0.0)
        r.append(1.0 if ans is not None and str(ans).replace(" ", "") == str(s.get("gt_label")).replace(" ", "") else 0.0)
    return torch.tensor(r), None, {"format_ok": torch.tensor(fmt)}


class RuleReward:
    def __init__(self, fn: Callable, tokenizer=None):
        self.fn, self.tok = fn, tokenizer

    def __call__(self, samples):
        out = self.fn(samples, tokenizer=self.tok, actor_tokenizer=self.tok) if _wants_tok(self.fn) else self.fn(samples)
        return _norm(out, len(samples))


class BtRmReward:
    """Bradley-Terry reward model: scalar score of the last token through a value-head engine; all micro-batches are
    accumulated then scored once (``GrpoBtRmActor``, gpatch_v4/actor/grpo_bt_rm_actor.py:108-147)."""

    def __init__(self, rm_engine):
        self.engine = rm_engine

    def __call__(self, samples):
        scored = self.engine.compute_values([dict(s) for s in samples])
        r = torch.stack([torch.as_tensor(s["values"])[-2 if len(s["values"]) > 1 else -1].float() for s in scored])
        return r, None, {}


class GenRmReward:
    """Generative reward model: builds a grading prompt per response, samples ``repeat_n`` verdicts, parses yes / no
    into +-1 and averages."""

    def __init__(self, engine, build_prompt: Callable, parse: Callable, sampling, repeat_n: int = 1):
        self.engine, self.build_prompt, self.parse, self.sampling, self.repeat_n = engine, build_prompt, parse, sampling, repeat_n

    def __call__(self, samples):
        prompts = [self.build_prompt(s) for s in samples]
        reqs = self.engine.generate(prompts, self.sampling, n=self.repeat_n)
        r = []
        for i in range(len(samples)):
            votes = [self.parse(q.out_tokens) for q in reqs[i * self.repeat_n:(i + 1) * self.repeat_n]]
            r.append(sum(votes) / max(len(votes), 1))
        return torch.tensor(r, dtype=torch.float32), None, {}


class MixReward:
    def __init__(self, parts: List[tuple]):
        """``parts``: list of (name, reward callable, weight)."""
        self.parts = parts

    def __call__(self, samples):
        total = torch.zeros(len(samples))
        metrics: Dict[str, torch.Tensor] = {}
        per_tok = None
        per_head = {}
        for name, fn, w in self.parts:
            r, pt, m = _norm(fn(samples), len(samples))
            total += w * r
            per_head[name] = r
            metrics[f"{name}/reward"] = r
            metrics.update({f"{name}/{k}": v for k, v in m.items()})
            if pt is not None:
                per_tok = pt if per_tok is None else [a + w * b for a, b in zip(per_tok, pt)]
        for i, s in enumerate(samples):
            s["reward_dict"] = {k: float(v[i]) for k, v in per_head.items()}
        return total, per_tok, metrics


def _wants_tok(fn) -> bool:
    import inspect
    try:
        return "tokenizer" in inspect.signature(fn).parameters
    except (TypeError, ValueError):
        return False


def _norm(out, n):
    if isinstance(out, tuple):
        r, pt, m = (list(out) + [None, {}])[:3]
    else:
        r, pt, m = out, None, {}
    r = torch.as_tensor(r, dtype=torch.float32).reshape(-1)
    assert r.numel() == n, f"reward fn returned {r.numel()} rewards for {n} samples"
    return r, pt, (m or {})


def build_reward(cfg, tokenizer=None, rm_engines: Optional[Dict[str, object]] = None, default_rule: Optional[Callable] = None):
    """``cfg``: ``RewardConfig``.  rule_only | rm_only | mix."""
    rule = None
    if cfg.rule_py_path:
        rule = RuleReward(import_from_path(cfg.rule_py_path, cfg.rule_fn_name or "reward_fn"), tokenizer)
    elif default_rule is not None:
        rule = RuleReward(default_rule, tokenizer)
    rms = [(info.name, BtRmReward(rm_engines[info.name]), info.reward_weight)
           for info in cfg.reward_model_info if rm_engines and info.name in rm_engines]
    if cfg.reward_type == "rule_only":
        if rule is None:
            raise ValueError("rule_only reward needs rule_py_path or a default rule")
        return rule
    if cfg.reward_type == "rm_only":
        if not rms:
            raise ValueError("rm_only reward needs reward_model_info with loaded engines")
        return MixReward(rms)
    parts = ([("rule", rule, 1.0)] if rule is not None else []) + rms
    return MixReward(parts)


class ExternalAsyncReward:
    """Base class of rewards computed by an outside service (a sandbox, a judge behind HTTP, a verifier cluster):
    ``score_one(sample) -> float | (float, dict)`` is the only method a subclass has to write.  Samples are submitted
    in micro-batches to a thread pool as soon as they exist (``submit``), results stream back while the caller does
    other work, and ``__call__`` / ``collect`` hands them out in submission order.  A request that raises or exceeds
    ``timeout_s`` is retried ``retries`` times and then gets ``fallback`` (the reference's external async reward
    base with per-micro-batch streaming: gpatch_v4/reward/base_external_reward.py)."""

    def __init__(self, max_workers: int = 8, micro_batch: int = 8, timeout_s: float = 60.0, retries: int = 1,
                 fallback: float = 0.0):
        from concurrent.futures import ThreadPoolExecutor
        self.pool = ThreadPoolExecutor(max_workers=max_workers)
        self.micro_batch, self.timeout_s, self.retries, self.fallback = micro_batch, timeout_s, retries, fallback
        self._pending: List[tuple] = []
        self.stats = {"requests": 0, "failures": 0, "retries": 0}

    def score_one(self, sample: dict):
        raise NotImplementedError

    def score_batch(self, samples: List[dict]) -> List:
        """One micro-batch; override when the service takes batches."""
        return [self.score_one(s) for s in samples]

    def _guarded(self, samples: List[dict]) -> List:
        for attempt in range(self.retries + 1):
            try:
                return self.score_batch(samples)
            except Exception:  # noqa: BLE001 - a failing service must not kill the training step
                self.stats["retries" if attempt < self.retries else "failures"] += 1
        return [self.fallback] * len(samples)

    def submit(self, samples: List[dict]) -> None:
        for i in range(0, len(samples), self.micro_batch):
            mb = samples[i:i + self.micro_batch]
            self.stats["requests"] += 1
            self._pending.append((mb, self.pool.submit(self._guarded, mb)))

    def collect(self):
        """Rewards of everything submitted so far, in submission order."""
        from concurrent.futures import TimeoutError as FutTimeout
        rewards, extra = [], {}
        for mb, fut in self._pending:
            try:
                res = fut.result(timeout=self.timeout_s)
            except FutTimeout:
                self.stats["failures"] += 1
                res = [self.fallback] * len(mb)
            for s, r in zip(mb, res):
                if isinstance(r, tuple):
                    r, info = r
                    for k, v in info.items():
                        extra.setdefault(k, []).append(float(v))
                rewards.append(float(r))
        self._pending = []
        n = len(rewards)
        return torch.tensor(rewards, dtype=torch.float32), None, {k: torch.tensor(v) for k, v in extra.items()
                                                                  if len(v) == n}

    def __call__(self, samples):
        self.submit(list(samples))
        return self.collect()

    def close(self):
        self.pool.shutdown(wait=False, cancel_futures=True)
