"""Rollout strategies on top of ``GrpoTrainer.rollout`` / ``score``:

* ``BaseRolloutGenerator``      - fixed: ``rollout_gbs`` prompts x ``sampling_repeat_n`` samples, keep-n of repeat-n.
* ``DynamicSamplingGenerator``  - DAPO-style: drop prompt groups whose rewards are all equal (no learning signal),
  track the kept ratio with an EMA and refill up to ``max_refill_times``
  (gpatch_v4/rollout_generator/ds_generator.py; docs/source/dynamic_sampling.md:46-82).
* ``StaleRolloutQueue``         - sliding pipeline of the single-controller trainer: the batch trained at step k was
  generated with the weights of step k - s (``rollout_max_staleness = s``,
  gpatch_v4/trainer/grpo_single_ctrl_trainer.py:26-31); off-policy correction consumes ``rollout_log_probs``.
"""
from __future__ import annotations

from collections import deque
from typing import Callable, List, Optional

import torch

from ..configs.base import import_from_path


def keep_n_of_group(samples: List[dict], repeat_n: int, keep_n: int, strategy: str = "all") -> List[dict]:
    if keep_n >= repeat_n or strategy == "all":
        return samples
    out = []
    for g0 in range(0, len(samples), repeat_n):
        grp = samples[g0:g0 + repeat_n]
        if strategy == "top":
            grp = sorted(grp, key=lambda s: -float(torch.as_tensor(s["rewards"]).sum()))[:keep_n]
        elif strategy == "extremes":
            srt = sorted(grp, key=lambda s: float(torch.as_tensor(s["rewards"]).sum()))
            grp = srt[:keep_n // 2] + srt[-(keep_n - keep_n // 2):]
        else:
            grp = grp[:keep_n]
        out.extend(grp)
    return out


def default_group_filter(group: List[dict]) -> bool:
    """Keep a prompt group only when its rewards are not all identical."""
    r = [float(torch.as_tensor(s["rewards"]).sum()) for s in group]
    return max(r) - min(r) > 1e-8


class BaseRolloutGenerator:
    def __init__(self, trainer, config):
        self.tr, self.cfg = trainer, config
        t = config.training
        self.filter_fn: Optional[Callable] = None
        if t.filter_sampling_py_path:
            self.filter_fn = import_from_path(t.filter_sampling_py_path, t.filter_sampling_fn_name or "filter_fn")

    def __call__(self, prompt_iter, step: int) -> List[dict]:
        t = self.cfg.training
        prompts = next(prompt_iter)
        samples = self.tr.score(self.tr.rollout(prompts))
        if self.filter_fn is not None and t.filter_sampling_stage == "pre":
            samples = self.filter_fn(samples)
        return keep_n_of_group(samples, t.sampling_repeat_n, t.sampling_keep_n, t.sampling_keeping_strategy)

    def state_dict(self):
        return {}

    def load_state_dict(self, sd):
        pass


class DynamicSamplingGenerator(BaseRolloutGenerator):
    def __init__(self, trainer, config, group_filter: Callable = default_group_filter):
        super().__init__(trainer, config)
        ds = config.training.dynamic_sampling
        self.ds = ds
        self.group_filter = group_filter
        if ds.filter_py_path:
            self.group_filter = import_from_path(ds.filter_py_path, ds.filter_fn_name or "filter_group")
        self.keep_ratio_ema = 1.0 / max(ds.oversampling_ratio, 1.0)
        self.stats = {"refills": 0, "kept_groups": 0, "seen_groups": 0}

    def __call__(self, prompt_iter, step: int) -> List[dict]:
        t, ds = self.cfg.training, self.ds
        n = t.sampling_repeat_n
        kept: List[dict] = []
        target_groups = None
        samples: List[dict] = []
        for _ in range(ds.max_refill_times + 1):
            prompts = next(prompt_iter)
            if target_groups is None:
                target_groups = len(prompts)
            samples = self.tr.score(self.tr.rollout(prompts))
            groups = [samples[i:i + n] for i in range(0, len(samples), n)]
            good = [g for g in groups if self.group_filter(g)]
            self.stats["seen_groups"] += len(groups)
            self.stats["kept_groups"] += len(good)
            ratio = len(good) / max(len(groups), 1)
            self.keep_ratio_ema = ds.ema_decay * self.keep_ratio_ema + (1 - ds.ema_decay) * ratio
            for g in good:
                if len(kept) < target_groups * n:
                    kept.extend(g)
            if len(kept) >= target_groups * n:
                break
            self.stats["refills"] += 1
        if not kept:  # nothing informative after all refills: fall back to the last batch so the step still runs
            kept = samples[:target_groups * n]
        for gi in range(0, len(kept), n):
            for s in kept[gi:gi + n]:
                s["group_id"] = gi // n
        return kept

    def suggested_oversampling(self) -> float:
        return min(max(1.0 / max(self.keep_ratio_ema, 1e-3), 1.0), 8.0)

    def state_dict(self):
        return {"keep_ratio_ema": self.keep_ratio_ema, "stats": dict(self.stats)}

    def load_state_dict(self, sd):
        self.keep_ratio_ema = sd.get("keep_ratio_ema", self.keep_ratio_ema)
        self.stats.update(sd.get("stats", {}))


class StaleRolloutQueue:
    """Holds ``staleness + 1`` generated batches; ``push`` after generating with the current weights, ``pop`` returns
    the oldest.  With staleness 0 this is a pass-through."""

    def __init__(self, staleness: int):
        self.s = staleness
        self.q: deque = deque()

    def primed(self) -> bool:
        return len(self.q) > self.s

    def push(self, samples: List[dict], weight_version: int):
        for x in samples:
            x["weight_version"] = weight_version
        self.q.append(samples)

    def pop(self) -> List[dict]:
        return self.q.popleft()
