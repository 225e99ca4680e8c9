"""Evaluation runner (gpatch_v4/evaluate/evaluate_runner.py, inference_runner.py): samples ``n`` responses per prompt
with the rollout engine, scores them with the job's reward function and reports mean reward, pass@k and response
length, reduced over data-parallel ranks."""
from __future__ import annotations

from math import comb
from typing import Callable, Dict, List, Sequence

import torch
import torch.distributed as dist


def pass_at_k(n: int, c: int, k: int) -> float:
    """Unbiased estimator: 1 - C(n - c, k) / C(n, k) for c correct of n samples."""
    if n - c < k:
        return 1.0
    return 1.0 - comb(n - c, k) / comb(n, k)


class EvaluateRunner:
    def __init__(self, generate: Callable[[List[List[int]]], List[dict]], score: Callable[[List[dict]], torch.Tensor],
                 n: int, ks: Sequence[int] = (1,), threshold: float = 0.5, dp_group=None):
        self.generate, self.score, self.n, self.ks, self.threshold, self.group = generate, score, n, tuple(ks), threshold, \
            dp_group

    def run(self, prompts: List[List[int]]) -> Dict[str, float]:
        samples = self.generate(prompts)
        assert len(samples) == len(prompts) * self.n, "the generator must return n samples per prompt, prompt-major"
        r = torch.as_tensor(self.score(samples), dtype=torch.float64).view(len(prompts), self.n)
        correct = (r > self.threshold).sum(1)
        acc = torch.zeros(3 + len(self.ks), dtype=torch.float64)
        acc[0] = r.sum()
        acc[1] = float(r.numel())
        acc[2] = float(sum(len(s["tokens"]) - int(s.get("prompt_length", 0)) for s in samples))
        for j, k in enumerate(self.ks):
            acc[3 + j] = sum(pass_at_k(self.n, int(c), k) for c in correct)
        prompts_n = torch.tensor([float(len(prompts))], dtype=torch.float64)
        if self.group is not None and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dev = "cuda" if dist.get_backend(self.group) == "nccl" else "cpu"
            a, p = acc.to(dev), prompts_n.to(dev)
            dist.all_reduce(a, group=self.group)
            dist.all_reduce(p, group=self.group)
            acc, prompts_n = a.cpu(), p.cpu()
        out = {"eval/reward_mean": float(acc[0] / acc[1]), "eval/response_length": float(acc[2] / acc[1]),
               "eval/num_samples": float(acc[1])}
        for j, k in enumerate(self.ks):
            out[f"eval/pass@{k}"] = float(acc[3 + j] / prompts_n[0])
        return out
