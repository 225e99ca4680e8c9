"""Evaluation / reward service over the RPC layer (the reference's eval server and client tools): a process that owns
a scoring function (a rule reward, a reward-model engine, an ``EvaluateRunner``) answers ``score`` and ``evaluate``
requests from training jobs or notebooks.

Server:  ``python -m gcore_b200.tools.eval_server --reward-py rewards.py --reward-fn reward_fn --port 8123``
Client:  ``EvalClient(["http://host:8123"]).score(samples)`` -> list of floats; ``.evaluate(samples, n, ks)`` ->
metrics (mean reward, pass@k).  Samples are dicts with ``tokens`` / ``prompt_length`` (token-id lists travel as JSON
or pickled tensors, as the RPC layer encodes them)."""
from __future__ import annotations

import argparse
import time
from typing import Callable, Dict, List, Sequence

import torch

from ..client.rpc import HttpRpcClient, serve
from ..evaluate.runner import pass_at_k


class EvalService:
    def __init__(self, reward_fn: Callable):
        self.reward_fn = reward_fn
        self.stats = {"requests": 0, "samples": 0}

    def _rewards(self, samples: List[dict]) -> List[float]:
        for s in samples:
            s["tokens"] = torch.as_tensor(s["tokens"])
        out = self.reward_fn(samples)
        r = out[0] if isinstance(out, tuple) else out
        self.stats["requests"] += 1
        self.stats["samples"] += len(samples)
        return [float(x) for x in torch.as_tensor(r, dtype=torch.float32).reshape(-1)]

    def score(self, samples: List[dict]) -> List[float]:
        return self._rewards(samples)

    def evaluate(self, samples: List[dict], n: int = 1, ks: Sequence[int] = (1,), threshold: float = 0.5) -> Dict[str, float]:
        """``samples`` prompt-major, ``n`` per prompt."""
        r = torch.tensor(self._rewards(samples)).view(-1, n)
        correct = (r > threshold).sum(1)
        out = {"eval/reward_mean": float(r.mean()), "eval/num_samples": float(r.numel())}
        for k in ks:
            out[f"eval/pass@{k}"] = sum(pass_at_k(n, int(c), int(k)) for c in correct) / max(r.shape[0], 1)
        return out

    def health(self) -> dict:
        return dict(self.stats)


class EvalClient:
    def __init__(self, urls: List[str], timeout_s: float = 600.0):
        self.rpc = HttpRpcClient(urls, timeout_s=timeout_s)

    @staticmethod
    def _plain(samples):
        return [{k: (v.tolist() if isinstance(v, torch.Tensor) else v) for k, v in s.items()
                 if k in ("tokens", "prompt_length", "gt_label", "response_text")} for s in samples]

    def score(self, samples, sample_idx: int = 0):
        return self.rpc.call("score", {"samples": self._plain(samples)}, sample_idx)

    def evaluate(self, samples, n: int = 1, ks=(1,), threshold: float = 0.5):
        return self.rpc.call("evaluate", {"samples": self._plain(samples), "n": n, "ks": list(ks),
                                          "threshold": threshold})

    def health(self):
        return self.rpc.multicast("health")


def main(argv=None):
    from ..configs.base import import_from_path
    ap = argparse.ArgumentParser()
    ap.add_argument("--reward-py", required=True)
    ap.add_argument("--reward-fn", default="reward_fn")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=0)
    a = ap.parse_args(argv)
    srv, url = serve(EvalService(import_from_path(a.reward_py, a.reward_fn)), a.host, a.port,
                     allowed=["score", "evaluate", "health"])
    print(f"eval service at {url}", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.shutdown()


if __name__ == "__main__":
    main()
