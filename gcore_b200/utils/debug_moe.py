"""Expert-load diagnostics for MoE models: forward hooks on every router record, per layer and call, how the tokens
were spread over the experts; ``summary()`` reduces the records to the figures one looks at when a run misbehaves
(load imbalance, dead experts, routing entropy) and ``dump()`` appends them to a jsonl file
(the reference's MoE debug dumps: ``gpatch_v4/utils/debug_moe.py``)."""
from __future__ import annotations

import json
import math
from typing import Dict, List, Optional

import torch


class MoeLoadRecorder:
    def __init__(self, model: torch.nn.Module, every: int = 1):
        from ..models.moe import Router
        self.every, self.calls = max(every, 1), 0
        self.records: Dict[int, List[torch.Tensor]] = {}
        self._handles = []
        for mod in model.modules():
            if isinstance(mod, Router):
                self._handles.append(mod.register_forward_hook(self._hook))

    def _hook(self, mod, args, out):
        self.calls += 1
        if self.calls % self.every:
            return
        idx = out[0].detach()
        E = mod.cfg.num_experts
        cnt = torch.zeros(E, dtype=torch.int64, device=idx.device).scatter_add_(
            0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.int64, device=idx.device))
        self.records.setdefault(mod.layer_idx, []).append(cnt.cpu())

    def summary(self) -> Dict[int, dict]:
        out = {}
        for layer, cnts in sorted(self.records.items()):
            tot = torch.stack(cnts).sum(0).double()
            p = tot / tot.sum().clamp_min(1.0)
            ent = float(-(p[p > 0] * p[p > 0].log()).sum())
            out[layer] = {"tokens": int(tot.sum()), "max_over_mean": float(tot.max() / tot.mean().clamp_min(1e-9)),
                          "dead_experts": int((tot == 0).sum()), "entropy": ent,
                          "entropy_frac": ent / math.log(len(tot)) if len(tot) > 1 else 1.0,
                          "counts": [int(x) for x in tot]}
        return out

    def dump(self, path: str, step: Optional[int] = None, reset: bool = True):
        with open(path, "a") as f:
            f.write(json.dumps({"step": step, "layers": {str(k): v for k, v in self.summary().items()}}) + "\n")
        if reset:
            self.records.clear()

    def close(self):
        for h in self._handles:
            h.remove()
        self._handles = []
