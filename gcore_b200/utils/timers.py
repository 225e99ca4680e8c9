"""Named phase timers (Megatron-style ``Timers`` of the reference, gpatch_v4/utils/timer_utils.py:96-481): wall-clock
by default, CUDA-event based when ``device_timing`` is set so the GPU time of a phase is measured on the stream, with
min / max reduction across ranks for reports."""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


def _world_group():
    from ..core import parallel_state as ps
    return ps.get_world_group()


class _Timer:
    def __init__(self, device_timing: bool):
        self.device = device_timing and torch.cuda.is_available()
        self.elapsed_total = 0.0
        self.count = 0
        self._last = 0.0
        self._t0 = None
        self._ev = None

    def start(self, barrier=False):
        if barrier and dist.is_initialized():
            dist.barrier(group=_world_group())
        if self.device:
            self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._ev[0].record()
        else:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self._t0 = time.perf_counter()

    def stop(self):
        if self.device:
            self._ev[1].record()
            self._ev[1].synchronize()
            self._last = self._ev[0].elapsed_time(self._ev[1]) / 1e3
        else:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self._last = time.perf_counter() - self._t0
        self.elapsed_total += self._last
        self.count += 1
        return self._last


class Timers:
    def __init__(self, device_timing: bool = False):
        self.device_timing = device_timing
        self._t: Dict[str, _Timer] = {}

    def __call__(self, name) -> _Timer:
        if name not in self._t:
            self._t[name] = _Timer(self.device_timing)
        return self._t[name]

    def start(self, name, barrier=False):
        self(name).start(barrier)

    def stop(self, name):
        return self(name).stop()

    def last(self, name) -> float:
        return self(name)._last

    def mean(self, name) -> float:
        t = self(name)
        return t.elapsed_total / max(t.count, 1)

    def reset(self):
        self._t.clear()

    def minmax_across_ranks(self, names: Optional[List[str]] = None, group=None) -> Dict[str, tuple]:
        names = names or sorted(self._t)
        vals = torch.tensor([self.last(n) for n in names], dtype=torch.float64)
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
            lo, hi = vals.clone().to(dev), vals.clone().to(dev)
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
            return {n: (float(lo[i]), float(hi[i])) for i, n in enumerate(names)}
        return {n: (float(v), float(v)) for n, v in zip(names, vals)}
