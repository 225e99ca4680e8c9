"""Step profiler: ``torch.profiler`` between ``profile_start_step`` and ``profile_end_step`` with a Chrome trace per
selected rank, a communication-vs-compute summary built from kernel names, NVTX ranges and a memory / time context
manager (the reference's ``ProfileMixin``, gpatch_v4/actor/mixin.py:1239-1380, and ``profile_memory_and_time``,
gpatch_v4/training_backend/megatron_backend/mcore_swap_impl.py:36-98)."""
from __future__ import annotations

import contextlib
import gzip
import os
import shutil
import time
from typing import Dict, List, Optional

import torch

COMM_MARKERS = ("nccl", "all_gather", "allgather", "reduce_scatter", "all_reduce", "allreduce", "alltoall", "sendrecv",
                "gemm_comm", "zero1", "ep_push", "ep_pull", "peer_", "broadcast")


class StepProfiler:
    def __init__(self, cfg=None, rank: int = 0, out_dir: Optional[str] = None):
        g = (lambda k, d: getattr(cfg, k, d)) if cfg is not None else (lambda k, d: d)
        self.enabled = bool(g("use_profiler", g("enable", False)))
        self.start_step, self.end_step = int(g("profile_start_step", 2)), int(g("profile_end_step", 3))
        ranks = g("export_ranks", None)
        self.export = ranks is None or rank in list(ranks)
        self.gzip = bool(g("gzip_trace", False) or g("gzip", False))
        self.rank = rank
        self.out_dir = out_dir or g("export_dir", None) or g("profile_dir", "./profile")
        self._prof = None
        self.summary: Dict[str, float] = {}

    def step_begin(self, step: int):
        if not self.enabled or self._prof is not None or step != self.start_step:
            return
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts, record_shapes=False, with_stack=False)
        self._prof.__enter__()

    def step_end(self, step: int):
        if self._prof is None or step != self.end_step:
            return
        prof, self._prof = self._prof, None
        prof.__exit__(None, None, None)
        self.summary = comm_compute_summary(prof)
        if self.export:
            os.makedirs(self.out_dir, exist_ok=True)
            path = os.path.join(self.out_dir, f"trace_rank{self.rank}_step{self.start_step}-{self.end_step}.json")
            prof.export_chrome_trace(path)
            if self.gzip:
                with open(path, "rb") as f, gzip.open(path + ".gz", "wb") as g:
                    shutil.copyfileobj(f, g)
                os.remove(path)
        return self.summary


def comm_compute_summary(prof) -> Dict[str, float]:
    """Device time split into communication and compute kernels by name (CPU-only profiles report CPU self time)."""
    comm = comp = 0.0
    for ev in prof.key_averages():
        t = float(getattr(ev, "self_device_time_total", 0.0) or getattr(ev, "self_cuda_time_total", 0.0) or 0.0)
        if t == 0.0:
            t = float(ev.self_cpu_time_total) if not torch.cuda.is_available() else 0.0
        name = ev.key.lower()
        if any(m in name for m in COMM_MARKERS):
            comm += t
        else:
            comp += t
    tot = comm + comp
    return {"comm_us": comm, "compute_us": comp, "comm_frac": comm / tot if tot else 0.0}


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


@contextlib.contextmanager
def profile_memory_and_time(tag: str, log=None, sync: bool = True):
    """Logs wall time and the change in allocated / reserved device memory across the block."""
    cuda = torch.cuda.is_available()
    if cuda and sync:
        torch.cuda.synchronize()
    a0 = torch.cuda.memory_allocated() if cuda else 0
    r0 = torch.cuda.memory_reserved() if cuda else 0
    t0 = time.perf_counter()
    out: Dict[str, float] = {}
    try:
        yield out
    finally:
        if cuda and sync:
            torch.cuda.synchronize()
        out.update(seconds=time.perf_counter() - t0,
                   allocated_delta_gb=((torch.cuda.memory_allocated() if cuda else 0) - a0) / 2**30,
                   reserved_delta_gb=((torch.cuda.memory_reserved() if cuda else 0) - r0) / 2**30)
        if log is not None:
            log.info(f"[{tag}] {out['seconds']:.3f}s allocated {out['allocated_delta_gb']:+.2f} GB "
                     f"reserved {out['reserved_delta_gb']:+.2f} GB")
