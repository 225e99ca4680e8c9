"""Asynchronous rollout controller of the single-controller trainer.

A controller owns the prompt source and one or more sampler endpoints (``client.SamplerClient``-like objects with
``generate(prompts, params)``).  It keeps up to ``max_inflight`` prompt groups in flight on a worker pool, tags every
finished group with the weight version it was generated with, and serves training batches subject to a staleness
window: a group generated with weights older than ``current_version - rollout_max_staleness`` is dropped (or, with
``keep_stale``, kept for off-policy correction).  Tail batching: when fewer than a full batch of groups is still in
flight at the end of a window the controller tops the batch up with the freshest finished groups instead of waiting
for stragglers.  Behavioural model: ``RolloutController`` (0-GPU actor: data source, fire / collect, staleness window,
tail batching, DP split; gpatch_v4/rollout_generator/async_rollout/rollout_controller.py:145-1459).
"""
from __future__ import annotations

import threading
import time
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterator, List, Optional


@dataclass
class RolloutGroup:
    prompt_id: int
    prompt: List[int]
    weight_version: int
    samples: List[dict] = field(default_factory=list)
    finished_at: float = 0.0


class RolloutController:
    def __init__(self, prompt_iter: Iterator[List[List[int]]], samplers: List[object], score_fn: Callable,
                 repeat_n: int, groups_per_batch: int, max_staleness: int = 1, max_inflight: Optional[int] = None,
                 keep_stale: bool = False, tail_wait_s: float = 0.0, sampling_params=None,
                 over_dispatch_ratio: float = 1.0, reuse_unused_prompts: bool = False):
        self.prompt_iter, self.samplers, self.score_fn = prompt_iter, samplers, score_fn
        self.repeat_n, self.groups_per_batch = repeat_n, groups_per_batch
        self.max_staleness, self.keep_stale, self.tail_wait_s = max_staleness, keep_stale, tail_wait_s
        # over-dispatch: more groups in flight than a batch needs, so a batch is made of the first to finish and
        # stragglers do not hold it up; prompts of groups that went stale unused can be generated again
        import math
        self.max_inflight = max_inflight or math.ceil(groups_per_batch * (max_staleness + 1) *
                                                      max(over_dispatch_ratio, 1.0))
        self.reuse_unused_prompts = reuse_unused_prompts
        self.params = sampling_params
        self.version = 0
        self._pool = ThreadPoolExecutor(max_workers=max(len(samplers), 1))
        self._inflight: Dict[int, Future] = {}
        self._done: List[RolloutGroup] = []
        self._lock = threading.Lock()
        self._next_id = 0
        self._pending_prompts: List[List[int]] = []
        self.stats = dict(fired=0, collected=0, dropped_stale=0, tail_batches=0, reused_prompts=0)

    # ---- weight versions
    def set_weight_version(self, v: int):
        self.version = v

    # ---- fire
    def _take_prompt(self) -> List[int]:
        if not self._pending_prompts:
            self._pending_prompts = list(next(self.prompt_iter))
        return self._pending_prompts.pop(0)

    def _run_group(self, g: RolloutGroup, sampler) -> RolloutGroup:
        outs = sampler.generate([g.prompt] * self.repeat_n, self.params)
        samples = []
        for o in outs:
            s = dict(o) if isinstance(o, dict) else {"tokens": o}
            s.update(prompt_id=g.prompt_id, group_id=g.prompt_id, weight_version=g.weight_version,
                     prompt_length=len(g.prompt))
            samples.append(s)
        g.samples = self.score_fn(samples)
        g.finished_at = time.time()
        return g

    def _run_groups(self, groups: List[RolloutGroup], sampler) -> List[RolloutGroup]:
        """All groups handed to one sampler in this dispatch, as ONE engine call: a continuous-batching engine decodes
        ``len(groups) * repeat_n`` sequences per step instead of ``repeat_n``."""
        outs = sampler.generate_groups([g.prompt for g in groups], self.repeat_n, self.params)
        assert len(outs) == len(groups) * self.repeat_n, "a batched sampler returns repeat_n samples per prompt, in order"
        now = time.time()
        for k, g in enumerate(groups):
            samples = []
            for o in outs[k * self.repeat_n:(k + 1) * self.repeat_n]:
                s = dict(o) if isinstance(o, dict) else {"tokens": o}
                s.update(prompt_id=g.prompt_id, group_id=g.prompt_id, weight_version=g.weight_version,
                         prompt_length=len(g.prompt))
                samples.append(s)
            g.samples = self.score_fn(samples)
            g.finished_at = now
        return groups

    def fire(self):
        """Tops the in-flight set up to ``max_inflight`` groups.  Samplers that offer ``generate_groups`` receive all
        of their new groups in one call; the others one call per group."""
        with self._lock:
            new: Dict[int, List[RolloutGroup]] = {}
            while len(self._inflight) + len(self._done) < self.max_inflight:
                g = RolloutGroup(self._next_id, self._take_prompt(), self.version)
                si = self._next_id % len(self.samplers)
                sampler = self.samplers[si]
                if hasattr(sampler, "generate_groups"):
                    new.setdefault(si, []).append(g)
                    self._inflight[g.prompt_id] = None  # filled below, once the sampler's round is complete
                else:
                    self._inflight[g.prompt_id] = self._pool.submit(self._run_group, g, sampler)
                self._next_id += 1
                self.stats["fired"] += 1
            for si, groups in new.items():
                fut = self._pool.submit(self._run_groups, groups, self.samplers[si])
                for g in groups:
                    self._inflight[g.prompt_id] = fut
                self.stats["batched_calls"] = self.stats.get("batched_calls", 0) + 1

    # ---- collect
    def _harvest(self):
        with self._lock:
            for pid in [p for p, f in self._inflight.items() if f is not None and f.done()]:
                if pid not in self._inflight:
                    continue  # finished together with an earlier group of the same batched call
                res = self._inflight.pop(pid).result()
                for g in (res if isinstance(res, list) else [res]):
                    self._inflight.pop(g.prompt_id, None)
                    self._done.append(g)
                    self.stats["collected"] += 1

    def _fresh(self) -> List[RolloutGroup]:
        keep, drop = [], 0
        for g in self._done:
            if self.version - g.weight_version <= self.max_staleness or self.keep_stale:
                keep.append(g)
            else:
                drop += 1
                if self.reuse_unused_prompts:
                    self._pending_prompts.append(g.prompt)
                    self.stats["reused_prompts"] += 1
        self._done = keep
        self.stats["dropped_stale"] += drop
        return keep

    def collect(self, timeout_s: float = 600.0) -> List[dict]:
        """Blocks until ``groups_per_batch`` fresh groups are available (oldest first) and returns their samples."""
        t0 = time.time()
        tail_deadline = None
        while True:
            self.fire()
            self._harvest()
            fresh = self._fresh()
            if len(fresh) >= self.groups_per_batch:
                break
            if self.tail_wait_s and fresh and tail_deadline is None:
                tail_deadline = time.time() + self.tail_wait_s
            if tail_deadline is not None and time.time() > tail_deadline and fresh:
                self.stats["tail_batches"] += 1  # serve a short batch rather than wait for stragglers
                break
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"rollout controller: {len(fresh)} of {self.groups_per_batch} groups after {timeout_s}s")
            time.sleep(0.001)
        fresh.sort(key=lambda g: (g.weight_version, g.prompt_id))
        take = fresh[:self.groups_per_batch]
        ids = {g.prompt_id for g in take}
        self._done = [g for g in self._done if g.prompt_id not in ids]
        return [s for g in take for s in g.samples]

    @staticmethod
    def split_for_dp(samples: List[dict], dp_size: int, repeat_n: int) -> List[List[dict]]:
        """Whole prompt groups per data-parallel rank, round-robin."""
        groups = [samples[i:i + repeat_n] for i in range(0, len(samples), repeat_n)]
        return [[s for g in groups[r::dp_size] for s in g] for r in range(dp_size)]

    def state_dict(self):
        return {"next_id": self._next_id, "version": self.version, "stats": dict(self.stats)}

    def load_state_dict(self, sd):
        self._next_id, self.version = sd["next_id"], sd["version"]
        self.stats.update(sd.get("stats", {}))

    def shutdown(self):
        self._pool.shutdown(wait=False, cancel_futures=True)
