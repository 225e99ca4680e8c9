"""Failure events, host-side fault injection, heartbeat-based hang detection and the relaunch loop.

The reference detects a hang when a train actor's ``last_progress_time`` goes stale and a crash when the awaited actor
task raises; it then tears everything down, optionally replaces nodes and relaunches from the latest checkpoint
(gpatch_v4/trainer/trainer_mixin.py:57-220, gpatch_v4/orches/failure.py:17-51, actor/mixin.py:1221-1236).  Here ranks
are plain processes: each stamps a heartbeat file per step, the launcher watches the files and the exit codes.
Faults are injected on the host only (an exception at a chosen step, a rank that stops stamping, a rank that exits);
nothing ever faults or hangs a GPU on purpose.
"""
from __future__ import annotations

import enum
import json
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


class FailureType(enum.Enum):
    CRASH = "crash"
    HANG = "hang"


@dataclass
class FailureEvent:
    type: FailureType
    rank: Optional[int] = None
    node: Optional[str] = None
    detail: str = ""
    time: float = field(default_factory=time.time)

    def to_dict(self):
        return dict(type=self.type.value, rank=self.rank, node=self.node, detail=self.detail, time=self.time)


class InjectedFault(RuntimeError):
    pass


class FaultInjector:
    """Host-side fault injection driven by ``debug.fault_injection``:
    ``{"raise_at_step": n, "rank": r}``, ``{"exit_at_step": n, "rank": r}``, ``{"stall_at_step": n, "rank": r}``,
    optionally ``"only_attempt": k`` so the relaunched attempt runs clean."""

    def __init__(self, spec: Optional[dict], rank: int, attempt: int = 0):
        self.spec = dict(spec or {})
        self.rank = rank
        self.attempt = attempt

    def _mine(self):
        if not self.spec:
            return False
        if "only_attempt" in self.spec and self.spec["only_attempt"] != self.attempt:
            return False
        return self.spec.get("rank", 0) == self.rank

    def at_step(self, step: int):
        if not self._mine():
            return
        if self.spec.get("raise_at_step") == step:
            raise InjectedFault(f"injected exception at step {step} on rank {self.rank}")
        if self.spec.get("exit_at_step") == step:
            os._exit(17)
        if self.spec.get("stall_at_step") == step:
            time.sleep(float(self.spec.get("stall_seconds", 3600)))


class Heartbeat:
    """One small json file per rank, rewritten at every step boundary (never from inside GPU work)."""

    def __init__(self, directory: str, rank: int):
        self.path = os.path.join(directory, f"heartbeat_{rank}.json")
        os.makedirs(directory, exist_ok=True)

    def stamp(self, step: int, **extra):
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump({"step": step, "time": time.time(), **extra}, f)
        os.replace(tmp, self.path)

    @staticmethod
    def read_all(directory: str) -> Dict[int, dict]:
        out = {}
        if not os.path.isdir(directory):
            return out
        for fn in os.listdir(directory):
            if fn.startswith("heartbeat_") and fn.endswith(".json"):
                try:
                    out[int(fn[len("heartbeat_"):-5])] = json.load(open(os.path.join(directory, fn)))
                except (ValueError, json.JSONDecodeError, OSError):
                    continue
        return out


def check_liveness(directory: str, world: int, max_wait_s: float, now: Optional[float] = None) -> Optional[FailureEvent]:
    """Returns a HANG event when any rank's last stamp is older than ``max_wait_s`` (a rank that never stamped is
    judged from the directory's creation time)."""
    now = now if now is not None else time.time()
    beats = Heartbeat.read_all(directory)
    t_dir = os.path.getmtime(directory) if os.path.isdir(directory) else now
    for r in range(world):
        last = beats.get(r, {}).get("time", t_dir)
        if now - last > max_wait_s:
            return FailureEvent(FailureType.HANG, rank=r, detail=f"no progress for {now - last:.1f}s")
    return None


class NodeReplacer:
    """Hook for swapping out a bad node before a relaunch (``training.node_replacer_cls``)."""

    def evict(self, event: FailureEvent):
        raise NotImplementedError

    def provision(self, n: int):
        raise NotImplementedError

    def wait_cluster_ready(self, expected_nodes: int, timeout_s: float) -> bool:
        raise NotImplementedError


class MockNodeReplacer(NodeReplacer):
    def __init__(self):
        self.evicted: List[FailureEvent] = []
        self.provisioned = 0

    def evict(self, event):
        self.evicted.append(event)

    def provision(self, n):
        self.provisioned += n

    def wait_cluster_ready(self, expected_nodes, timeout_s):
        return True


def run_with_recovery(launch_and_run: Callable[[int], Optional[FailureEvent]], max_restart_attempts: int,
                      node_replacer: Optional[NodeReplacer] = None, expected_nodes: int = 1,
                      on_event: Optional[Callable[[FailureEvent, int], None]] = None) -> List[FailureEvent]:
    """Calls ``launch_and_run(attempt)`` up to ``max_restart_attempts + 1`` times; it returns ``None`` on success or
    the failure that ended the attempt.  Resume state comes from the latest checkpoint inside ``launch_and_run``."""
    events: List[FailureEvent] = []
    for attempt in range(max_restart_attempts + 1):
        ev = launch_and_run(attempt)
        if ev is None:
            return events
        events.append(ev)
        if on_event:
            on_event(ev, attempt)
        if attempt == max_restart_attempts:
            raise RuntimeError(f"job failed after {attempt + 1} attempts: {[e.to_dict() for e in events]}")
        if node_replacer is not None:
            node_replacer.evict(ev)
            node_replacer.provision(1)
            if not node_replacer.wait_cluster_ready(expected_nodes, 600.0):
                raise RuntimeError("cluster did not become ready after node replacement")
    return events
