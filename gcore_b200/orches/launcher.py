"""Process launcher: one SPMD rank per GPU on this node (the role Ray + placement groups play for the reference,
gpatch_v4/orches/__init__.py:52-143, train_group.py:79-168).  Starts the ranks with the torchrun environment contract
(RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT), propagates selected env keys, watches exit codes and
heartbeats, and turns what it sees into ``FailureEvent``s for the relaunch loop."""
from __future__ import annotations

import os
import signal
import socket
import subprocess
import sys
import time
from typing import Dict, List, Optional, Sequence

from .failure import FailureEvent, FailureType, check_liveness

PROPAGATE_ENV_KEYS = ("PYTHONPATH", "NCCL_DEBUG", "NCCL_NVLS_ENABLE", "CUDA_VISIBLE_DEVICES", "GCORE_B200_FORCE_EAGER",
                      "GCORE_FUSED_TP", "OMP_NUM_THREADS")


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class LocalLauncher:
    def __init__(self, nproc: int, heartbeat_dir: Optional[str] = None, max_wait_s: float = 3600.0,
                 poll_s: float = 1.0, extra_env: Optional[Dict[str, str]] = None):
        self.nproc, self.heartbeat_dir, self.max_wait_s, self.poll_s = nproc, heartbeat_dir, max_wait_s, poll_s
        self.extra_env = extra_env or {}
        self.procs: List[subprocess.Popen] = []

    def launch(self, argv: Sequence[str], attempt: int = 0):
        port = free_port()
        self.procs = []
        for r in range(self.nproc):
            env = dict(os.environ)
            env.update(self.extra_env)
            env.update(RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(self.nproc), MASTER_ADDR="127.0.0.1",
                       MASTER_PORT=str(port), GCORE_ATTEMPT=str(attempt))
            if self.heartbeat_dir:
                env["GCORE_HEARTBEAT_DIR"] = self.heartbeat_dir
            self.procs.append(subprocess.Popen([sys.executable, *argv], env=env, start_new_session=True))
        return self

    def wait(self) -> Optional[FailureEvent]:
        """Blocks until every rank exits 0 (returns None), a rank fails (CRASH) or heartbeats go stale (HANG); the
        remaining ranks are then stopped by PID."""
        t_start = time.time()
        while True:
            codes = [p.poll() for p in self.procs]
            bad = [(r, c) for r, c in enumerate(codes) if c not in (None, 0)]
            if bad:
                self.shutdown()
                r, c = bad[0]
                return FailureEvent(FailureType.CRASH, rank=r, node=socket.gethostname(), detail=f"exit code {c}")
            if all(c == 0 for c in codes):
                return None
            if self.heartbeat_dir and time.time() - t_start > self.max_wait_s:
                ev = check_liveness(self.heartbeat_dir, self.nproc, self.max_wait_s)
                if ev is not None:
                    ev.node = socket.gethostname()
                    self.shutdown()
                    return ev
            time.sleep(self.poll_s)

    def shutdown(self, grace_s: float = 10.0):
        for p in self.procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)  # exact process group of a child we started
                except (ProcessLookupError, PermissionError):
                    pass
        t0 = time.time()
        for p in self.procs:
            try:
                p.wait(timeout=max(0.1, grace_s - (time.time() - t0)))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except (ProcessLookupError, PermissionError):
                    pass
