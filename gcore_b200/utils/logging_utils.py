"""Structured logging with the reference's record format ``time - level - role= - rank= - pid= - node= - msg``
(docs/source/logging.md:43-48): one task directory ``<base>/<run>_<timestamp>/``, ``training.log`` written by rank 0
only, optional per-rank DEBUG shards, and a ``TeeStream`` that mirrors stdout / stderr into the log atomically."""
from __future__ import annotations

import logging
import os
import socket
import sys
import threading
import time
from typing import Optional

_FMT = "%(asctime)s - %(levelname)s - role=%(role)s - rank=%(rank)s - pid=%(process)d - node=%(node)s - %(message)s"
_STATE = {"dir": None, "role": "driver", "rank": 0}


class _Ctx(logging.Filter):
    def filter(self, record):
        record.role = _STATE["role"]
        record.rank = _STATE["rank"]
        record.node = socket.gethostname()
        return True


class TeeStream:
    """Writes to the wrapped stream and appends whole lines to a file under a lock."""

    def __init__(self, stream, path):
        self.stream, self.path = stream, path
        self.lock = threading.Lock()
        self.buf = ""

    def write(self, data):
        self.stream.write(data)
        with self.lock:
            self.buf += data
            if "\n" in self.buf:
                lines, self.buf = self.buf.rsplit("\n", 1)
                with open(self.path, "a") as f:
                    f.write(lines + "\n")
        return len(data)

    def flush(self):
        self.stream.flush()

    def isatty(self):
        return False


def setup_logging(base_dir: str = "./logs", run_name: str = "run", role: str = "driver", rank: int = 0,
                  debug_shards: bool = False, level=logging.INFO, tee_stdout: bool = False) -> str:
    ts = time.strftime("%Y%m%d_%H%M%S")
    task_dir = _STATE["dir"] or os.path.join(base_dir, f"{run_name}_{ts}")
    os.makedirs(task_dir, exist_ok=True)
    _STATE.update(dir=task_dir, role=role, rank=rank)
    root = logging.getLogger("gcore_b200")
    root.setLevel(logging.DEBUG)
    root.handlers.clear()
    root.addFilter(_Ctx())
    fmt = logging.Formatter(_FMT)
    sh = logging.StreamHandler(sys.stderr)
    sh.setLevel(level)
    sh.setFormatter(fmt)
    sh.addFilter(_Ctx())
    root.addHandler(sh)
    if rank == 0:
        fh = logging.FileHandler(os.path.join(task_dir, "training.log"))
        fh.setLevel(level)
        fh.setFormatter(fmt)
        fh.addFilter(_Ctx())
        root.addHandler(fh)
    if debug_shards:
        d = os.path.join(task_dir, "debug")
        os.makedirs(d, exist_ok=True)
        dh = logging.FileHandler(os.path.join(d, f"{role}_rank{rank}_pid{os.getpid()}.log"))
        dh.setLevel(logging.DEBUG)
        dh.setFormatter(fmt)
        dh.addFilter(_Ctx())
        root.addHandler(dh)
    if tee_stdout and rank == 0:
        sys.stdout = TeeStream(sys.stdout, os.path.join(task_dir, "stdout.log"))
    return task_dir


def get_logger(name: Optional[str] = None) -> logging.Logger:
    lg = logging.getLogger("gcore_b200" + (("." + name) if name else ""))
    if not logging.getLogger("gcore_b200").handlers:
        logging.getLogger("gcore_b200").addHandler(logging.NullHandler())
    return lg


def mark_ppo_step(engine_log_path: str, step: int, begin: bool):
    """Step markers in the rollout-engine log, like the reference's ``ppo_step`` begin / end lines."""
    with open(engine_log_path, "a") as f:
        f.write(f"===== ppo_step {step} {'begin' if begin else 'end'} {time.time():.3f} =====\n")
