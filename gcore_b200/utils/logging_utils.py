"""Structured logging of a multi-process job.

Record format ``time - level - role= - rank= - pid= - node= - msg`` (the reference's, docs/source/logging.md:43-48;
gpatch_v4/utils/logging_utils.py:196-687).  Layout of a task directory ``<base>/<run>_<timestamp>/``:

* ``training.log``  - the aggregated log.  In the reference only the driver writes it and Ray forwards the actors'
  console output; here every rank appends its INFO-and-above records itself with one ``O_APPEND`` write per record,
  which the kernel serialises for writes of this size, so lines of different ranks never interleave and no forwarding
  process is needed.  ``aggregate_ranks`` limits which ranks take part (default: all; ``[0]`` = driver only).
* ``debug/<role>_rank<r>_pid<p>.log``  - DEBUG shard of one process (``debug_shards``).
* ``infer_engine_log/<role>_rank<r>.log`` - whatever native code and libraries print while the rollout engine runs:
  ``redirect_engine_output`` moves file descriptors 1 and 2 there (``dup2``, so C / CUDA / NCCL prints are caught
  too) between ``ppo_step N begin`` / ``end`` markers and restores them afterwards.
* ``stdout.log`` - ``tee_stdout`` mirrors Python-level stdout of rank 0.

The task directory is agreed on by rank 0 and shared through the environment (``GCORE_TASK_DIR``) so that every rank
of a launch lands in the same one.
"""
from __future__ import annotations

import contextlib
import logging
import os
import socket
import sys
import threading
import time
from typing import Iterable, Optional

_FMT = "%(asctime)s - %(levelname)s - role=%(role)s - rank=%(rank)s - pid=%(process)d - node=%(node)s - %(message)s"
_STATE = {"dir": None, "role": "driver", "rank": 0}
ROOT = "gcore_b200"


class _Ctx(logging.Filter):
    def filter(self, record):
        record.role = _STATE["role"]
        record.rank = _STATE["rank"]
        record.node = socket.gethostname()
        return True


class AtomicAppendHandler(logging.Handler):
    """One ``os.write`` on an ``O_APPEND`` descriptor per record: concurrent writers (other ranks, other threads) never
    split each other's lines."""

    def __init__(self, path: str, level=logging.INFO):
        super().__init__(level)
        self.path = path
        self.fd = os.open(path, os.O_WRONLY | os.O_APPEND | os.O_CREAT, 0o644)

    def emit(self, record):
        try:
            os.write(self.fd, (self.format(record) + "\n").encode("utf-8", "replace"))
        except Exception:  # noqa: BLE001
            self.handleError(record)

    def close(self):
        try:
            os.close(self.fd)
        except OSError:
            pass
        super().close()


class TeeStream:
    """Writes to the wrapped stream and appends whole lines to a file (one atomic append per flush of lines)."""

    def __init__(self, stream, path):
        self.stream, self.path = stream, path
        self.lock = threading.Lock()
        self.buf = ""
        self.fd = os.open(path, os.O_WRONLY | os.O_APPEND | os.O_CREAT, 0o644)

    def write(self, data):
        self.stream.write(data)
        with self.lock:
            self.buf += data
            if "\n" in self.buf:
                lines, self.buf = self.buf.rsplit("\n", 1)
                os.write(self.fd, (lines + "\n").encode("utf-8", "replace"))
        return len(data)

    def flush(self):
        self.stream.flush()

    def isatty(self):
        return False


def task_dir() -> Optional[str]:
    return _STATE["dir"]


def setup_logging(base_dir: str = "./logs", run_name: str = "run", role: str = "driver", rank: int = 0,
                  debug_shards: bool = False, level=logging.INFO, tee_stdout: bool = False,
                  aggregate_ranks: Optional[Iterable[int]] = None) -> str:
    """Creates (or joins) the task directory and installs the handlers described in the module docstring."""
    d = _STATE["dir"] or os.environ.get("GCORE_TASK_DIR")
    if not d:
        d = os.path.join(base_dir or "./logs", f"{run_name}_{time.strftime('%Y%m%d_%H%M%S')}")
        os.environ["GCORE_TASK_DIR"] = d   # child processes of this launch join the same directory
    os.makedirs(d, exist_ok=True)
    _STATE.update(dir=d, role=role, rank=rank)
    root = logging.getLogger(ROOT)
    root.setLevel(logging.DEBUG)
    for h in list(root.handlers):
        root.removeHandler(h)
        h.close()
    fmt = logging.Formatter(_FMT)

    def add(h, lvl):
        h.setLevel(lvl)
        h.setFormatter(fmt)
        h.addFilter(_Ctx())
        root.addHandler(h)

    add(logging.StreamHandler(sys.stderr), level if rank == 0 else max(level, logging.WARNING))
    if aggregate_ranks is None or rank in set(aggregate_ranks):
        add(AtomicAppendHandler(os.path.join(d, "training.log")), level)
    if debug_shards:
        dd = os.path.join(d, "debug")
        os.makedirs(dd, exist_ok=True)
        add(AtomicAppendHandler(os.path.join(dd, f"{role}_rank{rank}_pid{os.getpid()}.log")), logging.DEBUG)
    if tee_stdout and rank == 0 and not isinstance(sys.stdout, TeeStream):
        sys.stdout = TeeStream(sys.stdout, os.path.join(d, "stdout.log"))
    return d


def get_logger(name: Optional[str] = None) -> logging.Logger:
    lg = logging.getLogger(ROOT + (("." + name) if name else ""))
    if not logging.getLogger(ROOT).handlers:
        logging.getLogger(ROOT).addHandler(logging.NullHandler())
    return lg


def engine_log_path(role: str = "sampler", rank: Optional[int] = None) -> str:
    d = os.path.join(_STATE["dir"] or ".", "infer_engine_log")
    os.makedirs(d, exist_ok=True)
    return os.path.join(d, f"{role}_rank{_STATE['rank'] if rank is None else rank}.log")


def mark_ppo_step(path: str, step: int, begin: bool):
    """Step markers in the rollout-engine log, like the reference's ``ppo_step`` begin / end lines."""
    fd = os.open(path, os.O_WRONLY | os.O_APPEND | os.O_CREAT, 0o644)
    try:
        os.write(fd, f"===== ppo_step {step} {'begin' if begin else 'end'} {time.time():.3f} =====\n".encode())
    finally:
        os.close(fd)


@contextlib.contextmanager
def redirect_engine_output(step: int, role: str = "sampler", path: Optional[str] = None, enabled: bool = True):
    """File descriptors 1 and 2 point at the engine log for the duration (prints from native code included), between
    ``ppo_step`` markers; Python's ``sys.stdout`` / ``sys.stderr`` objects are flushed on both edges."""
    if not enabled:
        yield None
        return
    path = path or engine_log_path(role)
    mark_ppo_step(path, step, True)
    sys.stdout.flush()
    sys.stderr.flush()
    saved = (os.dup(1), os.dup(2))
    fd = os.open(path, os.O_WRONLY | os.O_APPEND | os.O_CREAT, 0o644)
    try:
        os.dup2(fd, 1)
        os.dup2(fd, 2)
        yield path
    finally:
        sys.stdout.flush()
        sys.stderr.flush()
        os.dup2(saved[0], 1)
        os.dup2(saved[1], 2)
        for x in (*saved, fd):
            os.close(x)
        mark_ppo_step(path, step, False)


def log_memory_usage(tag: str, logger: Optional[logging.Logger] = None):
    """One line with the device allocator's numbers (the snapshots the reference takes around every offload / onload,
    gpatch_v4/training_backend/megatron_backend/mcore_swap_impl.py:36,98)."""
    import torch
    lg = logger or get_logger("memory")
    if torch.cuda.is_available():
        free, total = torch.cuda.mem_get_info()
        lg.info(f"[mem] {tag}: allocated {torch.cuda.memory_allocated() / 2**30:.2f} GiB, reserved "
                f"{torch.cuda.memory_reserved() / 2**30:.2f} GiB, free {free / 2**30:.2f} of {total / 2**30:.2f} GiB")
    else:
        lg.info(f"[mem] {tag}: no device")
