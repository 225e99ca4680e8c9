"""Runtime bring-up of the image-generation entry points: data parallel only (one process per GPU, gradients averaged
with one all-reduce per optimizer step)."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..core import parallel_state as ps
from ..utils.logging_utils import setup_logging


def init_t2i_runtime(config) -> int:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or "RANK" in os.environ:
        ps.init_distributed(None)
    ps.set_seed(config.training.seed)
    rank = dist.get_rank() if dist.is_initialized() else 0
    setup_logging(config.report.log_dir, config.report.run_name or "t2i", role="train", rank=rank)
    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    return rank


def finalize_t2i():
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
