"""Shared entry-point plumbing: parse ``--config file.yaml key=value ...``, join the process group from the torchrun
environment, build the parallel state from ``policy.dist_config`` and hand a validated config object to a trainer."""
from __future__ import annotations

import argparse
import os
from typing import List, Tuple

import torch
import torch.distributed as dist

from ..configs.base import load_config
from ..core import parallel_state as ps
from ..utils.logging_utils import setup_logging


def parse_cli(argv: List[str] | None = None) -> Tuple[str | None, List[str]]:
    ap = argparse.ArgumentParser(add_help=True)
    ap.add_argument("--config", "-c", default=None, help="YAML file")
    ap.add_argument("overrides", nargs="*", help="dotted overrides: a.b=c, +a.b=c, ~a.b")
    ns = ap.parse_args(argv)
    return ns.config, ns.overrides


def init_runtime(config):
    d = config.policy.dist_config
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or "RANK" in os.environ:
        ps.init_distributed(None, d.torch_dist_timeout_minutes)
        ps.initialize_model_parallel(tp=d.tensor_model_parallel_size, pp=d.pipeline_model_parallel_size,
                                     cp=d.context_parallel_size, ep=d.expert_model_parallel_size,
                                     etp=d.expert_tensor_parallel_size if d.expert_model_parallel_size > 1 else None,
                                     timeout_minutes=d.torch_dist_timeout_minutes)
    if config.training.apply_deterministic_mode:
        ps.apply_deterministic_mode()
    ps.set_seed(config.training.seed)
    rank = dist.get_rank() if dist.is_initialized() else 0
    setup_logging(config.report.log_dir, config.report.run_name or "run", role="train", rank=rank,
                  debug_shards=config.report.debug_log_shards)
    return rank


def finalize():
    from ..checkpoint.torch_dist import wait_for_async_save
    wait_for_async_save()   # an asynchronous save still in flight is completed and published before the job ends
    if dist.is_initialized():
        dist.barrier(group=ps.get_world_group())
        dist.destroy_process_group()


def load(cls, argv=None):
    path, overrides = parse_cli(argv)
    return load_config(cls, path, overrides)
