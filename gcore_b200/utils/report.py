"""Metric reporting on the last rank: jsonl always available, TensorBoard / wandb when importable and requested
(gpatch_v4/utils/report_utils.py:8-248).  Keys ending in ``_histogram`` are logged as histograms; an optional map
translates metric names to verl's vocabulary."""
from __future__ import annotations

import json
import os
import time
from typing import Dict, Optional

VERL_NAME_MAP = {
    "rollout-rewards/mean": "critic/rewards/mean", "ppo-metrics/pg_loss": "actor/pg_loss",
    "ppo-metrics/clipfrac": "actor/pg_clipfrac", "ppo-metrics/kl_to_ref": "actor/kl_loss",
    "policy/grad_norm": "actor/grad_norm", "policy/lr": "actor/lr", "policy/entropy": "actor/entropy",
    "rollout-metrics/response_length": "response_length/mean", "time_perf/step": "timing_s/step",
    "time_perf/rollout": "timing_s/gen", "time_perf/train_step": "timing_s/update_actor",
}


class Reporter:
    def __init__(self, report_cfg, run_dir: str, enabled: bool = True):
        self.cfg, self.enabled = report_cfg, enabled
        self.run_dir = run_dir
        self.tb = self.wandb = None
        self.jsonl = None
        if not enabled:
            return
        os.makedirs(run_dir, exist_ok=True)
        self.jsonl = open(os.path.join(run_dir, "metrics.jsonl"), "a")
        if "tensorboard" in report_cfg.report_to:
            try:
                from torch.utils.tensorboard import SummaryWriter
                self.tb = SummaryWriter(os.path.join(run_dir, "tb"))
            except Exception:  # noqa: BLE001
                self.tb = None
        if "wandb" in report_cfg.report_to:
            try:
                import wandb
                os.environ.setdefault("WANDB_MODE", "offline")
                self.wandb = wandb.init(project=report_cfg.project, name=report_cfg.run_name, dir=run_dir)
            except Exception:  # noqa: BLE001
                self.wandb = None

    def log(self, metrics: Dict[str, float], step: int):
        if not self.enabled:
            return
        if self.cfg.use_verl_metric_names:
            metrics = {VERL_NAME_MAP.get(k, k): v for k, v in metrics.items()}
        scalars = {k: v for k, v in metrics.items() if not k.endswith("_histogram")}
        self.jsonl.write(json.dumps({"step": step, "time": time.time(), **{k: float(v) for k, v in scalars.items()}}) + "\n")
        self.jsonl.flush()
        if self.tb is not None:
            for k, v in scalars.items():
                self.tb.add_scalar(k, float(v), step)
            for k, v in metrics.items():
                if k.endswith("_histogram"):
                    self.tb.add_histogram(k, v, step)
        if self.wandb is not None:
            self.wandb.log(scalars, step=step)

    def close(self):
        if self.jsonl:
            self.jsonl.close()
        if self.tb:
            self.tb.close()
        if self.wandb:
            self.wandb.finish()


def reduce_metrics(metrics: Dict[str, float]) -> Dict[str, float]:
    """``_min`` / ``_max`` suffixes keep their semantics, everything else is averaged over a list of dicts or values."""
    out = {}
    for k, v in metrics.items():
        if isinstance(v, (list, tuple)):
            out[k] = min(v) if k.endswith("_min") else max(v) if k.endswith("_max") else sum(v) / max(len(v), 1)
        else:
            out[k] = v
    return out
