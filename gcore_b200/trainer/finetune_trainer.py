"""SFT / pre-training loop on one SPMD rank (``FinetuneActor._train_loop``, gpatch_v4/actor/finetune_actor.py:393-528):
dataloader batches -> ``TrainingEngine.finetune_step`` -> metrics / MFU -> periodic torch_dist checkpoint with dataloader
state; resumes automatically from the newest checkpoint; stamps a heartbeat and honours host-side fault injection at
every step boundary."""
from __future__ import annotations

import gc
import math
import os
import time
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..checkpoint.torch_dist import load_checkpoint, read_latest_step, save_checkpoint, wait_for_async_save
from ..configs.base import import_from_path
from ..core import parallel_state as ps
from ..data.datasets import default_dataset_fn
from ..engine import get_training_engine
from ..engine.train_engine import TrainingEngine
from ..orches.failure import FaultInjector, Heartbeat
from ..utils.flops_counter import mfu, train_flops
from ..utils.logging_utils import get_logger
from ..utils.report import Reporter
from ..utils.timers import Timers


class FinetuneTrainer:
    def __init__(self, config, model_cfg=None, tokenizer=None, dataset_fn=None):
        self.cfg, self.tokenizer, self.dataset_fn = config, tokenizer, dataset_fn
        t = config.training
        self.engine = get_training_engine(config.policy, config.optimizer, t, None, model_cfg=model_cfg,
                                     total_steps=t.total_training_step)
        self.step = 0
        self.log = get_logger("finetune")
        self.timers = Timers()
        rank = dist.get_rank() if dist.is_initialized() else 0
        self.rank = rank
        self.injector = FaultInjector(config.debug.fault_injection, rank, int(os.environ.get("GCORE_ATTEMPT", "0")))
        hb = os.environ.get("GCORE_HEARTBEAT_DIR") or config.monitor.heartbeat_dir
        self.heartbeat = Heartbeat(hb, rank) if hb else None
        self.reporter: Optional[Reporter] = None
        self.history = []

    def setup(self):
        cfg = self.cfg
        cfg.policy.without_ref = True
        self.engine.setup_model_and_get_optimizer()
        ck = cfg.checkpoint
        resume_from = ck.load_ckpt_path
        if cfg.training.auto_load_from_save_ckpt and ck.save_ckpt_path and read_latest_step(ck.save_ckpt_path) is not None:
            resume_from = ck.save_ckpt_path
        meta = None
        if resume_from and read_latest_step(resume_from) is not None:
            if hasattr(self.engine, "torch_opt"):
                self.step = self.engine.load_checkpoint(resume_from)
                self.engine.loaded_extra_state = {}
            else:
                self.step = load_checkpoint(self.engine, resume_from, load_optim=not ck.no_load_optim,
                                            load_rng=not ck.no_load_rng)
            meta = {"consumed_batches": self.engine.loaded_extra_state.get("consumed_batches", self.step),
                    "resume_step": self.step}
            self.log.info(f"resumed from {resume_from} at step {self.step}")
        fn = self.dataset_fn or default_dataset_fn
        if cfg.data.py_path:
            fn = import_from_path(cfg.data.py_path, cfg.data.fn_name or "build_dataset")
        dp_rank, dp_size = ps.get_data_parallel_rank(), ps.get_data_parallel_world_size()
        self.data = fn(cfg, self.tokenizer, dp_rank, dp_size, meta)
        self.loader_iter = iter(self.data["train_dataloader"])
        t = cfg.training
        self.total_steps = t.exit_step or t.total_training_step
        if not t.total_training_step:
            # no explicit length: training.num_train_epoches passes over this rank's share of the data
            # (gpatch_v4/actor/pretrain_actor.py:66); the learning-rate schedule decays over the same span
            s = self.data["train_sampler"]
            per_epoch = max(getattr(s, "per_rank", len(self.data["train_dataloader"])) //
                            max(t.train_gbs // max(dp_size, 1), 1), 1)
            span = int(math.ceil(per_epoch * max(t.num_train_epoches, 1)))
            self.total_steps = self.total_steps or span
            if self.engine.optimizer is not None and self.engine.optimizer.total_steps is None:
                self.engine.optimizer.total_steps = span
        if ps.is_last_rank():
            self.reporter = Reporter(cfg.report, os.path.join(cfg.report.log_dir, cfg.report.run_name or "finetune"))
        return self

    def _next_batch(self):
        try:
            return next(self.loader_iter)
        except StopIteration:
            s = self.data["train_sampler"]
            s.set_epoch(getattr(s, "epoch", 0) + 1)
            self.loader_iter = iter(self.data["train_dataloader"])
            return next(self.loader_iter)

    @staticmethod
    def _to_samples(batch) -> list:
        out = []
        for toks, labels, pl in zip(batch["tokens"], batch["labels"], batch["prompt_lengths"]):
            m = torch.zeros(toks.numel(), dtype=torch.float32)
            m[:-1] = (labels[1:] != -100).float()
            out.append({"tokens": toks, "loss_mask": m, "prompt_length": int(pl)})
        return out

    def train_one_step(self) -> Dict[str, float]:
        if getattr(self, "profiler", None) is None:
            from ..utils.profiler import StepProfiler
            pc = self.cfg.report.profile
            self.profiler = StepProfiler(pc, self.rank, pc.export_dir or os.path.join(self.cfg.report.log_dir or ".",
                                                                                      "profile"))
        step_id = self.step
        self.profiler.step_begin(step_id)
        self.injector.at_step(self.step)
        self.timers.start("train_step")
        samples = self._to_samples(self._next_batch())
        if self.cfg.policy.balance_dp_seqlen and ps.get_data_parallel_world_size() > 1:
            # the loss is normalised by the global token count, so samples may change ranks freely
            # (gpatch_v4/actor/finetune_actor.py "[DP balance]", core/dp_balancing.py:369)
            from ..core.dp_balancing import rebalance_across_dp_ranks
            samples, _ = rebalance_across_dp_ranks(samples, ps.get_data_parallel_group())
        m = self.engine.finetune_step(samples)
        dt = self.timers.stop("train_step")
        self.step += 1
        m["time_perf/train_step"] = dt
        if self.cfg.training.calc_mfu_freq and self.step % self.cfg.training.calc_mfu_freq == 0:
            world = dist.get_world_size() if dist.is_initialized() else 1
            fl = train_flops(self.engine.model_cfg, [len(s["tokens"]) for s in samples],
                             self.cfg.policy.recompute == "full") * ps.get_data_parallel_world_size()
            m["time_perf/mfu"] = mfu(fl, dt, world)
        if self.heartbeat:
            self.heartbeat.stamp(self.step)
        if self.reporter:
            self.reporter.log(m, self.step)
        summ = self.profiler.step_end(step_id)
        if summ:
            m.update({f"profile/{k}": v for k, v in summ.items()})
        self.history.append(m)
        return m

    def save(self):
        ck = self.cfg.checkpoint
        if not ck.save_ckpt_path:
            return None
        if hasattr(self.engine, "torch_opt"):   # ZeRO-3 engine: torch.distributed.checkpoint of the sharded state
            return self.engine.save_checkpoint(ck.save_ckpt_path, self.step)
        return save_checkpoint(self.engine, ck.save_ckpt_path, self.step, extra_state={"consumed_batches": self.step},
                               save_optim=not ck.no_save_optim, save_total_limit=ck.save_total_limit,
                               save_retain_interval=ck.save_retain_interval, async_save=ck.async_save)

    def train_loop(self):
        t = self.cfg.training
        total = self.total_steps or 0
        if t.manual_gc:
            # the collector runs between steps only, so that no rank stalls inside a step while the others wait in a
            # collective (gpatch_v4/actor/finetune_actor.py:346-357)
            gc.disable()
            gc.collect()
        while self.step < total:
            m = self.train_one_step()
            if t.manual_gc and self.step % max(t.manual_gc_interval, 1) == 0:
                gc.collect()
            if self.rank == 0 and self.step % max(self.cfg.report.log_interval, 1) == 0:
                self.log.info(f"step {self.step} lm_loss {m['lm_loss']:.4f} grad_norm {m['grad_norm']:.3f} "
                              f"{m['time_perf/train_step']:.3f}s")
            if t.save_interval and self.step % t.save_interval == 0:
                self.save()
        if t.manual_gc:
            gc.enable()
        if self.reporter:
            self.reporter.close()
        wait_for_async_save()
        return self.history
