"""RL driver loop on one SPMD rank: data -> rollout generator -> ``GrpoTrainer`` phases -> metrics, checkpoint / resume,
heartbeat, host-side fault injection.  Covers the synchronous trainer (``GrpoTrainer.launch`` + ``_train_loop``,
gpatch_v4/trainer/grpo_trainer.py:66-98, actor/grpo_train_actor.py:1466-1571) and the single-controller pipeline with
``rollout_max_staleness`` (gpatch_v4/trainer/grpo_single_ctrl_trainer.py:72-...)."""
from __future__ import annotations

import gc
import os
from typing import Dict, Iterator, List, Optional

import torch
import torch.distributed as dist

from ..checkpoint.torch_dist import load_checkpoint, read_latest_step, save_checkpoint, wait_for_async_save
from ..configs.base import import_from_path
from ..core import parallel_state as ps
from ..data.datasets import default_dataset_fn
from ..orches.failure import FaultInjector, Heartbeat
from ..rollout_generator.generators import StaleRolloutQueue, build_generator
from ..utils.logging_utils import get_logger
from ..utils.report import Reporter
from .grpo_trainer import GrpoTrainer


class RlLoop:
    def __init__(self, config, model_cfg=None, tokenizer=None, reward_fn=None, trainer=None):
        self.cfg, self.tokenizer = config, tokenizer
        self.trainer = trainer if trainer is not None else GrpoTrainer(config, model_cfg=model_cfg, reward_fn=reward_fn)
        self.log = get_logger("rl")
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.injector = FaultInjector(config.debug.fault_injection, self.rank, int(os.environ.get("GCORE_ATTEMPT", "0")))
        hb = os.environ.get("GCORE_HEARTBEAT_DIR") or config.monitor.heartbeat_dir
        self.heartbeat = Heartbeat(hb, self.rank) if hb else None
        self.reporter: Optional[Reporter] = None
        self.history: List[Dict[str, float]] = []
        self.consumed_batches = 0
        self.eval_history: List[Dict[str, float]] = []

    def setup(self):
        cfg, tr = self.cfg, self.trainer
        tr.setup()
        ck = cfg.checkpoint
        resume_from = ck.load_ckpt_path
        if cfg.training.auto_load_from_save_ckpt and ck.save_ckpt_path and read_latest_step(ck.save_ckpt_path) is not None:
            resume_from = ck.save_ckpt_path
        meta = None
        if resume_from and read_latest_step(resume_from) is not None:
            step = load_checkpoint(tr.policy, resume_from, load_optim=not ck.no_load_optim)
            tr.ppo_step = step
            extra = tr.policy.loaded_extra_state
            self.consumed_batches = extra.get("consumed_batches", step)
            meta = {"consumed_batches": self.consumed_batches, "resume_step": step}
            self.log.info(f"resumed RL job from {resume_from} at ppo step {step}")
        fn = default_dataset_fn
        if cfg.data.py_path:
            fn = import_from_path(cfg.data.py_path, cfg.data.fn_name or "build_dataset")
        self.data = fn(cfg, self.tokenizer, ps.get_data_parallel_rank(), ps.get_data_parallel_world_size(), meta)
        self.prompt_iter = self._prompts()
        self.generator = build_generator(tr, cfg)
        if meta and "rollout_generator" in tr.policy.loaded_extra_state:
            self.generator.load_state_dict(tr.policy.loaded_extra_state["rollout_generator"])
        self.queue = StaleRolloutQueue(cfg.training.rollout_max_staleness)
        if ps.is_last_rank():
            self.reporter = Reporter(cfg.report, os.path.join(cfg.report.log_dir, cfg.report.run_name or "rl"))
        return self

    def _prompts(self) -> Iterator[list]:
        while True:
            for batch in self.data["train_dataloader"]:
                self.consumed_batches += 1
                yield [p["prompt_token_ids"] for p in batch["prompt_token_ids"]]
            s = self.data["train_sampler"]
            s.set_epoch(getattr(s, "epoch", 0) + 1)

    def one_step(self) -> Dict[str, float]:
        cfg, tr = self.cfg, self.trainer
        if getattr(self, "profiler", None) is None:
            from ..utils.profiler import StepProfiler
            self.profiler = StepProfiler(cfg.report.profile, self.rank,
                                         cfg.report.profile.export_dir or os.path.join(cfg.report.log_dir or ".", "profile"))
        step_id = tr.ppo_step
        self.profiler.step_begin(step_id)
        self.injector.at_step(tr.ppo_step)
        tm = tr.timers
        tm.start("step")
        tm.start("rollout")
        while not self.queue.primed():
            self.queue.push(self.generator(self.prompt_iter, tr.ppo_step), tr.ppo_step)
        samples = self.queue.pop()
        tm.stop("rollout")
        metrics = tr.train_on_samples(samples)
        metrics["time_perf/rollout"] = tm.last("rollout")
        metrics["time_perf/step"] = tm.stop("step")
        metrics["rollout-metrics/weight_staleness"] = float(tr.ppo_step - 1 - samples[0].get("weight_version", tr.ppo_step - 1))
        if self.heartbeat:
            self.heartbeat.stamp(tr.ppo_step)
        if self.reporter:
            self.reporter.log(metrics, tr.ppo_step)
        summ = self.profiler.step_end(step_id)
        if summ:
            metrics.update({f"profile/{k}": v for k, v in summ.items()})
        self.history.append(metrics)
        return metrics

    def evaluate(self) -> Dict[str, float]:
        """Held-out evaluation with the current weights (``data.eval_data_path``; every ``training.eval_interval``
        steps from ``run``): ``task.eval.repeat_n`` samples per prompt (default ``sampling_repeat_n``) drawn with
        the sampler's ``eval_generate_params`` on top of the training sampling parameters, scored by the job's
        reward function; mean reward, pass@k and response length over the data-parallel ranks
        (the in-training evaluation of gpatch_v4/actor/grpo_train_actor.py; runner in evaluate/runner.py)."""
        dl = self.data.get("eval_dataloader")
        if dl is None:
            return {}
        from ..evaluate.runner import EvaluateRunner
        tr = self.trainer
        ev = dict((self.cfg.task or {}).get("eval", {}) or {})
        ie = self.cfg.sampler.infer_engine_configs[0]
        names = {"max_tokens": "max_new_tokens", "generate_max_tokens": "max_new_tokens"}
        override = {names.get(k, k): v for k, v in dict(ie.eval_generate_params or {}).items()
                    if names.get(k, k) in tr.sampling.__dict__}
        t = self.cfg.training
        n = int(ev.get("repeat_n", t.eval_sampling_repeat_n or t.sampling_repeat_n))
        runner = EvaluateRunner(lambda p: tr.rollout(p, n=n, sampling=override),
                                lambda s: [float(x["rewards"]) for x in tr.score(s)], n,
                                ks=tuple(ev.get("ks", (1,))), threshold=float(ev.get("threshold", 0.5)),
                                dp_group=ps.get_data_parallel_group())
        prompts, limit = [], int(ev.get("batches", 0))
        for i, batch in enumerate(dl):
            if limit and i >= limit:
                break
            prompts += [p["prompt_token_ids"] for p in batch["prompt_token_ids"]]
        metrics = runner.run(prompts)
        if self.reporter:
            self.reporter.log(metrics, tr.ppo_step)
        self.eval_history.append({"step": tr.ppo_step, **metrics})
        return metrics

    def save(self):
        ck = self.cfg.checkpoint
        if not ck.save_ckpt_path:
            return None
        extra = {"consumed_batches": self.consumed_batches, "rollout_generator": self.generator.state_dict()}
        return save_checkpoint(self.trainer.policy, ck.save_ckpt_path, self.trainer.ppo_step, extra_state=extra,
                               save_optim=not ck.no_save_optim, save_total_limit=ck.save_total_limit,
                               save_retain_interval=ck.save_retain_interval, async_save=ck.async_save)

    def run(self):
        t = self.cfg.training
        total = t.exit_step or t.total_ppo_step or 0
        tracer = None
        if self.cfg.debug.trace_python_calls:
            from ..utils.python_call_tracer import PythonCallTracer
            roots = self.cfg.debug.trace_roots or [os.path.dirname(os.path.dirname(os.path.abspath(__file__)))]
            out = os.path.join(self.cfg.report.log_dir or ".", f"python_calls_rank{self.rank}.log")
            os.makedirs(os.path.dirname(out), exist_ok=True)
            tracer = PythonCallTracer(roots, out)
            tracer.__enter__()
        if t.manual_gc:
            gc.disable()
            gc.collect()
        if t.eval_before_train and t.eval_interval and self.trainer.ppo_step < total:
            self.evaluate()
        while self.trainer.ppo_step < total:
            m = self.one_step()
            if t.manual_gc and self.trainer.ppo_step % max(t.manual_gc_interval, 1) == 0:
                gc.collect()
            if self.rank == 0:
                self.log.info(f"ppo_step {self.trainer.ppo_step} reward {m['rollout-rewards/mean']:.4f} "
                              f"step {m['time_perf/step']:.2f}s")
            if t.eval_interval and self.trainer.ppo_step % t.eval_interval == 0:
                em = self.evaluate()
                if em and self.rank == 0:
                    self.log.info(f"ppo_step {self.trainer.ppo_step} " + " ".join(f"{k}={v:.4f}" for k, v in em.items()))
            if t.save_interval and self.trainer.ppo_step % t.save_interval == 0:
                self.save()
        if t.manual_gc:
            gc.enable()
        if tracer is not None:
            tracer.__exit__(None, None, None)
        if self.reporter:
            self.reporter.close()
        wait_for_async_save()
        return self.history
