"""Synchronous GRPO / PPO step on one SPMD rank: rollout -> rewards -> prev / ref log-probs -> advantages -> policy
(and critic) update -> weight hand-over to the rollout engine.

Same phase structure and metric families as ``GrpoTrainActor.train_one_ppo_step`` (gpatch_v4/actor/
grpo_train_actor.py:1231-1434), without the Ray actor boundary: trainer and rollout engine share the process and,
when their tensor-parallel layouts match, the parameter storage.  The GPU is time-shared explicitly: the KV cache
exists only during rollout, the fp32 gradient buffers only during the update.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..configs.base import import_from_path
from ..configs.config import RlConfig
from ..core import parallel_state as ps
from ..core.advantage import compute_advantages
from ..core.packing import response_mask
from ..engine import get_training_engine
from ..engine.train_engine import TrainingEngine
from ..rollout.engine import InferEngine, RolloutWeights, SamplingParams
from ..utils.timers import Timers


def synthetic_reward(samples: Sequence[dict], **_) -> torch.Tensor:
    """Rule reward of the benchmark recipe: 1.0 when the response contains token id
    ``(sum(prompt) mod 150000) + 100``, else 0.0."""
    out = []
    for s in samples:
        p = int(s["prompt_length"])
        toks = s["tokens"]
        target = (int(toks[:p].sum()) % 150000) + 100
        out.append(1.0 if bool((toks[p:] == target).any()) else 0.0)
    return torch.tensor(out, dtype=torch.float32)


class GrpoTrainer:
    def __init__(self, config: RlConfig, model_cfg=None, reward_fn: Optional[Callable] = None,
                 prompt_source: Optional[Callable] = None, vision_cfg=None, image_token_id: Optional[int] = None,
                 teacher_model_cfg=None):
        self.cfg = config
        self.timers = Timers()
        self.reward_fn = reward_fn or self._load_reward_fn() or synthetic_reward
        self.prompt_source = prompt_source
        t = config.training
        self.policy = get_training_engine(config.policy, config.optimizer, t, config.ppo, model_cfg=model_cfg,
                                     total_steps=t.total_ppo_step, vision_cfg=vision_cfg,
                                     image_token_id=image_token_id)
        self.critic: Optional[TrainingEngine] = None
        self.teacher: Optional[TrainingEngine] = None
        self.teacher_model_cfg = teacher_model_cfg
        self.engine: Optional[InferEngine] = None
        self.ppo_step = 0
        self.last_metrics: Dict[str, float] = {}
        self.advantage_fn = None
        if config.ppo.advantage_py_path:
            self.advantage_fn = import_from_path(config.ppo.advantage_py_path,
                                                 config.ppo.advantage_fn_name or "advantage_fn")
        # optional user step after the advantages exist: fn(samples, ppo_cfg, dp_group) -> samples or
        # (samples, metrics); the hook point of gpatch_v4/actor/mixin.py:821-832
        self.post_advantage_fn = None
        if config.ppo.post_advantage_py_path:
            self.post_advantage_fn = import_from_path(config.ppo.post_advantage_py_path,
                                                      config.ppo.post_advantage_fn_name or "post_advantage_fn")

    def _load_reward_fn(self):
        b = self.cfg.bt_rm
        if b.rule_py_path:
            return import_from_path(b.rule_py_path, b.rule_fn_name or "reward_fn")
        return None

    # ------------------------------------------------------------------ setup
    def setup(self):
        cfg = self.cfg
        self.policy.setup_model_and_get_optimizer()
        ie = cfg.sampler.infer_engine_configs[0]
        self.policy.temperature = ie.temperature
        if cfg.require_critic_model():
            self.critic = get_training_engine(cfg.critic, cfg.critic.optimizer, cfg.training, cfg.ppo,
                                         model_cfg=self.policy.model_cfg, role="critic", value_head=True)
            self.critic.setup_model_and_get_optimizer(with_ref=False)
        if cfg.teacher is not None:
            # on-policy distillation: a frozen teacher scores the student's rollouts (forward only, no optimizer;
            # gpatch_v4/trainer on-policy distill trainer + teacher client)
            cfg.teacher.without_optim = True
            self.teacher = get_training_engine(cfg.teacher, cfg.optimizer, cfg.training, cfg.ppo,
                                          model_cfg=self.teacher_model_cfg or self.policy.model_cfg, role="teacher")
            self.teacher.setup_model_and_get_optimizer(with_ref=False, seed=cfg.training.seed + 7919)
            if cfg.teacher.hf_model_path:
                from ..checkpoint.hf import load_hf
                load_hf(self.teacher, cfg.teacher.hf_model_path)
        if cfg.debug.check_a2a_legality:
            from ..parallel import ep as ep_mod
            ep_mod.CHECK_A2A["enabled"] = True
        model = self.policy.model
        # with LoRA only the adapted projections differ from the frozen base: the rollout engine then owns copies of
        # those tensors (base + delta, rewritten at every resync) and shares the storage of all the others
        self.lora = bool(cfg.policy.lora.enabled)
        share = cfg.policy.share_rollout_weights
        # a separate rollout copy that exists only while the engine serves (rebuilt by every weight update, dropped
        # after every rollout): the memory behaviour of the reference's colocated engines in sleep mode
        self.release_rollout_weights = bool(not share and getattr(cfg.policy, "release_rollout_weights", False))
        weights = RolloutWeights.from_model(model, clone=not share)
        if self.lora and share:
            from ..rollout.weight_sync import detach_lora_targets
            detach_lora_targets(self.policy, weights)
        t = cfg.training
        n_req = max(t.rollout_gbs // max(ps.get_data_parallel_world_size(), 1), 1) * t.sampling_repeat_n
        self.engine = InferEngine(
            self.policy.model_cfg, weights, tp_size=model.tp_size,
            tp_group=ps.get_tensor_model_parallel_group() if model.tp_size > 1 else None,
            max_running_requests=ie.max_running_requests or n_req,
            max_model_len=ie.max_model_len or (cfg.data.max_prompt_length + ie.generate_max_tokens),
            kv_block_size=ie.kv_block_size, num_kv_blocks=ie.num_kv_blocks,
            gpu_memory_utilization=ie.gpu_memory_utilization, max_prefill_tokens=ie.max_prefill_tokens,
            use_cuda_graph=not ie.disable_cuda_graph, device=self.policy.device)
        self.sampling = SamplingParams(temperature=ie.temperature, top_k=ie.top_k, top_p=ie.top_p, min_p=ie.min_p, repetition_penalty=ie.repetition_penalty,
                                       max_new_tokens=ie.generate_max_tokens, seed=ie.seed,
                                       stop_token_ids=tuple(ie.generate_params.get("stop_token_ids", ())))
        # fp8 serving: asked for by the engine config, and implied by an fp8 policy so that trainer and rollout
        # compute the same quantised products
        self.serve_fp8 = bool(getattr(ie, "fp8_weights", False) or cfg.policy.fp8)
        if self.serve_fp8:
            self.engine.quantize_weights_fp8()
        self.engine.owns_weights = not share
        if getattr(cfg.policy, "offload_ref_model", False):
            self.policy.offload_ref_model()
        # gradient buffers are only needed inside the update phase
        self.policy.release_grad_buffers()
        return self

    # ------------------------------------------------------------------ phases
    def rollout(self, prompts: Sequence, n: Optional[int] = None, sampling: Optional[dict] = None) -> List[dict]:
        """``prompts``: token-id lists, or for a vision-language policy dicts with ``tokens``, ``pixel_patches`` and
        ``image_grid`` (the vision tower runs here, once per prompt; the engine only sees feature rows).  ``n`` samples
        per prompt (default ``training.sampling_repeat_n``); ``sampling`` overrides fields of the job's sampling
        parameters for this call (evaluation passes its own temperature / length)."""
        t = self.cfg.training
        n = int(n or t.sampling_repeat_n)
        release_pg = (self.cfg.policy.offload_process_group and dist.is_initialized() and ps.get_state().initialized
                      and self.engine.tp == 1 and self.engine.ep_group is None)
        if release_pg:   # the trainer's communicators hold device memory the KV cache can use
            self.policy.offload_process_groups()
        self.engine.wake_up(("kv_cache",))
        sp = SamplingParams(**{**self.sampling.__dict__, **(sampling or {}),
                               "seed": self.sampling.seed + self.ppo_step * 1000003})
        images = [p if isinstance(p, dict) and "pixel_patches" in p else None for p in prompts]
        prompts = [list(p["tokens"]) if isinstance(p, dict) else p for p in prompts]
        vl_kw = {}
        if any(im is not None for im in images):
            model = self.policy.model
            assert hasattr(model, "vision"), "image prompts need a vision-language policy"
            embeds = []
            with torch.no_grad():
                for im in images:
                    if im is None:
                        embeds.append(None)
                        continue
                    g = im["image_grid"]
                    grids = [tuple(x) for x in (g if isinstance(g[0], (list, tuple)) else [g])]
                    patches = torch.as_tensor(im["pixel_patches"], dtype=torch.float32).to(self.policy.device)
                    embeds.append(model.vision(patches.to(next(model.vision.parameters()).dtype), grids))
            vl_kw = dict(image_embeds=embeds, image_token_id=model.image_token_id)
        from ..utils.logging_utils import redirect_engine_output
        with redirect_engine_output(self.ppo_step, enabled=bool(getattr(self.cfg.report, "redirect_engine_log", False))):
            reqs = self.engine.generate(prompts, sp, n=n, **vl_kw)
        self.engine.sleep(("kv_cache", "weights") if self.release_rollout_weights else ("kv_cache",))
        if release_pg:
            self.policy.reload_process_groups()
        samples = []
        dp_rank = ps.get_data_parallel_rank()
        for k, r in enumerate(reqs):
            toks = torch.tensor(r.prompt + r.out_tokens, dtype=torch.int64)
            P, S = len(r.prompt), len(r.prompt) + len(r.out_tokens)
            lp = torch.zeros(S, dtype=torch.float32)
            lp[P - 1:S - 1] = torch.tensor(r.out_logprobs, dtype=torch.float32)
            samples.append(dict(tokens=toks, prompt_length=P, sequence_length=S, rollout_log_probs=lp,
                                group_id=k // n, unique_id=(self.ppo_step, dp_rank, k),
                                mask=response_mask(P, S), finish_reason=r.finish_reason))
            im = images[k // n]
            if im is not None:  # the training passes re-run the vision tower on the same pixels
                samples[-1]["pixel_patches"], samples[-1]["image_grid"] = im["pixel_patches"], im["image_grid"]
        return samples

    def score(self, samples: List[dict]) -> List[dict]:
        out = self.reward_fn(samples)
        rewards, per_tok, extra = (out if isinstance(out, tuple) else (out, None, {}))
        rewards = torch.as_tensor(rewards, dtype=torch.float32).reshape(-1)
        for i, s in enumerate(samples):
            s["rewards"] = rewards[i]
            if per_tok is not None:
                s["per_token_rewards"] = per_tok[i]
        self._reward_extra = extra
        return samples

    def step(self, prompts: Optional[Sequence[Sequence[int]]] = None) -> Dict[str, float]:
        """One full PPO step; returns the metric dict (timers under ``time_perf/``)."""
        cfg, t, tm = self.cfg, self.cfg.training, self.timers
        if prompts is None:
            prompts = self.prompt_source(self.ppo_step)
        tm.start("step")
        tm.start("rollout")
        samples = self.rollout(prompts)
        tm.stop("rollout")
        tm.start("reward")
        samples = self.score(samples)
        tm.stop("reward")
        metrics = self.train_on_samples(samples)
        tm.stop("step")
        for k in ("step", "rollout", "reward"):
            metrics[f"time_perf/{k}"] = tm.last(k)
        return metrics

    def train_on_samples(self, samples: List[dict]) -> Dict[str, float]:
        """Everything after rollout + reward: prev / ref log-probs, advantages, policy (and critic) update, weight
        hand-over.  ``samples`` may come from an earlier weight version (stale rollouts)."""
        cfg, t, tm = self.cfg, self.cfg.training, self.timers
        if cfg.debug.check_rollout_batches:
            from ..gdebug import check_rollout_batches
            check_rollout_batches(samples)
        tm.start("compute_logps")
        need_ref = not cfg.policy.without_ref and cfg.ppo.grpo_kl_loss_beta != 0
        swap_ref = need_ref and getattr(cfg.policy, "offload_ref_model", False)
        if swap_ref:
            # the frozen reference policy lives in pinned host memory between its forward passes; its upload runs on
            # a side stream under the old-policy pass (gpatch_v4/training_backend/megatron_backend/mcore_engine.py:
            # 373-531 swaps policy and reference around the two passes)
            self.policy.prefetch_ref_model()
        if not cfg.ppo.skip_prev_logps:
            self.policy.compute_log_probs(samples, use_ref=False)
        if need_ref:
            if swap_ref:
                self.policy.onload_ref_model()
            self.policy.compute_log_probs(samples, use_ref=True)
            if swap_ref:
                self.policy.offload_ref_model()
        if self.critic is not None:
            self.critic.compute_values(samples)
        if self.teacher is not None:
            self.teacher.compute_log_probs(samples, use_ref=False, with_entropy=False, out_key="teacher_logprobs")
        tm.stop("compute_logps")
        tm.start("generate_ppo_data")
        samples = compute_advantages(samples, cfg.ppo, ps.get_data_parallel_group(), self.advantage_fn)
        post_metrics: Dict[str, float] = {}
        if self.post_advantage_fn is not None:
            res = self.post_advantage_fn(samples, cfg.ppo, ps.get_data_parallel_group())
            samples, post_metrics = res if isinstance(res, tuple) else (res, {})
        tm.stop("generate_ppo_data")
        tm.start("train_step")
        metrics: Dict[str, float] = {k: float(v) for k, v in post_metrics.items()}
        if cfg.policy.balance_dp_seqlen and ps.get_data_parallel_world_size() > 1:
            # even out the token counts of the data-parallel ranks before the update: losses are normalised by global
            # counts, so which rank trains which sample does not change the gradient
            # (gpatch_v4/actor/grpo_train_actor.py:1344-1353, core/dp_balancing.py:369)
            from ..core.dp_balancing import rebalance_across_dp_ranks
            before = float(sum(s["sequence_length"] for s in samples))
            samples, _ = rebalance_across_dp_ranks(samples, ps.get_data_parallel_group())
            for s in samples:
                s.pop("_origin", None)
            metrics["rollout-metrics/dp_balance_tokens_before"] = before
            metrics["rollout-metrics/dp_balance_tokens_after"] = float(sum(s["sequence_length"] for s in samples))
        self.policy.allocate_grad_buffers()
        per_update = max(t.train_gbs // max(ps.get_data_parallel_world_size(), 1), 1)
        for _ in range(t.ppo_max_epochs_2):
            for s0 in range(0, len(samples), per_update):
                if self.critic is not None:
                    metrics.update(self.critic.rl_train_value(samples[s0:s0 + per_update]))
                if self.critic is None or self.ppo_step >= cfg.ppo.critic_model_warmup_steps:
                    metrics.update(self.policy.rl_train_actor(samples[s0:s0 + per_update]))
        self.policy.release_grad_buffers()
        tm.stop("train_step")
        tm.start("update_weights")
        self.update_weights()
        tm.stop("update_weights")
        metrics.update(self._rollout_metrics(samples))
        for k in ("compute_logps", "generate_ppo_data", "train_step", "update_weights"):
            metrics[f"time_perf/{k}"] = tm.last(k)
        self._maybe_dump_tokens(samples)
        self.ppo_step += 1
        self.last_metrics = metrics
        self.last_samples = samples
        return metrics

    def _maybe_dump_tokens(self, samples: List[dict]):
        """Per-token dump of what was trained on (tokens, mask, trainer / reference / rollout log-probs, advantages,
        rewards), one jsonl file per step and rank, every ``training.ppo_dump_metrics_interval`` steps
        (the reference's offline per-token dumps: gpatch_v4/actor/grpo_train_actor.py:167-216)."""
        t = self.cfg.training
        every = getattr(t, "ppo_dump_metrics_interval", 0)
        if not every or self.ppo_step % every:
            return
        import json
        import os
        d = getattr(t, "ppo_dump_metrics_dir", None) or os.path.join(self.cfg.report.log_dir or ".", "token_dumps")
        os.makedirs(d, exist_ok=True)
        rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
        tok = getattr(self, "tokenizer", None)
        with open(os.path.join(d, f"step{self.ppo_step:07d}_rank{rank}.jsonl"), "w") as f:
            for s in samples:
                row = {"prompt_length": int(s["prompt_length"]), "group_id": int(s.get("group_id", 0)),
                       "reward": float(torch.as_tensor(s["rewards"]).sum())}
                for k in ("tokens", "mask", "logprobs", "ref_logprobs", "rollout_log_probs", "teacher_logprobs",
                          "advantages", "values"):
                    if k in s and s[k] is not None:
                        v = torch.as_tensor(s[k])
                        row[k] = v.tolist() if k == "tokens" else [round(float(x), 6) for x in v.tolist()]
                if tok is not None:
                    row["text"] = tok.decode(torch.as_tensor(s["tokens"]).tolist())
                f.write(json.dumps(row) + "\n")

    def update_weights(self):
        """Hands the updated weights to the rollout engine (zero-copy when storage is shared)."""
        if self.cfg.policy.share_rollout_weights:
            if self.lora:
                from ..rollout.weight_sync import sync_lora_deltas
                sync_lora_deltas(self.policy, self.engine)
            self.engine.update_weights(None)
        elif self.release_rollout_weights:
            self.engine.load_weights_from(self.policy.model, self.cfg.policy.sampler_client.update_weight_max_size_mb)
        else:
            from ..rollout.weight_sync import sync_weights
            sync_weights(self.policy, self.engine)
        if self.cfg.debug.debug_update_weight and not self.lora and not self.serve_fp8:
            from ..rollout.weight_sync import verify
            bad = verify(self.policy, self.engine)
            if bad:
                raise RuntimeError(f"rollout weights differ from the trainer's after the hand-over: {bad[:6]}")
        if self.serve_fp8:
            # the engine's dense projections are re-quantised (e4m3, 128x128 scales) from the weights just handed over
            self.engine.quantize_weights_fp8()

    def offload_model(self):
        """Trainable weights to pinned host memory (early-swap mode of the reference's ``OffloadManager``,
        gpatch_v4/actor/mixin.py:360-393).  A rollout engine that reads the trainer's storage drops its views first,
        so the device memory is really returned."""
        if self.cfg.policy.share_rollout_weights and self.engine is not None:
            self.engine.w = None
            self.engine._graphs.clear()
        self.policy.offload_model()

    def onload_model(self):
        self.policy.onload_model()
        if self.cfg.policy.share_rollout_weights and self.engine is not None:
            w = RolloutWeights.from_model(self.policy.model, clone=False)
            if self.lora:
                from ..rollout.weight_sync import detach_lora_targets
                detach_lora_targets(self.policy, w)
            self.engine.w = w
            self.engine._graphs.clear()
            self.update_weights()

    def _rollout_metrics(self, samples):
        r = torch.stack([torch.as_tensor(s["rewards"]).float().sum() for s in samples])
        resp = torch.tensor([float(s["sequence_length"] - s["prompt_length"]) for s in samples])
        tot = torch.tensor([r.sum(), float(len(samples)), resp.sum(), float(sum(s["sequence_length"] for s in samples)),
                            float(sum(1 for s in samples if s["finish_reason"] == "length"))])
        g = ps.get_data_parallel_group()
        if g is not None and dist.get_world_size(g) > 1:
            tt = tot.to(self.policy.device) if dist.get_backend(g) == "nccl" else tot
            dist.all_reduce(tt, group=g)
            tot = tt.cpu()
        n = max(float(tot[1]), 1.0)
        return {"rollout-rewards/mean": float(tot[0]) / n, "rollout-metrics/response_length": float(tot[2]) / n,
                "rollout-metrics/num_samples": n, "rollout-metrics/total_tokens": float(tot[3]),
                "rollout-metrics/response_tokens": float(tot[2]), "rollout-metrics/truncated_frac": float(tot[4]) / n}
