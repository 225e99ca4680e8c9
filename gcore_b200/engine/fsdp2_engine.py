"""ZeRO-3 training engine: parameters, gradients and optimizer state are sharded over the data-parallel group with
PyTorch FSDP2 (``fully_shard`` per transformer layer, then the root), as in the reference's FSDP2 backend
(gpatch_v4/training_backend/fsdp2_backend/fsdp2_engine_lm.py:66, mixin.py:116-493, optimizer.py:30-63,
checkpoint.py:118-247): bf16 compute with fp32 gradient reduction, AdamW or Muon, DCP checkpoints.

It reuses the packing, log-prob and loss code of ``TrainingEngine`` (same public methods: ``finetune_step``,
``compute_log_probs``, ``rl_train_actor``); only model wrapping, the optimizer and the end-of-step differ.  The hot
kernels underneath are the same hand-written ones: FSDP2 hands the layers ordinary unsharded tensors while they run.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from ..core import parallel_state as ps
from ..parallel.distributed_optimizer import lr_at_step
from .train_engine import TrainingEngine


class _GradShim:
    """What ``TrainingEngine`` expects of its DDP wrapper, on top of plain autograd gradients."""

    def __init__(self, model):
        self.model = model
        self.buffers = []

    def zero_grad_buffer(self):
        for p in self.model.parameters():
            p.grad = None

    def allocate_grads(self):
        pass

    def release_grads(self):
        self.zero_grad_buffer()


class _OptShim:
    """The attributes of ``DistributedOptimizer`` that trainers read; ``total_steps`` feeds the learning-rate decay."""

    def __init__(self, engine=None):
        self.last_grad_norm = torch.zeros(())
        self.step_count = 0
        self._engine = engine

    @property
    def total_steps(self):
        return self._engine.total_steps if self._engine is not None else None

    @total_steps.setter
    def total_steps(self, v):
        if self._engine is not None:
            self._engine.total_steps = v


class Fsdp2Engine(TrainingEngine):
    def setup_model_and_get_optimizer(self, seed: Optional[int] = None, with_ref: Optional[bool] = None):
        from torch.distributed.device_mesh import init_device_mesh
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
        assert ps.get_tensor_model_parallel_world_size() == 1 and ps.get_pipeline_model_parallel_world_size() == 1, \
            "the FSDP2 engine shards over data parallel ranks only"
        with_ref = (not self.policy_cfg.without_ref) if with_ref is None else with_ref
        self.model = self._build(seed, self.value_head)
        if with_ref:
            self.ref_model = self._build(seed, False, recompute="none")
            for p in self.ref_model.parameters():
                p.requires_grad_(False)
        world = dist.get_world_size() if dist.is_initialized() else 1
        self.mesh = init_device_mesh(self.device.type, (world,)) if world > 1 else None
        if self.mesh is not None:
            mp = None
            if self.device.type == "cuda" and self.model_cfg.dtype == "bfloat16":
                mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
            kw = dict(mesh=self.mesh, **({"mp_policy": mp} if mp is not None else {}))
            for m in ([self.model] + ([self.ref_model] if self.ref_model is not None else [])):
                for layer in m.decoder.layers:
                    fully_shard(layer, **kw)
                fully_shard(m, **kw)
            # micro-batch losses are already normalised by global counts: gradients are summed over ranks (a custom
            # divide factor needs a pre-multiplied reduction, which only NCCL offers; elsewhere undo the average)
            if hasattr(self.model, "set_reduce_scatter_divide_factor") and dist.get_backend() == "nccl":
                self.model.set_reduce_scatter_divide_factor(1.0)
                self._grad_mult = 1.0
            else:
                self._grad_mult = float(world)
        else:
            self._grad_mult = 1.0
        cfg = self.opt_cfg
        params = [p for p in self.model.parameters() if p.requires_grad]
        if cfg.optimizer_type == "muon":
            from ..core.muon import Muon, split_muon_params
            mu, ad = split_muon_params(self.model)
            self.torch_opt = Muon(mu, ad, lr=cfg.lr, wd=cfg.weight_decay, momentum=cfg.muon_momentum,
                                  ns_steps=cfg.muon_ns_steps)
        else:
            self.torch_opt = torch.optim.AdamW(params, lr=cfg.lr, betas=(cfg.adam_beta1, cfg.adam_beta2),
                                               eps=cfg.adam_eps, weight_decay=cfg.weight_decay)
        self.ddp = _GradShim(self.model)
        self.optimizer = _OptShim(self)
        return self

    def _finish_step(self, lr=None):
        cfg = self.opt_cfg
        self.optimizer.step_count += 1
        lr = lr if lr is not None else lr_at_step(cfg, self.optimizer.step_count, self.total_steps)
        for g in self.torch_opt.param_groups:
            g["lr"] = lr
        if self._grad_mult != 1.0:
            for p in self.model.parameters():
                if p.grad is not None:
                    p.grad.mul_(self._grad_mult)
        params = [p for p in self.model.parameters() if p.grad is not None]
        max_norm = cfg.max_grad_norm if (cfg.max_grad_norm and cfg.max_grad_norm > 0) else float("inf")
        norm = torch.nn.utils.clip_grad_norm_(params, max_norm)
        if hasattr(norm, "full_tensor"):
            norm = norm.full_tensor()
        self.optimizer.last_grad_norm = norm.detach()
        self.torch_opt.step()
        self.torch_opt.zero_grad(set_to_none=True)
        self.step += 1
        return float(lr), float(norm)

    def release_grad_buffers(self):
        self.ddp.release_grads()

    def allocate_grad_buffers(self):
        pass

    # ------------------------------------------------------------------ DCP checkpoint
    def save_checkpoint(self, path: str, step: int):
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.state_dict import get_model_state_dict, get_optimizer_state_dict
        sd = {"model": get_model_state_dict(self.model)}
        if not isinstance(self.torch_opt, torch.optim.Optimizer) or self.opt_cfg.optimizer_type != "muon":
            sd["optim"] = get_optimizer_state_dict(self.model, self.torch_opt)
        d = os.path.join(path, f"iter_{step:07d}")
        dcp.save(sd, checkpoint_id=d)
        if not dist.is_initialized() or dist.get_rank() == 0:
            with open(os.path.join(path, "latest_checkpointed_iteration.txt"), "w") as f:
                f.write(str(step))
        return d

    def load_checkpoint(self, path: str, step: Optional[int] = None) -> int:
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.state_dict import (get_model_state_dict, get_optimizer_state_dict,
                                                             set_model_state_dict, set_optimizer_state_dict)
        if step is None:
            step = int(open(os.path.join(path, "latest_checkpointed_iteration.txt")).read().strip())
        sd = {"model": get_model_state_dict(self.model)}
        has_opt = self.opt_cfg.optimizer_type != "muon"
        if has_opt:
            sd["optim"] = get_optimizer_state_dict(self.model, self.torch_opt)
        dcp.load(sd, checkpoint_id=os.path.join(path, f"iter_{step:07d}"))
        set_model_state_dict(self.model, sd["model"])
        if has_opt:
            set_optimizer_state_dict(self.model, self.torch_opt, sd["optim"])
        self.optimizer.step_count = self.step = step
        return step
