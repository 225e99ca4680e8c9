"""Pipeline contract and what every pipeline shares: model / optimizer construction, data-parallel gradient
averaging, EMA weights, checkpoints.

The verbs are those of the reference's ``ExtendedPipelineAbc`` (gpatch_v4/extended_pipeline/pipeline_base.py:11-108):
``setup_pipeline``, ``encode_prompt``, ``repeat_interleave_tensor_or_list``, ``permute_timesteps``, ``__call__``
(rollout: returns the training rollout batch and the reward-model request), ``ppo_train_step``, ``sft_train_step``.
"""
from __future__ import annotations

import copy
import os
from abc import ABC, abstractmethod
from typing import Any, Dict, List, Optional, Union

import torch
import torch.distributed as dist


def unbind_to_list(t: torch.Tensor) -> List[torch.Tensor]:
    return list(t.unbind(0))


class EmaModel:
    """Exponential moving average of a module's parameters (the T2I engines' EMA copy,
    gpatch_v4/training_backend/fsdp2_backend/ema_model_t2i.py)."""

    def __init__(self, module: torch.nn.Module, decay: float = 0.999):
        self.decay = decay
        self.shadow = {n: p.detach().clone().float() for n, p in module.named_parameters() if p.requires_grad}

    @torch.no_grad()
    def update(self, module: torch.nn.Module):
        for n, p in module.named_parameters():
            if n in self.shadow:
                self.shadow[n].lerp_(p.detach().float(), 1 - self.decay)

    @torch.no_grad()
    def copy_to(self, module: torch.nn.Module):
        for n, p in module.named_parameters():
            if n in self.shadow:
                p.copy_(self.shadow[n].to(p.dtype))

    def state_dict(self):
        return {"decay": self.decay, "shadow": self.shadow}

    def load_state_dict(self, sd):
        self.decay = sd["decay"]
        for k, v in sd["shadow"].items():
            self.shadow[k].copy_(v)


class ExtendedPipeline(ABC):
    def __init__(self, config):
        self.config = config
        self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
            else torch.device("cpu")
        self.model: Optional[torch.nn.Module] = None
        self.optimizer: Optional[torch.optim.Optimizer] = None
        self.ema: Optional[EmaModel] = None
        self.step = 0

    # ---- contract
    @abstractmethod
    def setup_pipeline(self) -> int:
        ...

    @abstractmethod
    def encode_prompt(self, prompt: List[str], **kw):
        ...

    @abstractmethod
    def __call__(self, **kw):
        ...

    @abstractmethod
    def ppo_train_step(self, rollout_batches: List[Dict[str, Any]]) -> Dict[str, float]:
        ...

    @abstractmethod
    def sft_train_step(self, rollout_batches: List[Dict[str, Any]]) -> Dict[str, float]:
        ...

    def repeat_interleave_tensor_or_list(self, rb: Dict[str, Union[List[Any], torch.Tensor]], repeat: int):
        """Every prompt-level entry becomes ``repeat`` consecutive sample-level entries."""
        out = {}
        for k, v in rb.items():
            if isinstance(v, torch.Tensor):
                out[k] = v.repeat_interleave(repeat, dim=0)
            else:
                out[k] = [x for x in v for _ in range(repeat)]
        return out

    def permute_timesteps(self, rb: Dict[str, List[Any]], generator: Optional[torch.Generator] = None):
        """Shuffles the time axis of every sample's trajectory (the same permutation for all of its per-step fields)
        and records it under ``perms``: the update then trains on a random subset of steps
        (pipeline_flux.py:146-168)."""
        n = len(rb["timesteps"])
        perms = []
        for i in range(n):
            T = rb["timesteps"][i].shape[0]
            perm = torch.randperm(T, generator=generator)
            for k in ("timesteps", "latents", "next_latents", "log_probs"):
                rb[k][i] = rb[k][i][perm]
            perms.append(perm)
        rb["perms"] = perms
        return rb

    # ---- shared machinery
    def _dtype(self):
        return torch.bfloat16 if (self.device.type == "cuda" and self.config.training.use_bf16) else torch.float32

    def build_optimizer(self, module: torch.nn.Module):
        oc = self.config.optimizer
        params = [p for p in module.parameters() if p.requires_grad]
        self.optimizer = torch.optim.AdamW(params, lr=oc.lr, betas=(oc.adam_beta1, oc.adam_beta2), eps=oc.adam_eps,
                                           weight_decay=oc.weight_decay)
        if self.config.training.ema_decay:
            self.ema = EmaModel(module, self.config.training.ema_decay)
        return self.optimizer

    def sync_grads(self, module: torch.nn.Module):
        """Data-parallel mean of the gradients (one flat all-reduce)."""
        if not (dist.is_initialized() and dist.get_world_size() > 1):
            return
        grads = [p.grad for p in module.parameters() if p.grad is not None]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat)
        flat /= dist.get_world_size()
        o = 0
        for g in grads:
            g.copy_(flat[o:o + g.numel()].view_as(g))
            o += g.numel()

    def optimizer_step(self, module: torch.nn.Module) -> float:
        self.sync_grads(module)
        oc = self.config.optimizer
        max_norm = oc.max_grad_norm if (oc.max_grad_norm and oc.max_grad_norm > 0) else float("inf")
        norm = torch.nn.utils.clip_grad_norm_([p for p in module.parameters() if p.grad is not None], max_norm)
        self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)
        if self.ema is not None:
            self.ema.update(module)
        self.step += 1
        return float(norm)

    def reduce_mean(self, *vals) -> List[float]:
        t = torch.tensor([float(v) for v in vals], device=self.device if dist.is_initialized() and
                         dist.get_backend() == "nccl" else "cpu")
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(t)
            t /= dist.get_world_size()
        return t.tolist()

    # ---- checkpoints: iter_XXXXXXX/pipeline.pt + latest file, as the language-model trainers lay theirs out
    def save_checkpoint(self, root: str, step: Optional[int] = None) -> str:
        step = self.step if step is None else step
        d = os.path.join(root, f"iter_{step:07d}")
        if not dist.is_initialized() or dist.get_rank() == 0:
            os.makedirs(d, exist_ok=True)
            sd = {"model": self.model.state_dict(), "step": step,
                  "optimizer": self.optimizer.state_dict() if self.optimizer is not None else None,
                  "ema": self.ema.state_dict() if self.ema is not None else None}
            torch.save(sd, os.path.join(d, "pipeline.pt"))
            with open(os.path.join(root, "latest_checkpointed_iteration.txt"), "w") as f:
                f.write(str(step))
        if dist.is_initialized():
            dist.barrier()
        return d

    def load_checkpoint(self, root: str) -> int:
        p = os.path.join(root, "latest_checkpointed_iteration.txt")
        if not os.path.exists(p):
            return 0
        step = int(open(p).read().strip())
        sd = torch.load(os.path.join(root, f"iter_{step:07d}", "pipeline.pt"), map_location=self.device,
                        weights_only=False)
        self.model.load_state_dict(sd["model"])
        if sd.get("optimizer") is not None and self.optimizer is not None:
            self.optimizer.load_state_dict(sd["optimizer"])
        if sd.get("ema") is not None and self.ema is not None:
            self.ema.load_state_dict(sd["ema"])
        self.step = step
        return step

    def frozen_copy(self, module: torch.nn.Module) -> torch.nn.Module:
        ref = copy.deepcopy(module)
        for p in ref.parameters():
            p.requires_grad_(False)
        return ref.eval()
