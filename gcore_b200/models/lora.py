"""LoRA adapters for the tensor-parallel linears: ``y = x W^T + (alpha / r) * (x A^T) B^T``.

Covers what the reference gets from mbridge / Megatron-Bridge PEFT (gpatch_v4/training_backend/megatron_backend/
mcore_peft.py:72-449, docs/source/lora-peft.md): ``lora`` adapts the fused module as one matrix, ``canonical_lora``
gives every logical sub-matrix (q / k / v, gate / up) its own A and B; adapters are TP-sharded like their base
layer (column-parallel: B sharded, row-parallel: A sharded - the partial product joins the layer's existing
reduce), expert layers share one adapter or own one each; ``verify_lora_weight_consistency`` hashes the replicated
halves across the TP group; export gives adapter-only or merged weights.
"""
from __future__ import annotations

import hashlib
import math
import zlib
from typing import Dict, List

import torch
import torch.distributed as dist
import torch.nn as nn


class LoRAAdapter(nn.Module):
    def __init__(self, in_local: int, out_splits: List[int], rank: int, alpha: float, dropout: float, dtype, device,
                 a_init="xavier", b_init="zero", seed: int = 0):
        """``out_splits`` lists the output widths of the logical sub-matrices (one entry for plain ``lora``)."""
        super().__init__()
        self.scale = alpha / rank
        self.rank = rank
        self.out_splits = out_splits
        n = len(out_splits)
        self.lora_A = nn.Parameter(torch.empty(n * rank, in_local, dtype=dtype, device=device))
        self.lora_B = nn.ParameterList(
            [nn.Parameter(torch.zeros(o, rank, dtype=dtype, device=device)) for o in out_splits])
        self.dropout = nn.Dropout(dropout) if dropout > 0 else None
        g = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            if a_init == "xavier":
                bound = math.sqrt(6.0 / (in_local + rank))
                self.lora_A.copy_((torch.rand(n * rank, in_local, generator=g) * 2 - 1) * bound)
            else:
                self.lora_A.copy_(torch.randn(n * rank, in_local, generator=g) * 0.02)
            if b_init != "zero":
                for b in self.lora_B:
                    b.copy_(torch.randn(b.shape, generator=g) * 0.02)
        self.lora_A.is_lora = True
        for b in self.lora_B:
            b.is_lora = True

    def forward(self, x):
        if self.dropout is not None:
            x = self.dropout(x)
        xa = torch.nn.functional.linear(x, self.lora_A)  # [T, n*r]
        outs = []
        for i, b in enumerate(self.lora_B):
            outs.append(torch.nn.functional.linear(xa[..., i * self.rank:(i + 1) * self.rank], b))
        y = outs[0] if len(outs) == 1 else torch.cat(outs, dim=-1)
        return y * self.scale

    def delta_weight(self) -> torch.Tensor:
        """``[out_local, in_local]`` dense update (for merged export and the fp8 rollout path)."""
        parts = []
        for i, b in enumerate(self.lora_B):
            parts.append(b.float() @ self.lora_A[i * self.rank:(i + 1) * self.rank].float())
        return torch.cat(parts, 0) * self.scale


class ExpertLoRA(nn.Module):
    """Adapter of a grouped expert projection ``[E, out, in]`` applied to the expert-sorted token rows: one A / B pair
    shared by all local experts (``shared=True``: two dense products over all rows) or a pair per expert (rows are
    taken expert by expert from the offsets of the dispatch plan)."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, rank: int, alpha: float, shared: bool,
                 dtype, device, seed: int = 0):
        super().__init__()
        self.scale, self.rank, self.shared, self.num_experts = alpha / rank, rank, shared, num_experts
        n = 1 if shared else num_experts
        g = torch.Generator(device="cpu").manual_seed(seed)
        bound = math.sqrt(6.0 / (in_features + rank))
        self.lora_A = nn.Parameter(((torch.rand(n, rank, in_features, generator=g) * 2 - 1) * bound).to(dtype).to(device))
        self.lora_B = nn.Parameter(torch.zeros(n, out_features, rank, dtype=dtype, device=device))
        for p in (self.lora_A, self.lora_B):
            p.is_lora = True
            # a shared adapter is replicated like a dense parameter; per-expert adapters live with their experts
            p.tp_mode = "none" if shared else "expert"
            if not shared:
                p.is_expert = True
            else:
                # acts on the tokens of this rank's sequence-parallel shard, like the norm gains and the router
                p.sequence_parallel = True

    def forward(self, x_perm, offsets):
        x_perm = x_perm.to(self.lora_A.dtype)
        if self.shared:
            return torch.nn.functional.linear(torch.nn.functional.linear(x_perm, self.lora_A[0]), self.lora_B[0]) * self.scale
        out = x_perm.new_zeros(x_perm.shape[0], self.lora_B.shape[1])
        bounds = offsets.tolist()
        for e in range(self.num_experts):
            a, b = bounds[e], bounds[e + 1]
            if b > a:
                out[a:b] = torch.nn.functional.linear(torch.nn.functional.linear(x_perm[a:b], self.lora_A[e]),
                                                      self.lora_B[e]) * self.scale
        return out

    def delta_weight(self) -> torch.Tensor:
        """``[E, out, in]`` dense update."""
        d = torch.matmul(self.lora_B.float(), self.lora_A.float()) * self.scale
        return d.expand(self.num_experts, -1, -1) if self.shared else d


def _splits_for(name: str, module, cfg, tp_size: int, canonical: bool) -> List[int]:
    if not canonical:
        return [module.out_local]
    if name.endswith("linear_qkv"):
        D = cfg.head_dim
        return [cfg.num_attention_heads // tp_size * D, cfg.num_kv_heads // tp_size * D,
                cfg.num_kv_heads // tp_size * D]
    if name.endswith("linear_fc1"):
        return [module.out_local // 2, module.out_local // 2]
    return [module.out_local]


def apply_lora(model: nn.Module, lora_cfg, seed: int = 0) -> Dict[str, LoRAAdapter]:
    """Freezes the base model and attaches adapters to every ``ParallelLinear`` whose name matches
    ``target_modules`` (and none of ``exclude_modules``).  Returns ``{module name: adapter}``."""
    from .gpt import ParallelLinear
    if not lora_cfg.enabled:
        return {}
    for p in model.parameters():
        p.requires_grad_(False)
    cfg = model.cfg
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, None: None}.get(lora_cfg.dtype)
    adapters = {}
    for name, mod in model.named_modules():
        if not isinstance(mod, ParallelLinear):
            continue
        leaf = name.split(".")[-1]
        if leaf not in lora_cfg.target_modules or any(e in name for e in lora_cfg.exclude_modules):
            continue
        w = mod.weight
        ad = LoRAAdapter(mod.in_local, _splits_for(name, mod, cfg, mod.tp_size, lora_cfg.type == "canonical_lora"),
                         lora_cfg.rank, lora_cfg.alpha, lora_cfg.dropout, dtype or w.dtype, w.device,
                         lora_cfg.lora_A_init_method, lora_cfg.lora_B_init_method,
                         seed=(seed + zlib.crc32(name.encode())) & 0x7FFFFFFF)  # crc, not hash(): equal in every process
        # replicated halves must be identical across the TP group
        ad.lora_A.tp_mode = "row" if mod.mode == "row" else "none"
        for b in ad.lora_B:
            b.tp_mode = "column" if mod.mode == "column" else "none"
        if mod.tp_size > 1 and mod.mode in ("column", "row"):
            # the replicated half of an adapter on a sharded projection (A of a column-parallel layer, B of a
            # row-parallel one) receives from every TP rank only the part of its gradient that flows through that
            # rank's shard of the other half: the parts are summed over the TP group with the gradient reduction
            for q in ([ad.lora_A] if mod.mode == "column" else list(ad.lora_B)):
                q.tp_partial_grad = True
        elif getattr(w, "tp_partial_grad", False):
            # a replicated projection in front of sharded heads (latent-attention down-projections): both halves of
            # its adapter get per-rank partial gradients, like the weight itself
            for q in [ad.lora_A] + list(ad.lora_B):
                q.tp_partial_grad = True
        mod.lora = ad
        adapters[name] = ad
    # grouped expert projections: `linear_fc1` / `linear_fc2` among the targets also adapt the experts, with one
    # adapter per layer (`share_expert_adapters`) or one per expert
    from .moe import Experts
    for name, mod in model.named_modules():
        if not isinstance(mod, Experts) or any(e in name for e in lora_cfg.exclude_modules):
            continue
        for leaf in ("linear_fc1", "linear_fc2"):
            if leaf not in lora_cfg.target_modules:
                continue
            w = getattr(mod, leaf).weight
            ad = ExpertLoRA(w.shape[0], w.shape[2], w.shape[1], lora_cfg.rank, lora_cfg.alpha,
                            lora_cfg.share_expert_adapters, dtype or w.dtype, w.device,
                            seed=(seed + zlib.crc32(f"{name}.{leaf}".encode())) & 0x7FFFFFFF)
            setattr(mod, "lora_" + leaf[len("linear_"):], ad)
            adapters[f"{name}.{leaf}"] = ad
    if "router" in lora_cfg.target_modules:
        # the routing matrix [experts, hidden] is a plain fp32 parameter: its adapter is replicated over TP like it
        from .moe import Router
        for name, mod in model.named_modules():
            if isinstance(mod, Router) and not any(e in name for e in lora_cfg.exclude_modules):
                w = mod.weight
                ad = LoRAAdapter(w.shape[1], [w.shape[0]], lora_cfg.rank, lora_cfg.alpha, lora_cfg.dropout, w.dtype,
                                 w.device, lora_cfg.lora_A_init_method, lora_cfg.lora_B_init_method,
                                 seed=(seed + zlib.crc32(name.encode())) & 0x7FFFFFFF)
                ad.lora_A.tp_mode = "none"
                ad.lora_A.sequence_parallel = True     # sees the tokens of this rank's sequence-parallel shard
                for b in ad.lora_B:
                    b.tp_mode = "none"
                    b.sequence_parallel = True
                mod.lora = ad
                adapters[name] = ad
    if lora_cfg.check_lora_all_coverage:
        missing = [n for n, m in model.named_modules() if isinstance(m, ParallelLinear) and m.lora is None
                   and n.split(".")[-1] in lora_cfg.target_modules]
        if missing:
            raise RuntimeError(f"LoRA coverage check failed for: {missing}")
    return adapters


def lora_coverage_report(model) -> Dict[str, bool]:
    from .gpt import ParallelLinear
    return {n: m.lora is not None for n, m in model.named_modules() if isinstance(m, ParallelLinear)}


def verify_lora_weight_consistency(adapters: Dict[str, LoRAAdapter], group) -> bool:
    """Replicated adapter halves must hash identically on every rank of the TP group
    (gpatch_v4/training_backend/megatron_backend/mcore_peft.py:275-449)."""
    h = hashlib.sha256()
    for name in sorted(adapters):
        ad = adapters[name]
        if getattr(ad.lora_A, "tp_mode", "none") == "none":
            h.update(ad.lora_A.detach().float().cpu().numpy().tobytes())
        for b in ad.lora_B:
            if getattr(b, "tp_mode", "none") == "none":
                h.update(b.detach().float().cpu().numpy().tobytes())
    digest = int.from_bytes(h.digest()[:7], "big")
    if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return True
    t = torch.tensor([digest, -digest], dtype=torch.int64)
    if dist.get_backend(group) == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return int(t[0]) == -int(t[1])


def merge_lora_(model) -> None:
    """Folds every adapter into its base weight in place (merged export)."""
    from .gpt import ParallelLinear
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, ParallelLinear) and m.lora is not None:
                m.weight.add_(m.lora.delta_weight().to(m.weight.dtype))
            elif type(m).__name__ == "Router" and getattr(m, "lora", None) is not None:
                m.weight.add_(m.lora.delta_weight().to(m.weight.dtype))
            elif type(m).__name__ == "Experts":
                for leaf in ("fc1", "fc2"):
                    ad = getattr(m, "lora_" + leaf, None)
                    if ad is not None:
                        w = getattr(m, "linear_" + leaf).weight
                        w.add_(ad.delta_weight().to(w.dtype))


def lora_state_dict(model) -> Dict[str, torch.Tensor]:
    return {n: p.detach() for n, p in model.named_parameters() if getattr(p, "is_lora", False)}
