"""Mixture-of-experts layer: router (softmax top-k for Qwen3-MoE, sigmoid group-limited top-k with selection bias for
DeepSeek-V3), capacity-free token dispatch into an expert-sorted buffer whose segments are padded to 128 rows, ragged
grouped GEMMs on the tcgen05 kernel, weighted combine, optional shared expert, load-balancing / z losses, and router
replay (recorded expert ids from the rollout engine override the top-k choice, as in
gpatch_v4/training_backend/megatron_backend/router_replay_manager.py:15).

Dispatch semantics follow ``DeepseekV4Experts._forward_eager`` (gpatch_v4/models/deepseek_v4/modeling_deepseek_v4.py:
1221-1289): sort by destination rank, exchange counts, exchange tokens, sort by local expert, grouped MM, reverse.
"""
from __future__ import annotations


import torch
import torch.nn as nn

from ..core import parallel_state as ps
from ..ops import fused
from ..ops.gemm import grouped_gemm, grouped_wgrad
from .config import ModelConfig

SEG = 128  # expert segments are padded to the GEMM tile height


class RouterReplay:
    """Per-step store of routed expert ids, keyed by layer index ([T, K] int64 each)."""
    _store = {}
    mode = "off"  # off | record | replay

    @classmethod
    def set(cls, mode, store=None):
        cls.mode = mode
        cls._store = store if store is not None else {}

    @classmethod
    def get(cls, layer):
        return cls._store.get(layer)

    @classmethod
    def put(cls, layer, idx):
        cls._store[layer] = idx


class Router(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device=None):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.weight = nn.Parameter(torch.empty(cfg.num_experts, cfg.hidden_size, dtype=torch.float32, device=device))
        self.weight.tp_mode = "none"
        self.weight.sequence_parallel = True
        if cfg.moe_router_bias:
            # selection-only bias updated outside autograd (aux-loss-free balancing)
            self.register_buffer("expert_bias", torch.zeros(cfg.num_experts, dtype=torch.float32, device=device))
            # tokens routed to each expert since the last bias update (training passes only)
            self.register_buffer("tokens_per_expert", torch.zeros(cfg.num_experts, dtype=torch.float32, device=device),
                                 persistent=False)
        else:
            self.expert_bias = None
            self.tokens_per_expert = None
        self.lora = None   # optional low-rank adapter on the routing matrix ("router" in lora.target_modules)

    def forward(self, x):
        cfg = self.cfg
        E, K = cfg.num_experts, cfg.moe_top_k
        logits = torch.nn.functional.linear(x.float(), self.weight)  # [T, E]
        if self.lora is not None:
            logits = logits + self.lora(x.float())
        replay = RouterReplay.get(self.layer_idx) if RouterReplay.mode == "replay" else None
        from ..ops.router import route
        sigmoid = cfg.moe_router_type != "softmax"
        idx, w = route(logits, self.expert_bias if sigmoid else None, replay, K, cfg.moe_n_group if sigmoid else 1,
                       cfg.moe_topk_group if sigmoid else 1, sigmoid, cfg.moe_norm_topk_prob,
                       cfg.moe_routed_scaling_factor if sigmoid else 1.0)
        if RouterReplay.mode == "record":
            RouterReplay.put(self.layer_idx, idx.detach())
        if self.tokens_per_expert is not None and self.training and torch.is_grad_enabled():
            # with activation recomputation the first pass runs without grad, so every token is counted once
            with torch.no_grad():
                flat = idx.reshape(-1)
                self.tokens_per_expert.scatter_add_(0, flat, torch.ones_like(flat, dtype=torch.float32))
        aux = None
        if self.training and (cfg.moe_aux_loss_coef > 0 or cfg.moe_z_loss_coef > 0):
            aux = x.new_zeros((), dtype=torch.float32)
            if cfg.moe_aux_loss_coef > 0:
                T = logits.shape[0]
                f = torch.zeros(E, dtype=torch.float32, device=x.device)
                f.scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=x.device))
                f = f * (E / (K * max(T, 1)))
                if sigmoid:
                    scores = torch.sigmoid(logits)
                    P = (scores / scores.sum(-1, keepdim=True).clamp_min(1e-20)).mean(0)
                else:
                    P = torch.softmax(logits, dim=-1).mean(0)
                aux = aux + cfg.moe_aux_loss_coef * (f * P).sum()
            if cfg.moe_z_loss_coef > 0:
                aux = aux + cfg.moe_z_loss_coef * torch.logsumexp(logits, -1).pow(2).mean()
        return idx, w, aux


@torch.no_grad()
def update_router_bias(model: nn.Module, speed: float, use_abs: bool = True, groups=()):
    """Loss-free load balancing (arXiv 2408.15664): after an optimizer step the selection bias of every expert moves by
    ``speed`` towards the mean load, ``sign(mean - count)`` (``use_abs``) or ``log((mean + 1) / (count + 1))``; counts
    are summed over ``groups`` (the groups that shard tokens: data / context parallel and the sequence-parallel tensor
    group).  Returns (max, mean) over layers of the maximal violation ``(max_e count - mean) / mean``, or None when no
    router carries a bias (gpatch_v4/models/deepseek_v4/freeze_update_router.py:120-178)."""
    import torch.distributed as dist
    routers = [m for m in model.modules() if isinstance(m, Router) and m.tokens_per_expert is not None]
    if not routers:
        return None
    counts = torch.stack([r.tokens_per_expert for r in routers]).double()
    for g in groups:
        if g is not None and dist.is_initialized() and dist.get_world_size(g) > 1:
            dist.all_reduce(counts, group=g)
    avg = counts.mean(-1, keepdim=True)
    if use_abs:
        delta = torch.sign(avg - counts) * speed
    else:
        delta = torch.log((avg + 1.0) / (counts + 1.0)) * speed
    for i, r in enumerate(routers):
        r.expert_bias.add_(delta[i].to(r.expert_bias.dtype))
        r.tokens_per_expert.zero_()
    vio = (counts.max(-1).values - avg[:, 0]) / avg[:, 0].clamp_min(1e-12)
    return float(vio.max()), float(vio.mean())


def build_dispatch_plan(expert_ids: torch.Tensor, num_experts: int):
    """expert_ids [N] (N = tokens * K, values in [0, E)) -> (dest_row [N], offsets [E+1] int32) for the padded
    expert-sorted layout; no host synchronisation."""
    N = expert_ids.numel()
    # scatter_add, not bincount: bincount reads its maximum back to the host, which a CUDA-graph capture (decode
    # steps of the rollout engine) does not allow
    counts = torch.zeros(num_experts, dtype=torch.int64, device=expert_ids.device).scatter_add_(
        0, expert_ids, torch.ones_like(expert_ids, dtype=torch.int64))
    padded = (counts + (SEG - 1)) // SEG * SEG
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=expert_ids.device)
    offsets[1:] = padded.cumsum(0)
    starts = counts.cumsum(0) - counts
    order = torch.argsort(expert_ids, stable=True)
    e_sorted = expert_ids[order]
    pos_in_e = torch.arange(N, device=expert_ids.device) - starts[e_sorted]
    dest = torch.empty(N, dtype=torch.int64, device=expert_ids.device)
    dest[order] = offsets[e_sorted] + pos_in_e
    return dest, offsets.to(torch.int32)


def padded_rows_bound(n_rows: int, num_experts: int) -> int:
    return ((n_rows + num_experts * (SEG - 1)) + SEG - 1) // SEG * SEG


class _GroupedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, offsets, main_grad):
        ctx.save_for_backward(x, w, offsets)
        ctx.main_grad = main_grad
        return grouped_gemm(x, w, offsets)

    @staticmethod
    def backward(ctx, dy):
        x, w, offsets = ctx.saved_tensors
        dy = dy.contiguous()
        dx = grouped_gemm(dy, w, offsets, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            if ctx.main_grad is not None:
                grouped_wgrad(dy, x, offsets, w.shape[0], out=ctx.main_grad, accumulate=True)
            else:
                dw = grouped_wgrad(dy, x, offsets, w.shape[0]).to(w.dtype)
        return dx, dw, None, None


class _GroupedFp8LinearFn(torch.autograd.Function):
    """Grouped expert projection in block-scaled e4m3 (activations 1x128 per token, weights 128x128, cached until the
    parameter changes); like the dense fp8 linear, the data gradient runs on the same grouped GEMM against the
    transposed e4m3 cache, the weight gradient in bf16, skipped for a frozen base (the reference's grouped fp8 linear:
    gpatch_v4/models/deepseek_v4/fp8.py:181-394)."""

    @staticmethod
    def forward(ctx, x, w, offsets, main_grad, cache):
        from ..ops import quant
        G, N, K = w.shape
        ver = (w._version, w.data_ptr())
        if cache.get("ver") != ver:
            q, s = quant.quant_weight_128x128(w.detach().to(torch.bfloat16).reshape(G * N, K).contiguous())
            cache.update(ver=ver, q=q, s=s)
        aq, as_ = quant.quant_act_1x128(x.to(torch.bfloat16).contiguous())
        y = quant.gemm_fp8_grouped(aq, as_, cache["q"], cache["s"], offsets, G, out_dtype=x.dtype
                                   if x.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16)
        ctx.save_for_backward(x if w.requires_grad else x.new_empty(0), w, offsets)
        ctx.cache, ctx.main_grad = cache, main_grad
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops import quant
        x, w, offsets = ctx.saved_tensors
        G, N, K = w.shape
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            from ..ops.lowp_linear import fp8_dgrad_enabled
            if fp8_dgrad_enabled() and dy.shape[0] % 128 == 0:
                dx = quant.fp8_dgrad(dy, ctx.cache, dy.dtype, offsets=offsets, groups=G)
            else:
                w_dq = quant.dequant_128x128(ctx.cache["q"], ctx.cache["s"])[:G * N, :K].to(dy.dtype).view(G, N, K)
                dx = grouped_gemm(dy, w_dq.contiguous(), offsets, b_mn=True)
        if ctx.needs_input_grad[1]:
            if ctx.main_grad is not None:
                grouped_wgrad(dy, x, offsets, G, out=ctx.main_grad, accumulate=True)
            else:
                dw = grouped_wgrad(dy, x, offsets, G).to(w.dtype)
        return dx, dw, None, None, None


def grouped_linear(x, w, offsets, precision=None, cache=None):
    """``y[seg_g] = x[seg_g] @ w[g]^T`` with autograd; ``w`` [G, N, K].  ``precision="fp8"`` runs the product on the
    grouped block-fp8 GEMM (N and K multiples of 128)."""
    mg = getattr(w, "main_grad", None) if w.requires_grad else None
    if precision == "fp8" and w.shape[1] % 128 == 0 and w.shape[2] % 128 == 0:
        return _GroupedFp8LinearFn.apply(x, w, offsets, mg, cache if cache is not None else {})
    return _GroupedLinearFn.apply(x, w, offsets, mg)


class Experts(nn.Module):
    def __init__(self, cfg: ModelConfig, num_local: int, device=None):
        super().__init__()
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[cfg.dtype]
        F, H = cfg.moe_ffn_hidden_size, cfg.hidden_size
        self.linear_fc1 = nn.Module()
        self.linear_fc2 = nn.Module()
        self.linear_fc1.weight = nn.Parameter(torch.empty(num_local, 2 * F, H, dtype=dt, device=device))
        self.linear_fc2.weight = nn.Parameter(torch.empty(num_local, H, F, dtype=dt, device=device))
        self.linear_fc1.weight.tp_mode = "expert"
        self.linear_fc2.weight.tp_mode = "expert"
        self.linear_fc1.weight.is_expert = True
        self.linear_fc2.weight.is_expert = True
        self.lora_fc1 = self.lora_fc2 = None   # models/lora.py::ExpertLoRA when the experts are adapted
        self.precision = None                  # None (bf16) | "fp8": grouped block-fp8 GEMM (policy.fp8)
        self._fp8_cache = ({}, {})

    def forward(self, x_perm, offsets):
        h = grouped_linear(x_perm, self.linear_fc1.weight, offsets, self.precision, self._fp8_cache[0])
        if self.lora_fc1 is not None:
            h = h + self.lora_fc1(x_perm, offsets).to(h.dtype)
        # offsets[-1] = rows in use (the buffer is sized for the worst case): without autograd only those are activated
        h = fused.swiglu(h, n_rows=offsets[-1:] if offsets.dtype == torch.int32 else None)
        y = grouped_linear(h, self.linear_fc2.weight, offsets, self.precision, self._fp8_cache[1])
        if self.lora_fc2 is not None:
            y = y + self.lora_fc2(h, offsets).to(y.dtype)
        return y


class MoELayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, tp_size: int, ep_size: int, device=None):
        super().__init__()
        self.cfg, self.layer_idx, self.ep_size = cfg, layer_idx, ep_size
        assert cfg.num_experts % ep_size == 0
        self.num_local = cfg.num_experts // ep_size
        self.router = Router(cfg, layer_idx, device)
        self.experts = Experts(cfg, self.num_local, device)
        if cfg.moe_shared_expert_ffn:
            from .gpt import MLP
            # shared expert is replicated (not TP-sharded) because it runs on the sequence-parallel token shard
            self.shared_experts = MLP(cfg, cfg.moe_shared_expert_ffn, 1, device)
        else:
            self.shared_experts = None
        self.shared_expert_gate = None
        if self.shared_experts is not None and getattr(cfg, "moe_shared_expert_gate", False):
            dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[cfg.dtype]
            self.shared_expert_gate = nn.Module()
            self.shared_expert_gate.weight = nn.Parameter(torch.zeros(1, cfg.hidden_size, dtype=dt, device=device))
            self.shared_expert_gate.weight.tp_mode = "none"
            self.shared_expert_gate.weight.sequence_parallel = True

    def forward(self, x):
        cfg = self.cfg
        T, H = x.shape
        K = cfg.moe_top_k
        idx, w, aux = self.router(x)
        if self.ep_size > 1:
            from ..parallel.ep import ep_moe_forward
            y = ep_moe_forward(self, x, idx, w)
        else:
            flat_e = idx.reshape(-1)
            dest, offsets = build_dispatch_plan(flat_e, cfg.num_experts)
            rows = padded_rows_bound(T * K, cfg.num_experts)
            x_perm = torch.zeros(rows, H, dtype=x.dtype, device=x.device)
            token_of = torch.arange(T, device=x.device).repeat_interleave(K)
            x_perm = x_perm.index_copy(0, dest, x[token_of])
            y_perm = self.experts(x_perm, offsets)
            y = (y_perm[dest].view(T, K, H) * w.to(x.dtype)[:, :, None]).sum(1)
        if self.shared_experts is not None:
            ys = self.shared_experts(x)
            if self.shared_expert_gate is not None:
                ys = ys * torch.sigmoid(torch.nn.functional.linear(x, self.shared_expert_gate.weight))
            y = y + ys
        return y, aux
