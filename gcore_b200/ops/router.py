"""Expert routing op: scores -> (expert ids [T, K] int64, weights [T, K] fp32), one kernel forward, one backward
(``csrc/router.cu``).  ``route_ref`` is the PyTorch definition: the CPU path and the oracle of the kernel test.

Semantics: softmax routers pick the top-k probabilities and optionally renormalise them (Qwen MoE families); sigmoid
routers add a selection-only bias, optionally keep only the best ``topk_group`` of ``n_group`` expert groups (group
score = sum of its two best biased scores), pick the top-k, take the unbiased scores as weights, renormalise and scale
(DeepSeek families; the reference's gate: gpatch_v4/models/deepseek_v4/modeling_deepseek_v4.py:1120-1219).
"""
from __future__ import annotations

import torch

from . import _lib

LAUNCHES = {"router": 0}


def route_ref(logits, bias, replay, K, n_group, topk_group, sigmoid, norm, scale):
    E = logits.shape[-1]
    scores = torch.sigmoid(logits) if sigmoid else torch.softmax(logits, dim=-1)
    if replay is not None:
        idx = replay.to(logits.device)
    else:
        sel = scores + bias if bias is not None else scores
        if n_group > 1:
            grp = sel.view(-1, n_group, E // n_group).topk(2, dim=-1).values.sum(-1)
            gidx = grp.topk(topk_group, dim=-1).indices
            gmask = torch.zeros_like(grp).scatter_(1, gidx, 1.0)
            sel = sel.masked_fill(gmask[:, :, None].expand(-1, n_group, E // n_group).reshape(-1, E) == 0,
                                  float("-inf"))
        idx = sel.topk(K, dim=-1).indices
    w = scores.gather(-1, idx)
    if norm:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return idx, w * scale


class _Route(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, replay, K, n_group, topk_group, sigmoid, norm, scale):
        T, E = logits.shape
        logits = logits.contiguous()
        idx = torch.empty(T, K, dtype=torch.int64, device=logits.device)
        w = torch.empty(T, K, dtype=torch.float32, device=logits.device)
        LAUNCHES["router"] += 1
        # named copies: a temporary inside the call expression would be released before the asynchronous launch reads it
        bias_f = bias.float().contiguous() if bias is not None else None
        replay_l = replay.to(device=logits.device, dtype=torch.int64).contiguous() if replay is not None else None
        _lib.check(_lib.kernels().gk_router_fwd(
            _lib.ptr(logits), _lib.ptr(bias_f),
            _lib.ptr(replay_l),
            _lib.ptr(idx), _lib.ptr(w), T, E, K, n_group, topk_group, int(sigmoid), int(norm), float(scale),
            _lib.stream_ptr()), "router_fwd")
        ctx.save_for_backward(logits, idx)
        ctx.cfg = (K, int(sigmoid), int(norm), float(scale))
        ctx.mark_non_differentiable(idx)
        return idx, w

    @staticmethod
    def backward(ctx, _g_idx, g_w):
        logits, idx = ctx.saved_tensors
        K, sigmoid, norm, scale = ctx.cfg
        T, E = logits.shape
        dl = torch.empty_like(logits)
        LAUNCHES["router"] += 1
        g_w = g_w.float().contiguous()
        _lib.check(_lib.kernels().gk_router_bwd(_lib.ptr(logits), _lib.ptr(idx), _lib.ptr(g_w),
                                                _lib.ptr(dl), T, E, K, sigmoid, norm, scale, _lib.stream_ptr()),
                   "router_bwd")
        return dl, None, None, None, None, None, None, None, None


def route(logits, bias=None, replay=None, K=2, n_group=1, topk_group=1, sigmoid=False, norm=True, scale=1.0):
    """``logits`` [T, E] fp32 -> ``(idx [T, K] int64, w [T, K] fp32)``; ``w`` is differentiable in ``logits``."""
    E = logits.shape[-1]
    native = (_lib.use_native(logits) and logits.dtype == torch.float32 and E in (32, 64, 128, 256, 512)
              and 1 <= K <= 16 and K <= E and 1 <= n_group <= 8 and E % n_group == 0 and logits.shape[0] > 0
              and hasattr(_lib.kernels(), "gk_router_fwd"))
    if not native:
        return route_ref(logits, bias, replay, K, n_group, topk_group, sigmoid, norm, scale)
    return _Route.apply(logits, bias, replay, K, n_group, topk_group, sigmoid, norm, scale)
