"""Ops of the DeepSeek-V4-class attention stack: lightning-indexer scores, top-k sparse multi-query attention with a
shared key / value row and per-head sinks, Walsh-Hadamard rotation.  Native kernels in ``csrc/dsv4.cu``; the PyTorch
definitions below are the CPU path and the oracles of the kernel tests.

Semantics follow the reference's kernels: indexer ``sum_h w_h relu(q_h . k)`` with per-row key bounds
(gpatch_v4/models/deepseek_v4/kernel/tilelang_indexer_fwd.py:21-240), sparse attention over gathered rows with the
sink in the softmax denominator (kernel/tilelang_sparse_mla_fwd.py:25-155, eager oracle kernel/eager_topk_attn.py),
``rotate_activation`` = Hadamard transform scaled by ``n ** -0.5`` (kernel/hadamard_transform.py:9-19).
"""
from __future__ import annotations

import math

import torch

from . import _lib

LAUNCHES = {"dsv4": 0}


# ---------------------------------------------------------------------------------------------------- indexer
def indexer_scores_ref(q, k, w, ks, ke, scale):
    """q [S, H, D], k [T, D], w [S, H] fp32, ks / ke [S] -> [S, T] fp32 with -inf outside [ks, ke)."""
    s = torch.einsum("shd,td->sht", q.float(), k.float())
    out = (torch.relu(s) * w.float()[:, :, None]).sum(1) * scale
    pos = torch.arange(k.shape[0], device=q.device)[None, :]
    return out.masked_fill((pos < ks[:, None]) | (pos >= ke[:, None]), float("-inf"))


def indexer_scores(q, k, w, ks, ke, scale):
    """Forward only (its consumer is a top-k; gradients flow through ``indexer_selected_scores``)."""
    S, H, D = q.shape
    T = k.shape[0]
    if not (_lib.use_native(q) and q.dtype == torch.bfloat16 and D % 2 == 0 and D <= 256 and H <= 128):
        return indexer_scores_ref(q, k, w, ks, ke, scale)
    out = torch.empty(S, T, dtype=torch.float32, device=q.device)
    LAUNCHES["dsv4"] += 1
    # converted / compacted copies get names: a temporary inside the call expression is released as soon as its pointer
    # has been taken, and the next temporary may be given the same block before the asynchronous kernel has read it
    q, k, w, ks, ke = q.contiguous(), k.contiguous(), w.float().contiguous(), ks.int().contiguous(), ke.int().contiguous()
    _lib.check(_lib.kernels().gk_dsv4_indexer_fwd(_lib.ptr(q), _lib.ptr(k),
                                                  _lib.ptr(w), _lib.ptr(ks),
                                                  _lib.ptr(ke), _lib.ptr(out), S, T, H, D,
                                                  float(scale), _lib.stream_ptr()), "dsv4_indexer_fwd")
    return out


def _selected_ref(q, k, w, idx, scale):
    valid = idx >= 0
    rows = k.float()[idx.clamp_min(0).long()]                       # [S, K, D]
    s = torch.einsum("shd,skd->shk", q.float(), rows)
    out = (torch.relu(s) * w.float()[:, :, None]).sum(1) * scale
    return torch.where(valid, out, torch.zeros_like(out))


class _IndexerSelected(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, w, idx, scale):
        ctx.save_for_backward(q, k, w, idx)
        ctx.scale = scale
        with torch.no_grad():
            return _selected_ref(q, k, w, idx, scale)

    @staticmethod
    def backward(ctx, ds):
        q, k, w, idx = ctx.saved_tensors
        S, H, D = q.shape
        T, K = k.shape[0], idx.shape[1]
        dq = torch.empty(S, H, D, dtype=torch.float32, device=q.device)
        dk = torch.zeros(T, D, dtype=torch.float32, device=q.device)
        dw = torch.empty(S, H, dtype=torch.float32, device=q.device)
        LAUNCHES["dsv4"] += 1
        qc, kc, wc, ic, dsc = (q.contiguous(), k.contiguous(), w.float().contiguous(), idx.int().contiguous(),
                               ds.float().contiguous())   # named: they must outlive the asynchronous launch
        _lib.check(_lib.kernels().gk_dsv4_indexer_bwd(
            _lib.ptr(qc), _lib.ptr(kc), _lib.ptr(wc),
            _lib.ptr(ic), _lib.ptr(dsc), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dw),
            S, T, H, D, K, float(ctx.scale), _lib.stream_ptr()), "dsv4_indexer_bwd")
        return dq.to(q.dtype), dk.to(k.dtype), dw.to(w.dtype), None, None


def indexer_selected_scores(q, k, w, idx, scale):
    """Scores of the selected entries ``idx`` [S, K] (-1 = none -> 0), differentiable in q, k and w: the path the
    indexer's training signal takes (the reference's backward runs on the top-k only,
    kernel/tilelang_indexer_bwd.py:21-143)."""
    S, H, D = q.shape
    native = (_lib.use_native(q) and q.dtype == torch.bfloat16 and D <= 256 and H <= 128
              and (H * D * 6 + D * 2 + H * 4) <= 200 * 1024)
    if native and torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or w.requires_grad):
        return _IndexerSelected.apply(q, k, w, idx, scale)
    return _selected_ref(q, k, w, idx, scale)


# ---------------------------------------------------------------------------------------------------- sparse MQA
def sparse_mqa_ref(q, kv, sinks, idx, scale):
    """q [S, H, D], kv [T, D], sinks [H] | None, idx [S, K] (-1 = none) -> (out [S, H, D], lse [S, H])."""
    valid = idx >= 0
    rows = kv.float()[idx.clamp_min(0).long()]                      # [S, K, D]
    s = torch.einsum("shd,skd->shk", q.float(), rows) * scale
    s = s.masked_fill(~valid[:, None, :], float("-inf"))
    if sinks is not None:
        lse = torch.logsumexp(torch.cat([s, sinks.float()[None, :, None].expand(s.shape[0], -1, 1)], -1), -1)
    else:
        lse = torch.logsumexp(s, -1)
    p = torch.exp(s - lse[..., None])
    p = torch.where(torch.isfinite(lse)[..., None], p, torch.zeros_like(p))
    return torch.einsum("shk,skd->shd", p, rows).to(q.dtype), lse


class _SparseMqa(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, kv, sinks, idx, scale):
        S, H, D = q.shape
        T, K = kv.shape[0], idx.shape[1]
        q, kv, idx = q.contiguous(), kv.contiguous(), idx.int().contiguous()
        out = torch.empty_like(q)
        lse = torch.empty(S, H, dtype=torch.float32, device=q.device)
        sk = sinks.float().contiguous() if sinks is not None else None
        LAUNCHES["dsv4"] += 1
        _lib.check(_lib.kernels().gk_dsv4_sparse_mqa_fwd(_lib.ptr(q), _lib.ptr(kv), _lib.ptr(sk), _lib.ptr(idx),
                                                         _lib.ptr(out), _lib.ptr(lse), S, T, H, D, K, float(scale),
                                                         _lib.stream_ptr()), "dsv4_sparse_mqa_fwd")
        ctx.save_for_backward(q, kv, sk if sk is not None else torch.empty(0, device=q.device), idx, out, lse)
        ctx.has_sinks, ctx.scale, ctx.sink_dtype = sinks is not None, scale, (sinks.dtype if sinks is not None else None)
        return out

    @staticmethod
    def backward(ctx, do):
        q, kv, sk, idx, out, lse = ctx.saved_tensors
        S, H, D = q.shape
        T, K = kv.shape[0], idx.shape[1]
        dq = torch.empty(S, H, D, dtype=torch.float32, device=q.device)
        dkv = torch.zeros(T, D, dtype=torch.float32, device=q.device)
        dsk = torch.zeros(H, dtype=torch.float32, device=q.device)
        LAUNCHES["dsv4"] += 1
        do = do.contiguous()
        _lib.check(_lib.kernels().gk_dsv4_sparse_mqa_bwd(
            _lib.ptr(q), _lib.ptr(kv), _lib.ptr(sk if ctx.has_sinks else None), _lib.ptr(idx), _lib.ptr(out),
            _lib.ptr(lse), _lib.ptr(do), _lib.ptr(dq), _lib.ptr(dkv), _lib.ptr(dsk), S, T, H, D, K,
            float(ctx.scale), _lib.stream_ptr()), "dsv4_sparse_mqa_bwd")
        return dq.to(q.dtype), dkv.to(kv.dtype), (dsk.to(ctx.sink_dtype) if ctx.has_sinks else None), None, None


def sparse_mqa(q, kv, sinks, idx, scale=None):
    """Attention of every query over ITS OWN list of rows of the shared key / value matrix ``kv``."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _lib.use_native(q) and q.dtype == torch.bfloat16 and D in (32, 64, 128, 256, 512):
        return _SparseMqa.apply(q, kv, sinks, idx, scale)
    return sparse_mqa_ref(q, kv, sinks, idx, scale)[0]


# ---------------------------------------------------------------------------------------------------- Hadamard
def hadamard_ref(x):
    n = x.shape[-1]
    assert n & (n - 1) == 0, "the Hadamard transform needs a power-of-two width"
    y = x.float().reshape(-1, n)
    h = 1
    while h < n:
        y = y.view(-1, n // (2 * h), 2, h)
        y = torch.stack([y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]], 2).reshape(-1, n)
        h *= 2
    return (y * n ** -0.5).reshape(x.shape).to(x.dtype)


class _Hadamard(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _hadamard_native(x)

    @staticmethod
    def backward(ctx, g):
        return _hadamard_native(g)   # the scaled transform is symmetric and orthogonal


def _hadamard_native(x):
    n = x.shape[-1]
    x2 = x.contiguous().view(-1, n)
    y = torch.empty_like(x2)
    LAUNCHES["dsv4"] += 1
    _lib.check(_lib.kernels().gk_hadamard(_lib.ptr(x2), _lib.ptr(y), x2.shape[0], n, _lib.stream_ptr()), "hadamard")
    return y.view(x.shape)


def rotate_activation(x):
    """``H_n x / sqrt(n)`` along the last dimension (spreads outliers before low-precision quantisation)."""
    n = x.shape[-1]
    if _lib.use_native(x) and x.dtype == torch.bfloat16 and 2 <= n <= 4096 and n & (n - 1) == 0:
        return _Hadamard.apply(x)
    return hadamard_ref(x)
