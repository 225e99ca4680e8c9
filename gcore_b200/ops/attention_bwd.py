"""Backward of ``flash_attn_varlen``.

Uses the native dQ / dK,dV kernels (``gk_attn_bwd`` in ``csrc/attention_bwd.cu``) when the library exports them;
otherwise recomputes the forward per sequence in PyTorch and differentiates it (exact same masking rules, fp32
softmax), which keeps every feature (window, sinks, prefix offset) trainable while the native kernel is absent.
Gradient definitions follow gfused/myfa_varlen_sw_sinks.py:197-451 (delta pre-pass, dsink = -exp(sink - lse)*delta).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def _recompute_bwd(do, q, k, v, sinks, cu_q, cu_k, causal, window, scale):
    from .attention import attn_varlen_ref
    with torch.enable_grad():
        qq = q.detach().requires_grad_(True)
        kk = k.detach().requires_grad_(True)
        vv = v.detach().requires_grad_(True)
        ss = sinks.detach().float().requires_grad_(True) if sinks is not None else None
        cq, ck = cu_q.tolist(), cu_k.tolist()
        plain = (not window) and ss is None and causal
        if plain and q.is_cuda:
            # memory-efficient interim path for the common case (library SDPA per sequence)
            outs = []
            for b in range(len(cq) - 1):
                qb = qq[cq[b]:cq[b + 1]].transpose(0, 1)[None]
                kb = kk[ck[b]:ck[b + 1]].transpose(0, 1)[None]
                vb = vv[ck[b]:ck[b + 1]].transpose(0, 1)[None]
                if qb.shape[2] == kb.shape[2]:
                    ob = torch.nn.functional.scaled_dot_product_attention(qb, kb, vb, is_causal=True, scale=scale,
                                                                          enable_gqa=True)
                else:
                    lq, lk = qb.shape[2], kb.shape[2]
                    m = torch.ones(lq, lk, dtype=torch.bool, device=q.device).tril(lk - lq)
                    ob = torch.nn.functional.scaled_dot_product_attention(qb, kb, vb, attn_mask=m, scale=scale,
                                                                          enable_gqa=True)
                outs.append(ob[0].transpose(0, 1))
            out = torch.cat(outs, 0)
        else:
            out = attn_varlen_ref(qq, kk, vv, cu_q, cu_k, causal, window, ss, scale)
        ins = [qq, kk, vv] + ([ss] if ss is not None else [])
        grads = torch.autograd.grad(out, ins, do)
    dq, dk, dv = grads[:3]
    ds = grads[3].to(sinks.dtype) if sinks is not None else None
    return dq, dk, dv, ds


def attn_bwd(do, q, k, v, out, lse, sinks, cu_q, cu_k, max_q, max_k, causal, window, scale):
    lib = _lib.kernels() if _lib.use_native(q) else None
    fn = getattr(lib, "gk_attn_bwd_dv", None) if lib is not None else None
    if fn is None:
        return _recompute_bwd(do, q, k, v, sinks, cu_q, cu_k, causal, window, scale)
    Tq, Hq, D = q.shape
    Tk, Hk, _ = k.shape
    Dv = v.shape[-1]       # equal to D, or 128 beside 192-wide queries / keys (expanded latent attention)
    B = cu_q.numel() - 1
    g = Hq // Hk
    dq = torch.empty_like(q)
    # per-query-head dK/dV, reduced over the GQA group afterwards (deterministic, no atomics)
    dk_h = torch.empty(Tk, Hq, D, dtype=q.dtype, device=q.device)
    dv_h = torch.empty(Tk, Hq, Dv, dtype=q.dtype, device=q.device)
    delta = torch.empty(Hq, Tq, dtype=torch.float32, device=q.device)
    strides = (ctypes.c_longlong * 4)(q.stride(0), k.stride(0), v.stride(0), out.stride(0))
    se = (ctypes.c_void_p * 2)(torch.cuda.current_stream().cuda_stream, _lib.err_flag(q.device).data_ptr())
    rc = fn(_lib.ptr(do), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(delta),
            _lib.ptr(dq), _lib.ptr(dk_h), _lib.ptr(dv_h), _lib.ptr(cu_q), _lib.ptr(cu_k), B, Tq, Tk, Hq, Hk, D, Dv,
            int(max_q), int(max_k), float(scale), int(causal), int(window or 0),
            ctypes.cast(strides, ctypes.c_void_p), ctypes.cast(se, ctypes.c_void_p))
    _lib.check(rc, "gk_attn_bwd")
    if g == 1:
        dk, dv = dk_h, dv_h
    else:
        dk = dk_h.view(Tk, Hk, g, D).float().sum(2).to(q.dtype)
        dv = dv_h.view(Tk, Hk, g, Dv).float().sum(2).to(q.dtype)
    ds = None
    if sinks is not None:
        # d sink_h = -sum_t exp(sink_h - lse[h, t]) * delta[h, t]   (rows without any visible key carry lse = -max)
        ok = lse > -1e30
        wgt = torch.where(ok, torch.exp(sinks.float()[:, None] - torch.where(ok, lse, torch.zeros_like(lse))),
                          torch.zeros_like(lse))
        ds = (-(wgt * delta).sum(1)).to(sinks.dtype)
    return dq, dk, dv, ds
