"""Attention front-ends.

* ``flash_attn_varlen`` - training / prefill attention over packed (THD) sequences: causal or full, GQA, sliding
  window, learned per-head sink logit, prefix-K offset.  Forward runs the tcgen05 kernel
  (``csrc/attention_fwd.cu``); backward runs ``csrc/attention_bwd.cu`` when built, else a recompute through the
  PyTorch reference.  Same call contract as ``myfa_varlen_sw_sinks`` (gfused/myfa_varlen_sw_sinks.py:704).
* ``paged_decode`` / ``kv_append_rope`` - rollout decoder (``csrc/paged_attention.cu``).
* ``mla_paged_decode`` - rollout decoder of latent-attention models on the paged latent cache (``csrc/mla_decode.cu``).
* ``attn_varlen_ref`` - the fp32 PyTorch oracle (mirrors tests/test_gfused/test_myfa_varlen_sw_sinks.py:33-98).
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from . import _lib

LAUNCHES = {"attention": 0}


def attn_varlen_ref(q, k, v, cu_q, cu_k, causal=True, window=0, sinks=None, scale=None, return_lse=False):
    """fp32 reference.  q [Tq,Hq,D], k/v [Tk,Hk,D]; key j is visible to query i (indices inside a sequence) when
    ``j <= i + (lk - lq)`` (causal) and ``j > i + (lk - lq) - window`` (window > 0)."""
    Tq, Hq, D = q.shape
    Hk = k.shape[1]
    g = Hq // Hk
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros(Tq, Hq, v.shape[-1], dtype=torch.float32, device=q.device)
    lse = torch.full((Hq, Tq), float("-inf"), dtype=torch.float32, device=q.device)
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for b in range(len(cq) - 1):
        qs, qe, ks, ke = cq[b], cq[b + 1], ck[b], ck[b + 1]
        lq, lk = qe - qs, ke - ks
        if lq == 0:
            continue
        qb = q[qs:qe].float().transpose(0, 1)  # [Hq, lq, D]
        kb = k[ks:ke].float().transpose(0, 1).repeat_interleave(g, 0)
        vb = v[ks:ke].float().transpose(0, 1).repeat_interleave(g, 0)
        s = torch.einsum("hqd,hkd->hqk", qb, kb) * scale
        qi = torch.arange(lq, device=q.device)[:, None] + (lk - lq)
        kj = torch.arange(lk, device=q.device)[None, :]
        mask = torch.ones(lq, lk, dtype=torch.bool, device=q.device)
        if causal:
            mask &= kj <= qi
        if window and window > 0:
            mask &= kj > qi - window
        s = s.masked_fill(~mask[None], float("-inf"))
        if sinks is not None:
            s_aug = torch.cat([s, sinks.float()[:, None, None].expand(Hq, lq, 1)], dim=-1)
            l = torch.logsumexp(s_aug, dim=-1)
        else:
            l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l[..., None])
        p = torch.nan_to_num(p, nan=0.0)
        out[qs:qe] = torch.einsum("hqk,hkd->hqd", p, vb).transpose(0, 1)
        lse[:, qs:qe] = l
    if return_lse:
        return out.to(q.dtype), lse
    return out.to(q.dtype)


def _native_fwd(q, k, v, cu_q, cu_k, max_q, causal, window, sinks, scale):
    Tq, Hq, D = q.shape
    Tk, Hk, _ = k.shape
    Dv = v.shape[-1]
    out = torch.empty(Tq, Hq, Dv, dtype=q.dtype, device=q.device)
    lse = torch.empty(Hq, Tq, dtype=torch.float32, device=q.device)
    B = cu_q.numel() - 1
    strides = (ctypes.c_longlong * 4)(q.stride(0), k.stride(0), v.stride(0), out.stride(0))
    se = (ctypes.c_void_p * 2)(torch.cuda.current_stream().cuda_stream, _lib.err_flag(q.device).data_ptr())
    LAUNCHES["attention"] += 1
    rc = _lib.kernels().gk_attn_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse),
                                    _lib.ptr(cu_q), _lib.ptr(cu_k), _lib.ptr(sinks), B, Tq, Tk, Hq, Hk, D,
                                    int(max_q), int(causal), float(scale), int(window or 0), Dv,
                                    ctypes.cast(strides, ctypes.c_void_p), ctypes.cast(se, ctypes.c_void_p))
    _lib.check(rc, "gk_attn_fwd")
    return out, lse


def _native_ok(q, k, v):
    D, Dv = q.shape[-1], v.shape[-1]
    # equal head dims, or the 192 / 128 geometry of latent attention expanded to per-head keys (forward kernel only)
    return (q.dtype == torch.bfloat16 and _lib.use_native(q) and ((D in (64, 128) and Dv == D) or (D, Dv) == (192, 128))
            and q.stride(2) == 1 and q.stride(1) == D and k.stride(2) == 1 and k.stride(1) == D
            and v.stride(2) == 1 and v.stride(1) == Dv and q.stride(0) % 8 == 0 and k.stride(0) % 8 == 0
            and v.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and k.data_ptr() % 16 == 0
            and v.data_ptr() % 16 == 0)


def _have_native_bwd():
    return getattr(_lib.kernels(), "gk_attn_bwd_dv", None) is not None


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, sinks, cu_q, cu_k, max_q, max_k, causal, window, scale):
        out, lse = _native_fwd(q, k, v, cu_q, cu_k, max_q, causal, window, sinks, scale)
        ctx.save_for_backward(q, k, v, out, lse, sinks if sinks is not None else torch.empty(0), cu_q, cu_k)
        ctx.cfg = (max_q, max_k, causal, window, scale, sinks is not None)
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse, sinks, cu_q, cu_k = ctx.saved_tensors
        max_q, max_k, causal, window, scale, has_sinks = ctx.cfg
        sinks = sinks if has_sinks else None
        from .attention_bwd import attn_bwd
        dq, dk, dv, dsinks = attn_bwd(do.contiguous(), q, k, v, out, lse, sinks, cu_q, cu_k, max_q, max_k, causal,
                                      window, scale)
        return dq, dk, dv, dsinks, None, None, None, None, None, None, None


class _FlashAttnWideKeyFn(torch.autograd.Function):
    """Causal self-attention with 192-wide queries / keys and 128-wide values: forward and backward are the tcgen05
    kernels' 192 / 128 instances.  ``GCORE_WIDE_KEY_BWD=flash`` takes the gradient from the library's flash backward
    on the saved output and log-sum-exp instead (values, output and its gradient zero-padded to the key width, which
    that routine wants equal), ``=recompute`` from a per-sequence recompute through the library's fused attention."""

    @staticmethod
    def forward(ctx, q, k, v, cu, max_s, scale):
        out, lse = _native_fwd(q, k, v, cu, cu, max_s, True, 0, None, scale)
        ctx.save_for_backward(q, k, v, out, lse, cu)
        ctx.cfg = (max_s, scale)
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse, cu = ctx.saved_tensors
        max_s, scale = ctx.cfg
        D, Dv = q.shape[-1], v.shape[-1]
        pad = (0, D - Dv)
        how = os.environ.get("GCORE_WIDE_KEY_BWD", "native")
        if how == "native" and _have_native_bwd():
            from .attention_bwd import attn_bwd
            dq, dk, dv, _ = attn_bwd(do.contiguous(), q, k, v, out, lse, None, cu, cu, max_s, max_s, True, 0, scale)
            return dq, dk, dv, None, None, None
        if how in ("native", "flash"):
            try:
                F = torch.nn.functional
                dq, dk, dvp = torch.ops.aten._flash_attention_backward(
                    F.pad(do, pad).contiguous(), q.contiguous(), k.contiguous(), F.pad(v, pad).contiguous(),
                    F.pad(out, pad).contiguous(), lse.contiguous(), cu, cu, int(max_s), int(max_s), 0.0, True,
                    torch.zeros(2, dtype=torch.int64, device=q.device), torch.empty(0, device=q.device), scale=scale)
                return dq, dk, dvp[..., :Dv].contiguous(), None, None, None
            except (RuntimeError, NotImplementedError, AttributeError):
                pass
        bounds = cu.tolist()
        dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
        for a, b in zip(bounds[:-1], bounds[1:]):
            if b <= a:
                continue
            with torch.enable_grad():
                qs, ks, vs = (t[a:b].detach().requires_grad_(True) for t in (q, k, v))
                o = torch.nn.functional.scaled_dot_product_attention(
                    qs.transpose(0, 1)[None], ks.transpose(0, 1)[None],
                    torch.nn.functional.pad(vs, pad).transpose(0, 1)[None], is_causal=True, scale=scale)
                o = o[0].transpose(0, 1)[..., :Dv]
                gq, gk, gv = torch.autograd.grad(o, (qs, ks, vs), do[a:b])
            dq[a:b], dk[a:b], dv[a:b] = gq, gk, gv
        return dq, dk, dv, None, None, None


def flash_attn_varlen(q, k, v, cu_q, cu_k, max_q, max_k, causal=True, window=0, sinks=None, scale=None):
    """Packed varlen attention; returns ``[Tq, Hq, Dv]``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if _native_ok(q, k, v):
        cu_q = cu_q if cu_q.dtype == torch.int32 else cu_q.to(torch.int32)
        cu_k = cu_k if cu_k.dtype == torch.int32 else cu_k.to(torch.int32)
        needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad or
                                                  (sinks is not None and sinks.requires_grad))
        if needs_grad and v.shape[-1] != q.shape[-1]:
            assert causal and not window and sinks is None, \
                "the wide-key geometry is differentiable for causal self-attention only"
            return _FlashAttnWideKeyFn.apply(q, k, v, cu_q, max_q, scale)
        if needs_grad:
            return _FlashAttnFn.apply(q, k, v, sinks, cu_q, cu_k, max_q, max_k, causal, window, scale)
        return _native_fwd(q, k, v, cu_q, cu_k, max_q, causal, window, sinks, scale)[0]
    if q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and sinks is None and causal \
            and q.shape[0] == k.shape[0]:
        # eager baseline backend on a GPU: the library's fused variable-length attention (with autograd); grouped
        # key / value heads are expanded because the library call takes one head count
        try:
            from torch.nn.attention.varlen import varlen_attn
        except ImportError:
            varlen_attn = None
        if varlen_attn is not None:
            g = q.shape[1] // k.shape[1]
            kk = k.repeat_interleave(g, 1) if g > 1 else k
            vv = v.repeat_interleave(g, 1) if g > 1 else v
            cq = cu_q if cu_q.dtype == torch.int32 else cu_q.to(torch.int32)
            ck = cu_k if cu_k.dtype == torch.int32 else cu_k.to(torch.int32)
            return varlen_attn(q.contiguous(), kk.contiguous(), vv.contiguous(), cq, ck, int(max_q), int(max_k),
                               scale=scale, window_size=(int(window) - 1 if window else -1, 0))
    return attn_varlen_ref(q, k, v, cu_q, cu_k, causal, window, sinks, scale)


# ---------------------------------------------------------------------------------------------- decoder side
def kv_append_rope(qkv, pos, slots, k_cache, v_cache, Hq, Hk, D, theta, rot=None, do_rope=True):
    """RoPE on the q and k parts of ``qkv`` [T, (Hq+2Hk)*D] in place, then k/v rows go to cache slot ``slots[t]``
    (``k_cache``/``v_cache``: [num_blocks, block_size, Hk, D])."""
    T = qkv.shape[0]
    rot = rot or D
    if _lib.use_native(qkv) and qkv.dtype == torch.bfloat16:
        LAUNCHES["attention"] += 1
        _lib.check(_lib.kernels().gk_kv_append_rope(_lib.ptr(qkv), _lib.ptr(pos), _lib.ptr(slots), _lib.ptr(k_cache),
                                                    _lib.ptr(v_cache), T, Hq, Hk, D, rot, int(do_rope), float(theta),
                                                    0, _lib.stream_ptr()), "kv_append_rope")
        return
    from .fused import rope_ref
    x = qkv.view(T, Hq + 2 * Hk, D)
    if do_rope:
        x[:, :Hq + Hk] = rope_ref(x[:, :Hq + Hk], pos, theta, rot)
    kc = k_cache.view(-1, Hk, D)
    vc = v_cache.view(-1, Hk, D)
    valid = slots >= 0
    if qkv.is_cuda:
        # no boolean indexing on a GPU (it synchronises): rows without a slot rewrite the value a live row of the
        # same call writes anyway (or, when the call has no live row, the first slot's current content)
        sl = slots.long()
        first = torch.argmax(valid.to(torch.int8))
        sl = torch.where(valid, sl, sl[first].clamp_min(0))
        src = torch.where(valid, torch.arange(T, device=qkv.device), first)
        any_valid = valid.any()
        knew = torch.where(any_valid, x[src, Hq:Hq + Hk], kc[sl])
        vnew = torch.where(any_valid, x[src, Hq + Hk:], vc[sl])
        kc.index_copy_(0, sl, knew)
        vc.index_copy_(0, sl, vnew)
        return
    kc[slots[valid].long()] = x[valid, Hq:Hq + Hk]
    vc[slots[valid].long()] = x[valid, Hq + Hk:]


_PD_SCRATCH: dict = {}


def paged_decode(q, k_cache, v_cache, block_table, ctx_len, max_ctx, scale=None, window=0, sinks=None, out=None):
    """One-token-per-request attention over the paged cache.  q: [B, Hq, D] (row stride may be a packed QKV row);
    block_table: [B, max_blocks] int32; ctx_len: [B] int32 (tokens in the cache, including the new one)."""
    B, Hq, D = q.shape
    nb, bs, Hk, _ = k_cache.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty(B, Hq, D, dtype=q.dtype, device=q.device)
    if _lib.use_native(q) and q.dtype == torch.bfloat16 and D == 128:
        lib = _lib.kernels()
        need = ctypes.c_longlong()
        lib.gk_paged_decode_scratch(B, Hq, D, int(max_ctx), ctypes.byref(need))
        key = q.device.index
        sc = _PD_SCRATCH.get(key)
        if sc is None or sc.numel() < need.value:
            sc = torch.empty(max(need.value, 1), dtype=torch.float32, device=q.device)
            _PD_SCRATCH[key] = sc
        LAUNCHES["attention"] += 1
        _lib.check(lib.gk_paged_decode(_lib.ptr(q), _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(block_table),
                                       _lib.ptr(ctx_len), _lib.ptr(sinks), _lib.ptr(out), _lib.ptr(sc), B, Hq, Hk, D,
                                       bs, block_table.shape[1], int(max_ctx), float(scale), int(window or 0),
                                       q.stride(0), _lib.stream_ptr()), "paged_decode")
        return out
    g = Hq // Hk
    kc = k_cache.view(-1, Hk, D)
    vc = v_cache.view(-1, Hk, D)
    if q.is_cuda:
        # library path on a GPU (the eager baseline backend): one gather of every request's rows through the block
        # table, then the library's fused attention with a length mask - no host synchronisation, static shapes
        L = min(block_table.shape[1] * bs, (int(max_ctx) + bs - 1) // bs * bs)
        p = torch.arange(L, device=q.device)
        idx = block_table.long()[:, p // bs] * bs + (p % bs)[None, :]
        n = ctx_len.long()[:, None]
        mask = p[None, :] < n
        if window and window > 0:
            mask = mask & (p[None, :] >= n - window)
        kk, vv = kc[idx], vc[idx]                                   # [B, L, Hk, D]
        if sinks is None:
            o = torch.nn.functional.scaled_dot_product_attention(
                q.unsqueeze(2), kk.permute(0, 2, 1, 3), vv.permute(0, 2, 1, 3), attn_mask=mask[:, None, None, :],
                scale=scale, enable_gqa=True)
            out.copy_(torch.nan_to_num(o.squeeze(2)))
            return out
        sc = torch.einsum("bhd,blhd->bhl", q.float(), kk.float().repeat_interleave(g, 2)) * scale
        sc = sc.masked_fill(~mask[:, None, :], float("-inf"))
        lse = torch.logsumexp(torch.cat([sc, sinks.float()[None, :, None].expand(B, Hq, 1)], -1), -1)
        pr = torch.exp(sc - lse[..., None])
        out.copy_(torch.einsum("bhl,blhd->bhd", pr, vv.float().repeat_interleave(g, 2)).to(out.dtype))
        return out
    for b in range(B):
        n = int(ctx_len[b])
        start = max(0, n - window) if window and window > 0 else 0
        toks = torch.arange(start, n, device=q.device)
        slots = block_table[b, toks // bs].long() * bs + toks % bs
        kk = kc[slots].float().repeat_interleave(g, 1)  # [n, Hq, D]
        vv = vc[slots].float().repeat_interleave(g, 1)
        s = torch.einsum("hd,nhd->hn", q[b].float(), kk) * scale
        if sinks is not None:
            l = torch.logsumexp(torch.cat([s, sinks.float()[:, None]], -1), -1)
        else:
            l = torch.logsumexp(s, -1)
        p = torch.exp(s - l[:, None])
        out[b] = torch.einsum("hn,nhd->hd", p, vv).to(out.dtype)
    return out


def paged_decode_append_supported(qkv, Hq, Hk, D, rot) -> bool:
    """True when rotary embedding, cache append and decode attention run as one kernel for these operands."""
    return (_lib.use_native(qkv) and qkv.dtype == torch.bfloat16 and D == 128 and Hq % Hk == 0 and Hq // Hk <= 8
            and 0 < rot <= D and rot % 16 == 0 and os.environ.get("GCORE_FUSED_KV_APPEND", "1") != "0"
            and hasattr(_lib.kernels(), "gk_paged_decode_append"))


def paged_decode_append(qkv, pos, slots, k_cache, v_cache, block_table, ctx_len, max_ctx, Hq, Hk, D, theta, rot=None,
                        scale=None, window=0, sinks=None):
    """``kv_append_rope`` followed by ``paged_decode`` on the packed ``[T, (Hq + 2 Hk) * D]`` rows of the QKV
    projection.  One launch where the tensor-core decode kernel serves the shape (the rotation and the append happen
    inside it: the packed rows are then left unrotated), otherwise the two kernels one after the other."""
    T = qkv.shape[0]
    rot = rot or D
    if paged_decode_append_supported(qkv, Hq, Hk, D, rot):
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
        out = torch.empty(T, Hq, D, dtype=qkv.dtype, device=qkv.device)
        lib = _lib.kernels()
        need = ctypes.c_longlong()
        lib.gk_paged_decode_scratch(T, Hq, D, int(max_ctx), ctypes.byref(need))
        key = qkv.device.index
        sc = _PD_SCRATCH.get(key)
        if sc is None or sc.numel() < need.value:
            sc = torch.empty(max(need.value, 1), dtype=torch.float32, device=qkv.device)
            _PD_SCRATCH[key] = sc
        LAUNCHES["attention"] += 1
        _lib.check(lib.gk_paged_decode_append(_lib.ptr(qkv), _lib.ptr(k_cache), _lib.ptr(v_cache),
                                              _lib.ptr(block_table), _lib.ptr(ctx_len), _lib.ptr(slots),
                                              _lib.ptr(sinks), _lib.ptr(out), _lib.ptr(sc), T, Hq, Hk, D,
                                              k_cache.shape[1], block_table.shape[1], int(max_ctx), float(scale),
                                              int(window or 0), qkv.stride(0), int(rot), float(theta),
                                              _lib.stream_ptr()), "paged_decode_append")
        return out
    kv_append_rope(qkv, pos, slots, k_cache, v_cache, Hq, Hk, D, theta, rot)
    q = qkv.view(T, Hq + 2 * Hk, D)[:, :Hq]
    return paged_decode(q, k_cache, v_cache, block_table, ctx_len, max_ctx, scale=scale, window=window, sinks=sinks)


def mla_decode_supported(q_lat, q_rope) -> bool:
    """True when the latent decode kernel serves these operands (bf16 on a GPU, a built geometry)."""
    if not (_lib.use_native(q_lat) and q_lat.dtype == torch.bfloat16 and q_rope.dtype == torch.bfloat16):
        return False
    lib = _lib.kernels()
    return hasattr(lib, "gk_mla_paged_decode") and bool(lib.gk_mla_decode_supported(q_lat.shape[-1], q_rope.shape[-1]))


def mla_paged_decode_ref(q_lat, q_rope, cache, block_table, ctx_len, scale):
    """fp32 reference of ``mla_paged_decode``: per request, softmax over its cached rows of
    ``q_lat . row[:C] + q_rope . row[C:]``, output = weighted sum of ``row[:C]``; a request without rows gives zeros."""
    B, H, C = q_lat.shape
    bs = cache.shape[1]
    flat = cache.reshape(-1, cache.shape[-1]).float()
    out = torch.zeros(B, H, C, dtype=torch.float32, device=q_lat.device)
    for b in range(B):
        n = int(ctx_len[b])
        if n == 0:
            continue
        toks = torch.arange(n, device=q_lat.device)
        rows = flat[block_table[b, toks // bs].long() * bs + toks % bs]          # [n, C + dr]
        s = (q_lat[b].float() @ rows[:, :C].T + q_rope[b].float() @ rows[:, C:].T) * scale
        out[b] = torch.softmax(s, -1) @ rows[:, :C]
    return out


def mla_paged_decode(q_lat, q_rope, cache, block_table, ctx_len, max_ctx, scale, out=None):
    """One query token per request of absorbed multi-head latent attention.  q_lat: [B, H, C] (query times the key
    up-projection), q_rope: [B, H, dr], cache: [blocks, block_size, C + dr] latent rows shared by all heads,
    block_table: [B, max_blocks] int32, ctx_len: [B] int32.  Returns [B, H, C] in q_lat's dtype (``out`` may be any
    strided view whose last dimension is contiguous: the kernel writes through batch / head strides)."""
    B, H, C = q_lat.shape
    dr = q_rope.shape[-1]
    if out is None:
        out = torch.empty(B, H, C, dtype=q_lat.dtype, device=q_lat.device)
    if not mla_decode_supported(q_lat, q_rope):
        if q_lat.is_cuda and not _lib.force_eager() and q_lat.dtype == torch.bfloat16:
            raise RuntimeError(f"mla_paged_decode: no kernel for kv_lora_rank={C}, rope dim={dr}")
        out.copy_(mla_paged_decode_ref(q_lat, q_rope, cache, block_table, ctx_len, scale).to(out.dtype))
        return out
    assert q_lat.stride(2) == 1 and q_rope.stride(2) == 1 and out.stride(2) == 1 and cache.is_contiguous()
    assert cache.dtype == torch.bfloat16 and cache.shape[-1] == C + dr
    lib = _lib.kernels()
    need = ctypes.c_longlong()
    lib.gk_mla_decode_scratch(B, H, C, int(max_ctx), ctypes.byref(need))
    key = ("mla", q_lat.device.index)
    sc = _PD_SCRATCH.get(key)
    if sc is None or sc.numel() < need.value:
        sc = torch.empty(max(need.value, 1), dtype=torch.float32, device=q_lat.device)
        _PD_SCRATCH[key] = sc
    LAUNCHES["attention"] += 1
    _lib.check(lib.gk_mla_paged_decode(_lib.ptr(q_lat), q_lat.stride(0), q_lat.stride(1), _lib.ptr(q_rope),
                                       q_rope.stride(0), q_rope.stride(1), _lib.ptr(cache), _lib.ptr(block_table),
                                       _lib.ptr(ctx_len), _lib.ptr(out), out.stride(0), out.stride(1), _lib.ptr(sc),
                                       B, H, C, dr, cache.shape[1], block_table.shape[1], int(max_ctx), float(scale),
                                       _lib.stream_ptr()), "mla_paged_decode")
    return out


class _FlashAttnPackedFn(torch.autograd.Function):
    """Attention over a packed ``[T, hq + 2*hk, D]`` buffer (the QKV GEMM output): one autograd input, so the
    backward returns a single packed gradient instead of three strided view gradients."""

    @staticmethod
    def forward(ctx, qkv, sinks, cu, max_s, hq, hk, causal, window, scale):
        q, k, v = qkv[:, :hq], qkv[:, hq:hq + hk], qkv[:, hq + hk:]
        out, lse = _native_fwd(q, k, v, cu, cu, max_s, causal, window, sinks, scale)
        ctx.save_for_backward(qkv, out, lse, sinks if sinks is not None else torch.empty(0), cu)
        ctx.cfg = (max_s, hq, hk, causal, window, scale, sinks is not None)
        return out

    @staticmethod
    def backward(ctx, do):
        qkv, out, lse, sinks, cu = ctx.saved_tensors
        max_s, hq, hk, causal, window, scale, has_sinks = ctx.cfg
        q, k, v = qkv[:, :hq], qkv[:, hq:hq + hk], qkv[:, hq + hk:]
        from .attention_bwd import attn_bwd
        dq, dk, dv, ds = attn_bwd(do.contiguous(), q, k, v, out, lse, sinks if has_sinks else None, cu, cu, max_s,
                                  max_s, causal, window, scale)
        return torch.cat([dq, dk, dv], dim=1), ds, None, None, None, None, None, None, None


def flash_attn_qkvpacked(qkv, hq, hk, cu_seqlens, max_seqlen, causal=True, window=0, sinks=None, scale=None):
    """Self-attention where q, k, v are head ranges of one packed ``[T, hq + 2*hk, D]`` tensor."""
    scale = scale if scale is not None else 1.0 / math.sqrt(qkv.shape[-1])
    q, k, v = qkv[:, :hq], qkv[:, hq:hq + hk], qkv[:, hq + hk:]
    if _native_ok(q, k, v):
        cu = cu_seqlens if cu_seqlens.dtype == torch.int32 else cu_seqlens.to(torch.int32)
        if torch.is_grad_enabled() and qkv.requires_grad:
            return _FlashAttnPackedFn.apply(qkv, sinks, cu, max_seqlen, hq, hk, causal, window, scale)
        return _native_fwd(q, k, v, cu, cu, max_seqlen, causal, window, sinks, scale)[0]
    return attn_varlen_ref(q, k, v, cu_seqlens, cu_seqlens, causal, window, sinks, scale)
