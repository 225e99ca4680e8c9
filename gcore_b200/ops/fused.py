"""Autograd wrappers for the bandwidth-bound block kernels (``csrc/elementwise.cu``): RMSNorm with fused residual
add, RoPE, SwiGLU.  Each has a plain PyTorch implementation used on CPU and as the test oracle."""
from __future__ import annotations

import torch

from . import _lib

LAUNCHES = {"elementwise": 0}


# ------------------------------------------------------------------------------------------------ RMSNorm
def rmsnorm_ref(x, w, eps, residual=None):
    if residual is not None:
        x = (x.float() + residual.float()).to(x.dtype)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype), x


class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual, eps):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        T = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        res_out = None
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, H)
            res_out = torch.empty_like(x2)
        LAUNCHES["elementwise"] += 1
        _lib.check(_lib.kernels().gk_rmsnorm_fwd(_lib.ptr(x2), _lib.ptr(r2), _lib.ptr(w), _lib.ptr(y),
                                                 _lib.ptr(res_out), _lib.ptr(rstd), T, H, float(eps),
                                                 _lib.stream_ptr()), "rmsnorm_fwd")
        normed_in = res_out if residual is not None else x2
        ctx.save_for_backward(normed_in, w, rstd)
        ctx.shape = x.shape
        ctx.has_res = residual is not None
        if residual is not None:
            return y.reshape(x.shape), res_out.reshape(x.shape)
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, gy, gres=None):
        xin, w, rstd = ctx.saved_tensors
        T, H = xin.shape
        lib = _lib.kernels()
        gy2 = gy.reshape(T, H).contiguous()
        gres2 = gres.reshape(T, H).contiguous() if gres is not None else None
        dx = torch.empty_like(xin)
        parts = lib.gk_rmsnorm_bwd_parts(T)
        partial = torch.empty(parts * H, dtype=torch.float32, device=xin.device)
        dw = torch.empty(H, dtype=torch.float32, device=xin.device)
        LAUNCHES["elementwise"] += 2
        _lib.check(lib.gk_rmsnorm_bwd(_lib.ptr(gy2), _lib.ptr(xin), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(gres2),
                                      _lib.ptr(dx), _lib.ptr(partial), _lib.ptr(dw), 0, T, H, _lib.stream_ptr()),
                   "rmsnorm_bwd")
        dx = dx.reshape(ctx.shape)
        return dx, dw.to(w.dtype), (dx if ctx.has_res else None), None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, residual: torch.Tensor | None = None):
    """Returns ``(norm(x + residual) * w, x + residual)``; with ``residual=None`` the second value is ``x``."""
    if x.dtype == torch.bfloat16 and _lib.use_native(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        if not x.is_contiguous():
            x = x.contiguous()
        if residual is not None and not residual.is_contiguous():
            residual = residual.contiguous()
        if residual is None:
            return _RmsNormFn.apply(x, w, None, eps), x
        return _RmsNormFn.apply(x, w, residual, eps)
    return rmsnorm_ref(x, w, eps, residual)


# ------------------------------------------------------------------------------------------------ RoPE
def mrope_tables(pos3: torch.Tensor, theta: float, rot: int, sections, interleaved_sections: bool = True):
    """Multi-axis rotary tables.  ``pos3`` [T, 3] = (temporal, height, width) index of every token; frequency ``i``
    of the ``rot / 2`` frequencies takes its angle from one of the three axes: chunked (``sections = (t, h, w)``
    consecutive frequencies per axis, Qwen2-VL) or interleaved (frequency ``i`` uses axis ``i % 3`` while that axis
    still has budget, the rest temporal, Qwen3-VL; gpatch_v4/extended_model/qwen3_vl.py).  Returns ``(cos, sin)``
    fp32 ``[T, rot / 2]``, accepted wherever a rotary op takes position ids."""
    half = rot // 2
    assert sum(sections) == half, f"mrope sections {sections} must sum to {half}"
    inv = theta ** (-torch.arange(0, half, device=pos3.device, dtype=torch.float32) * 2.0 / rot)
    axis = torch.zeros(half, dtype=torch.long, device=pos3.device)
    if interleaved_sections:
        idx = torch.arange(half, device=pos3.device)
        for a in (1, 2):
            axis[(idx % 3 == a) & (idx < 3 * sections[a])] = a
    else:
        o = 0
        for a, n in enumerate(sections):
            axis[o:o + n] = a
            o += n
    ang = pos3.float()[:, axis] * inv[None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


def rope_ref(x, pos, theta, rot=None, interleaved=False, backward=False):
    """x: [T, nheads, D]; rotate-half pairing (i, i + rot/2) unless ``interleaved``.  ``pos``: position ids [T] or a
    ``(cos, sin)`` pair of tables [T, rot / 2] (see ``mrope_tables``)."""
    D = x.shape[-1]
    rot = rot or D
    half = rot // 2
    if isinstance(pos, tuple):
        c, s = pos[0][:, None, :], pos[1][:, None, :]
    else:
        inv = theta ** (-torch.arange(0, half, device=x.device, dtype=torch.float32) * 2.0 / rot)
        ang = pos.float()[:, None] * inv[None, :]
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    if backward:
        s = -s
    xf = x.float()
    xr = xf[..., :rot]
    if interleaved:
        a, b = xr[..., 0::2], xr[..., 1::2]
        o = torch.stack([a * c - b * s, b * c + a * s], dim=-1).flatten(-2)
    else:
        a, b = xr[..., :half], xr[..., half:]
        o = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
    return torch.cat([o, xf[..., rot:]], dim=-1).to(x.dtype)


def rope_inplace(x: torch.Tensor, pos: torch.Tensor, theta: float, rot: int | None = None,
                 interleaved: bool = False, backward: bool = False):
    """In-place RoPE on ``x`` [T, nheads, D]; ``x`` may be a slice of a packed QKV buffer (any token stride)."""
    T, nh, D = x.shape
    rot = rot or D
    if x.dtype == torch.bfloat16 and _lib.use_native(x) and x.stride(2) == 1 and x.stride(1) == D:
        if isinstance(pos, tuple):
            LAUNCHES["elementwise"] += 1
            _lib.check(_lib.kernels().gk_rope_table(_lib.ptr(x), _lib.ptr(pos[0]), _lib.ptr(pos[1]), T, nh, D, rot,
                                                    x.stride(0), int(backward), int(interleaved), _lib.stream_ptr()),
                       "rope_table")
            return x
        p32 = pos if pos.dtype == torch.int32 else pos.to(torch.int32)
        LAUNCHES["elementwise"] += 1
        _lib.check(_lib.kernels().gk_rope(_lib.ptr(x), _lib.ptr(p32), T, nh, D, rot, x.stride(0), float(theta),
                                          int(backward), int(interleaved), _lib.stream_ptr()), "rope")
        return x
    x.copy_(rope_ref(x, pos, theta, rot, interleaved, backward))
    return x


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos, theta, rot, interleaved):
        ctx.pos = pos   # position ids or (cos, sin) tables: never differentiated
        ctx.args = (theta, rot, interleaved)
        return rope_inplace(x.clone(), pos, theta, rot, interleaved, False)

    @staticmethod
    def backward(ctx, g):
        pos = ctx.pos
        theta, rot, interleaved = ctx.args
        return rope_inplace(g.clone(), pos, theta, rot, interleaved, True), None, None, None, None


def rope(x, pos, theta, rot=None, interleaved=False):
    return _RopeFn.apply(x, pos, theta, rot, interleaved)


# ------------------------------------------------------------------------------------------------ SwiGLU
def qk_headnorm_(qkv: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, Hq: int, Hk: int, D: int, eps: float):
    """In-place per-head RMSNorm of the query and key heads of packed ``[T, (Hq + 2 Hk) * D]`` rows (inference: no
    autograd).  One kernel on a GPU; the same arithmetic through ``rmsnorm`` elsewhere."""
    T = qkv.shape[0]
    if (qkv.dtype == torch.bfloat16 and _lib.use_native(qkv) and D % 8 == 0 and D <= 256 and qkv.stride(1) == 1
            and wq.dtype == torch.bfloat16 and hasattr(_lib.kernels(), "gk_qk_headnorm")):
        LAUNCHES["elementwise"] += 1
        _lib.check(_lib.kernels().gk_qk_headnorm(_lib.ptr(qkv), _lib.ptr(wq), _lib.ptr(wk), T, Hq, Hk, D,
                                                 qkv.stride(0), float(eps), _lib.stream_ptr()), "qk_headnorm")
        return qkv
    v = qkv.view(T, Hq + 2 * Hk, D)
    v[:, :Hq] = rmsnorm(v[:, :Hq].reshape(-1, D), wq, eps)[0].view(T, Hq, D)
    v[:, Hq:Hq + Hk] = rmsnorm(v[:, Hq:Hq + Hk].reshape(-1, D), wk, eps)[0].view(T, Hk, D)
    return qkv


def swiglu_ref(x):
    g, u = x.float().chunk(2, dim=-1)
    return (torch.nn.functional.silu(g) * u).to(x.dtype)


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        F = x.shape[-1] // 2
        x2 = x.reshape(-1, 2 * F)
        out = torch.empty(x2.shape[0], F, dtype=x.dtype, device=x.device)
        LAUNCHES["elementwise"] += 1
        _lib.check(_lib.kernels().gk_swiglu_fwd(_lib.ptr(x2), _lib.ptr(out), x2.shape[0], F, _lib.stream_ptr()),
                   "swiglu_fwd")
        ctx.save_for_backward(x2)
        ctx.shape = x.shape
        return out.reshape(*x.shape[:-1], F)

    @staticmethod
    def backward(ctx, g):
        (x2,) = ctx.saved_tensors
        F = x2.shape[1] // 2
        g2 = g.reshape(-1, F).contiguous()
        din = torch.empty_like(x2)
        LAUNCHES["elementwise"] += 1
        _lib.check(_lib.kernels().gk_swiglu_bwd(_lib.ptr(g2), _lib.ptr(x2), _lib.ptr(din), x2.shape[0], F,
                                                _lib.stream_ptr()), "swiglu_bwd")
        return din.reshape(ctx.shape)


def swiglu(x: torch.Tensor, n_rows: torch.Tensor = None) -> torch.Tensor:
    """``silu(x[..., :F]) * x[..., F:]`` for ``x = [gate | up]``.  ``n_rows`` (one int32 on the device, inference only):
    rows of the 2-D ``x`` at or beyond it are not computed and their output is undefined - for expert-sorted buffers
    that are sized for the worst case and carry the count of rows in use on the device."""
    if x.dtype == torch.bfloat16 and _lib.use_native(x) and (x.shape[-1] // 2) % 8 == 0:
        if not x.is_contiguous():
            x = x.contiguous()
        if n_rows is not None and x.dim() == 2 and not (torch.is_grad_enabled() and x.requires_grad) \
                and n_rows.dtype == torch.int32 and hasattr(_lib.kernels(), "gk_swiglu_fwd_rows"):
            F = x.shape[1] // 2
            out = torch.empty(x.shape[0], F, dtype=x.dtype, device=x.device)
            LAUNCHES["elementwise"] += 1
            _lib.check(_lib.kernels().gk_swiglu_fwd_rows(_lib.ptr(x), _lib.ptr(out), x.shape[0], F, _lib.ptr(n_rows),
                                                         _lib.stream_ptr()), "swiglu_fwd_rows")
            return out
        return _SwigluFn.apply(x)
    return swiglu_ref(x)
