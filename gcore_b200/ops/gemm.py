"""bf16 GEMM front-end for the tcgen05 kernel (``csrc/gemm_tcgen05.cu``) and the autograd ``linear`` built on it.

Layout vocabulary: the kernel computes ``C[M,N] = sum_k A[m,k] * B[n,k]``.  An operand is *K-major* when the
contraction index is its contiguous (last) dimension and *MN-major* when it is its first dimension.  A linear
layer ``y = x W^T`` therefore uses (K,K) in forward, (K,MN) for dgrad ``dy W`` and (MN,MN) for wgrad ``dy^T x``;
no operand is ever transposed in memory.

On CPU tensors, or with ``GCORE_B200_FORCE_EAGER=1``, the same functions run plain PyTorch matmuls: that path is
the numerical oracle of the tests and the ``nccl_eager`` baseline backend.
"""
from __future__ import annotations

import ctypes

import math
import os

import torch

from . import _lib

_SCRATCH: dict = {}
LAUNCHES = {"gemm": 0}


def _scratch(device, ws_floats: int, counters: int):
    key = (device.index,)
    ws, cnt = _SCRATCH.get(key, (None, None))
    if ws is None or ws.numel() < ws_floats:
        ws = torch.empty(max(ws_floats, 1 << 20), dtype=torch.float32, device=device)
    if cnt is None or cnt.numel() < counters:
        cnt = torch.zeros(max(counters, 4096), dtype=torch.int32, device=device)
    _SCRATCH[key] = (ws, cnt)
    return ws, cnt


def _pick_bn(n: int, m: int = 0, b_mn: bool = False) -> int:
    """Tile width: the widest tile the output allows (most reuse per byte of L2 traffic)."""
    if n < 192:
        if n > 64:
            return 128
        if n > 32:
            return 64
        return 32
    return 256  # 192 / 224 wide tiles exist in the kernel but did not pay off on B200 (the kernel is L2-bound)


WIDE = {"enabled": os.environ.get("GCORE_WIDE_GEMM", "1") != "0", "gain": 1.05,
        "tail_split": os.environ.get("GCORE_WIDE_TAIL_SPLIT", "1") != "0"}


def _use_wide(M: int, N: int, K: int) -> bool:
    """256 x 256 tiles move 17 % less shared-memory traffic per FLOP than 128 x 256 ones (the limiter at training
    shapes) but quantise worse over 148 SMs: take them when the wave efficiency they lose is less than what they gain."""
    if not WIDE["enabled"] or M < 1024 or N < 512 or K < 256:
        return False
    nt = (N + 255) // 256
    tw = ((M + 255) // 256) * nt
    tg = ((M + 127) // 128) * nt
    eff_w = tw / _wide_waves(tw, (K + 63) // 64) / 148
    eff_g = tg / (((tg + 147) // 148) * 148)
    return eff_w * WIDE["gain"] > eff_g


def _wide_waves(tiles: int, kblocks: int) -> float:
    """Waves the 256 x 256 kernel needs on 148 SMs.  A partial last wave of at most half the SMs is cut along K into
    slices (the kernel's tail split): it then costs the share of a tile one slice is, plus the partial-sum pass."""
    full, tail = divmod(tiles, 148)
    if tail == 0:
        return float(full)
    if WIDE["tail_split"] and tail * 2 <= 148 and kblocks >= 8:
        ks = min(148 // tail, kblocks // 4, 4)
        if ks >= 2:
            per = -(-kblocks // ks)
            return full + per / kblocks + 0.08
    return float(full + 1)


# The CTA-pair kernel is numerically verified but measures 5-10 % behind the one-CTA 256 x 256 kernel on the training
# shapes (forward 0.207 vs 0.188 ms on [8192 x 3584] x [4608 x 3584]^T, 1.65 vs 1.53 ms on the 37888-wide MLP shape),
# so it is opt-in: GCORE_GEMM_2CTA=1.
TWO_CTA = {"enabled": os.environ.get("GCORE_GEMM_2CTA", "0") == "1", "min_tiles": 37}


def _use_two_cta(M: int, N: int, K: int) -> bool:
    """The pair kernel works on 256 x 256 tiles over 74 SM pairs: problems with too few tiles to fill half of them
    stay on the one-CTA kernels (which also split K)."""
    if M < 256 or N < 256 or K < 128:
        return False
    return ((M + 255) // 256) * ((N + 255) // 256) >= TWO_CTA["min_tiles"]


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None, bias: torch.Tensor | None = None, bias_along_m: bool = False,
         alpha: float = 1.0, accumulate: bool = False, transposed: bool = False, bn: int | None = None,
         ksplit: int = 1) -> torch.Tensor:
    """``C = alpha * A @ B^T (+ bias) (+ C)``; see the module docstring for the layout flags.

    ``a`` is ``[M,K]`` (K-major) or ``[K,M]`` (``a_mn``); ``b`` is ``[N,K]`` or ``[K,N]`` (``b_mn``).  With
    ``transposed`` the result is written as ``C^T`` (shape ``[N,M]``).
    """
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        assert not accumulate
        out = torch.empty((N, M) if transposed else (M, N), dtype=out_dtype or a.dtype, device=a.device)
    if not _lib.use_native(a):
        af = (a.t() if a_mn else a).float()
        bf = (b.t() if b_mn else b).float()
        c = alpha * (af @ bf.t())
        if bias is not None:
            c = c + (bias.float()[:, None] if bias_along_m else bias.float()[None, :])
        if transposed:
            c = c.t()
        if accumulate:
            out.add_(c.to(out.dtype))
        else:
            out.copy_(c.to(out.dtype))
        return out
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "native GEMM operands are bf16"
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
    if K == 0:
        if not accumulate:
            out.zero_()
        return out
    lib = _lib.kernels()
    if (TWO_CTA["enabled"] and bn is None and ksplit == 1 and not transposed and not bias_along_m
            and (b_mn or not a_mn) and _use_two_cta(M, N, K) and out.dtype in (torch.bfloat16, torch.float32)
            and hasattr(lib, "gk_gemm_2cta")):
        # CTA pairs on 256 x 256 tiles (tcgen05.mma.cta_group::2): each SM stages half of the B tile
        LAUNCHES["gemm"] += 1
        rc = lib.gk_gemm_2cta(_lib.ptr(a), a.stride(0), a.shape[0], int(a_mn), _lib.ptr(b), b.stride(0), b.shape[0],
                              int(b_mn), _lib.ptr(out), out.stride(0), int(out.dtype == torch.float32), int(accumulate),
                              _lib.ptr(bias), int(bias is not None and bias.dtype == torch.float32), float(alpha),
                              M, N, K, _lib.ptr(_lib.err_flag(a.device)), _lib.stream_ptr())
        _lib.check(rc, "gk_gemm_2cta")
        return out
    if (bn is None and ksplit == 1 and not transposed and not bias_along_m and _use_wide(M, N, K)
            and out.dtype in (torch.bfloat16, torch.float32) and hasattr(lib, "gk_gemm_wide")):
        LAUNCHES["gemm"] += 1
        ws, cnt = _scratch(a.device, 16 << 20, 4096)     # 64 MB: K-split partials of the partial last wave
        rc = lib.gk_gemm_wide(_lib.ptr(a), a.stride(0), a.shape[0], int(a_mn), _lib.ptr(b), b.stride(0), b.shape[0],
                              int(b_mn), _lib.ptr(out), out.stride(0), int(out.dtype == torch.float32), int(accumulate),
                              _lib.ptr(bias), int(bias is not None and bias.dtype == torch.float32), float(alpha),
                              M, N, K, _lib.ptr(ws), ws.numel(), _lib.ptr(cnt), cnt.numel(),
                              _lib.ptr(_lib.err_flag(a.device)), _lib.stream_ptr())
        _lib.check(rc, "gk_gemm_wide")
        return out
    if bn is None:
        bn = _pick_bn(N, M, b_mn) if (ksplit == 1 and not transposed) else _pick_bn(N)
    if b_mn and bn < 64:
        bn = 64
    ws = cnt = None
    if ksplit > 1:
        wsf, cn = ctypes.c_longlong(), ctypes.c_longlong()
        lib.gk_gemm_splitk_scratch(M, N, bn, ksplit, ctypes.byref(wsf), ctypes.byref(cn))
        ws, cnt = _scratch(a.device, wsf.value, cn.value)
    LAUNCHES["gemm"] += 1
    rc = lib.gk_gemm_bf16(
        _lib.ptr(a), a.stride(0), a.shape[0], int(a_mn), _lib.ptr(b), b.stride(0), b.shape[0], int(b_mn),
        _lib.ptr(out), out.stride(0), int(out.dtype == torch.float32), int(transposed), int(accumulate),
        _lib.ptr(bias), int(bias is not None and bias.dtype == torch.float32), int(bias_along_m), float(alpha),
        M, N, K, bn, ksplit, 0, 0, None, 0, 0, 0, _lib.ptr(ws), _lib.ptr(cnt), _lib.ptr(_lib.err_flag(a.device)),
        _lib.stream_ptr())
    _lib.check(rc, "gk_gemm_bf16")
    return out


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor, *, b_mn: bool = False,
                 out: torch.Tensor | None = None, out_dtype=torch.bfloat16, max_rows: int | None = None):
    """Ragged-M grouped GEMM: rows ``offsets[g]:offsets[g+1]`` of ``a`` ([Mtot,K]) use weight ``b[g]``.

    ``b`` is ``[G,N,K]`` (``b_mn=False``: ``y = x W_g^T``) or ``[G,K,N]`` (``b_mn=True``: ``y = x W_g``).
    ``offsets`` (int32, on device) must be multiples of 128; rows between a segment's real end and its padded
    end must be zero.  Mirrors the grouped expert GEMM the reference reaches through TransformerEngine
    (gpatch_v4/models/deepseek_v4/fp8.py:181-394) without the 128-row buffer copies.
    """
    G = b.shape[0]
    Mtot, K = a.shape
    N = b.shape[2] if b_mn else b.shape[1]
    if out is None:
        out = torch.empty((Mtot, N), dtype=out_dtype, device=a.device)
    if not _lib.use_native(a):
        off = offsets.tolist()
        out.zero_()
        for g in range(G):
            s, e = off[g], off[g + 1]
            if e > s:
                w = b[g].float()
                out[s:e] = (a[s:e].float() @ (w if b_mn else w.t())).to(out.dtype)
        return out
    b2 = b.reshape(-1, b.shape[-1])
    bn = _pick_bn(N)
    if b_mn and bn < 64:
        bn = 64
    hint = (max_rows if max_rows is not None else Mtot) // 128 + 1
    LAUNCHES["gemm"] += 1
    rc = _lib.kernels().gk_gemm_bf16(
        _lib.ptr(a), a.stride(0), Mtot, 0, _lib.ptr(b2), b2.stride(0), b2.shape[0], int(b_mn), _lib.ptr(out),
        out.stride(0), int(out.dtype == torch.float32), 0, 0, None, 0, 0, 1.0, Mtot, N, K, bn, 1, 1, G,
        _lib.ptr(offsets), b.shape[1], 0, hint, None, None, _lib.ptr(_lib.err_flag(a.device)), _lib.stream_ptr())
    _lib.check(rc, "gk_gemm_bf16[grouped]")
    return out


def grouped_wgrad(dy: torch.Tensor, x: torch.Tensor, offsets: torch.Tensor, num_groups: int, *,
                  out: torch.Tensor | None = None, accumulate: bool = False, out_dtype=torch.float32):
    """Ragged-K grouped GEMM: ``dW[g] = dy[seg_g]^T @ x[seg_g]`` -> ``[G, N, K]``."""
    Mtot, N = dy.shape
    K = x.shape[1]
    if out is None:
        out = torch.empty((num_groups, N, K), dtype=out_dtype, device=dy.device)
        accumulate = False
    if not _lib.use_native(dy):
        off = offsets.tolist()
        for g in range(num_groups):
            s, e = off[g], off[g + 1]
            r = (dy[s:e].float().t() @ x[s:e].float()).to(out.dtype)
            if accumulate:
                out[g] += r
            else:
                out[g] = r
        return out
    bn = max(_pick_bn(K), 64)
    LAUNCHES["gemm"] += 1
    rc = _lib.kernels().gk_gemm_bf16(
        _lib.ptr(dy), dy.stride(0), Mtot, 1, _lib.ptr(x), x.stride(0), Mtot, 1, _lib.ptr(out), out.stride(1),
        int(out.dtype == torch.float32), 0, int(accumulate), None, 0, 0, 1.0, N, K, Mtot, bn, 1, 2, num_groups,
        _lib.ptr(offsets), 0, out.stride(0), 0, None, None, _lib.ptr(_lib.err_flag(dy.device)), _lib.stream_ptr())
    _lib.check(rc, "gk_gemm_bf16[wgrad-grouped]")
    return out


# ----------------------------------------------------------------------------------------------------------
_SKINNY = [__import__("os").environ.get("GCORE_SKINNY_GEMM", "1") != "0"]


_SKINNY_PLANS: dict = {}
# output tiles (of 128 features) up to which the cluster kernel is tried: the 36-tile qkv projection measured slower on it (18.5 vs 15.4 us) than on the persistent kernel
SKINNY_MAX_TILES = [int(os.environ.get("GCORE_SKINNY_MAX_TILES", "32"))]


def _skinny_plan(T: int, tiles: int, kb: int, K: int):
    """Cluster size (CTAs that split K for one 128-feature tile) and padded token count: the largest cluster whose
    tiles all fit on the GPU in one wave (asked from the occupancy API once per shape)."""
    key = (T, tiles, kb)
    plan = _SKINNY_PLANS.get(key)
    if plan is None:
        lib = _lib.kernels()
        best = (1, (T + 15) // 16 * 16, tiles)
        for ks in range(2, 9):
            if kb // ks < 2:
                break
            step = 16 * ks // math.gcd(16, ks)
            tpad = (T + step - 1) // step * step
            if tpad > 256:
                continue
            if lib.gk_gemm_skinny_max_clusters(tpad, ks, K) >= tiles and tiles * ks > best[2]:
                best = (ks, tpad, tiles * ks)
        plan = best[:2]
        _SKINNY_PLANS[key] = plan
    return plan


def linear_forward(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                   out: torch.Tensor | None = None, out_dtype=None) -> torch.Tensor:
    """``y[T,N] = x[T,K] @ w[N,K]^T + bias``.  Few tokens (decode) run swap-AB + split-K so the weight streams
    from HBM exactly once with every SM busy."""
    T, K = x.shape
    N = w.shape[0]
    if _lib.use_native(x) and T <= 128 and N >= 256:
        bn = 32 if T <= 32 else (64 if T <= 64 else 128)
        tiles = (N + 127) // 128
        kb = (K + 63) // 64
        # measured on B200 under graph replay: the cluster kernel wins for few tiles and moderate K (projections of a
        # tensor-parallel shard); the persistent kernel's global split-K wins for more tiles or very long K
        if (tiles <= SKINNY_MAX_TILES[0] and kb <= 160 and _SKINNY[0] and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
                and hasattr(_lib.kernels(), "gk_gemm_skinny")):
            # few output tiles: cluster split-K with the reduction in distributed shared memory
            ks, tpad = _skinny_plan(T, tiles, kb, K)
            od = out_dtype or (out.dtype if out is not None else x.dtype)
            y = out if out is not None else torch.empty((T, N), dtype=od, device=x.device)
            if y.dtype in (torch.bfloat16, torch.float32) and y.stride(1) == 1:
                LAUNCHES["gemm"] += 1
                rc = _lib.kernels().gk_gemm_skinny(
                    _lib.ptr(w), w.stride(0), _lib.ptr(x), x.stride(0), _lib.ptr(y), y.stride(0),
                    int(y.dtype == torch.float32), _lib.ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                    T, tpad, N, K, ks, _lib.ptr(_lib.err_flag(x.device)), _lib.stream_ptr())
                _lib.check(rc, "gk_gemm_skinny")
                return y
        ksplit = max(1, min(148 // tiles, kb // 4, 16)) if tiles < 120 else 1
        return gemm(w, x, out=out, out_dtype=out_dtype, bias=bias, bias_along_m=True, transposed=True, bn=bn,
                    ksplit=ksplit)
    return gemm(x, w, out=out, out_dtype=out_dtype, bias=bias)


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
                 accumulate: bool = False) -> torch.Tensor:
    """``dx[T,K] = dy[T,N] @ w[N,K]``."""
    return gemm(dy, w, b_mn=True, out=out, accumulate=accumulate)


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False,
                 out_dtype=torch.float32) -> torch.Tensor:
    """``dw[N,K] = dy[T,N]^T @ x[T,K]`` (fp32 by default so micro-batches accumulate into the main grad)."""
    return gemm(dy, x, a_mn=True, b_mn=True, out=out, out_dtype=out_dtype, accumulate=accumulate)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, w, bias, main_grad):
        # 2-D in, 2-D out: the output must be a fresh tensor (not a view made inside the Function) because callers
        # rotate / overwrite it in place
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.main_grad = main_grad
        return linear_forward(x2, w, bias)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy if dy.is_contiguous() else dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = linear_dgrad(dy2, w)
        if ctx.needs_input_grad[1]:
            mg = ctx.main_grad
            if mg is not None:
                # accumulate straight into the fp32 main-grad buffer (Megatron "gradient accumulation fusion")
                linear_wgrad(dy2, x2, out=mg, accumulate=True)
                dw = None
            else:
                dw = linear_wgrad(dy2, x2, out_dtype=torch.float32).to(w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           main_grad: torch.Tensor | None = None) -> torch.Tensor:
    """Autograd linear layer on the tcgen05 GEMM.  When ``main_grad`` (fp32, same shape as ``w``) is given the
    weight gradient is accumulated into it inside the GEMM epilogue and autograd sees no ``w.grad``."""
    if x.dtype != torch.bfloat16 or not _lib.use_native(x):
        return torch.nn.functional.linear(x, w, bias)
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = _LinearFn.apply(x2, w, bias, main_grad)
    return y if len(shp) == 2 else y.reshape(*shp[:-1], w.shape[0])
