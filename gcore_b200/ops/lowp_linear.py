"""Low-precision variants of the linear layer, selected per module by ``ParallelLinear.precision``:

* ``fp8``      - block-scaled e4m3 compute: activations quantised 1x128 per token on the fly, the weight 128x128
  (cached until the parameter changes), product on the fp8 tensor-core GEMM.  The data gradient runs in bf16 against
  the dequantised weight, or with ``GCORE_FP8_DGRAD=1`` on the same fp8 GEMM (dY quantised 1x128 along the output
  features, the cached e4m3 weight transposed once per version); the weight gradient (skipped for a frozen base
  under LoRA) runs in bf16 from the saved activations, or with ``GCORE_FP8_WGRAD=1`` on the fp8 GEMM with both
  operands quantised along the token axis.  Both fp8 gradients are off by default: they measured slower than bf16.
* ``fp8_qat`` / ``fp4_qat`` - quantisation-aware training: the bf16 GEMM sees the weight after a quantise ->
  dequantise round trip (128x128 e4m3 blocks, or 1x32 e2m1 groups with power-of-two scales); gradients pass straight
  through to the bf16 parameter.

(The reference's fp8 training path and fp8 / fp4 QAT: gpatch_v4/models/deepseek_v4/fp8.py, kernel/quantize/qat.py.)
"""
from __future__ import annotations

import os

import torch

from . import quant
from .gemm import linear, linear_dgrad, linear_wgrad


def fake_quant_weight(w: torch.Tensor, kind: str) -> torch.Tensor:
    """Quantise -> dequantise copy of ``w`` (no gradient)."""
    with torch.no_grad():
        if kind == "fp8_qat":
            return quant.qat_fp8_(w.detach().clone().contiguous(), block="128x128")
        if kind == "fp4_qat":
            if w.numel() % 32:
                return w.detach()
            return quant.fp4_quant_1x32_ref(w.detach())[2].to(w.dtype) if not w.is_cuda else _fp4_dq_native(w)
    raise ValueError(kind)


def _fp4_dq_native(w: torch.Tensor) -> torch.Tensor:
    from . import _lib
    x = w.detach().contiguous()
    if not (_lib.use_native(x) and x.dtype == torch.bfloat16):
        return quant.fp4_quant_1x32_ref(x)[2].to(w.dtype)
    n = x.numel()
    packed = torch.empty(n // 2, dtype=torch.uint8, device=x.device)
    e8 = torch.empty(n // 32, dtype=torch.uint8, device=x.device)
    s = torch.empty(n // 32, dtype=torch.float32, device=x.device)
    dq = torch.empty_like(x)
    _lib.check(_lib.kernels().gk_fp4_quant_1x32(_lib.ptr(x), _lib.ptr(packed), _lib.ptr(e8), _lib.ptr(s), _lib.ptr(dq),
                                                n, _lib.stream_ptr()), "fp4_quant")
    return dq


def qat_linear(x, w, bias, main_grad, kind: str):
    """Straight-through estimator: forward with the fake-quantised weight, gradient to ``w`` as if it were used."""
    w_eff = w + (fake_quant_weight(w, kind) - w).detach() if main_grad is None else _Ste.apply(w, kind)
    return linear(x, w_eff, bias, main_grad)


class _Ste(torch.autograd.Function):
    """Fake-quantised weight whose gradient goes to ``main_grad`` inside the wgrad GEMM (nothing flows back here)."""

    @staticmethod
    def forward(ctx, w, kind):
        return fake_quant_weight(w, kind)

    @staticmethod
    def backward(ctx, g):
        return g, None


def fp8_dgrad_enabled() -> bool:
    # opt-in: quantising dY plus the block-fp8 GEMM measured 3.75 / 1.64 / 0.64 ms against 3.89 / 1.34 / 0.51 ms for
    # dequantise + bf16 GEMM on 16384-token gradients of 7168x18432, 24576x1536 and 7168x2048 weights (B200)
    return os.environ.get("GCORE_FP8_DGRAD", "0") == "1"


def fp8_wgrad_enabled() -> bool:
    return os.environ.get("GCORE_FP8_WGRAD", "0") == "1"


class _Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, w, bias, main_grad, cache):
        ver = (w._version, w.data_ptr())
        if cache.get("ver") != ver:
            q, s = quant.quant_weight_128x128(w.detach().to(torch.bfloat16).contiguous())
            cache.update(ver=ver, q=q, s=s)
        aq, as_ = quant.quant_act_1x128(x2.to(torch.bfloat16).contiguous())
        y = quant.gemm_fp8_blockscaled(aq, as_, cache["q"], cache["s"], out_dtype=x2.dtype
                                       if x2.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16)
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(x2 if w.requires_grad else x2.new_empty(0), w)
        ctx.cache, ctx.main_grad, ctx.has_bias = cache, main_grad, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            if fp8_dgrad_enabled() and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0:
                dx = quant.fp8_dgrad(dy2, ctx.cache, dy2.dtype)
            else:
                w_dq = quant.dequant_128x128(ctx.cache["q"], ctx.cache["s"]).to(dy2.dtype)
                dx = linear_dgrad(dy2, w_dq[:w.shape[0], :w.shape[1]].contiguous())
        if ctx.needs_input_grad[1]:
            if fp8_wgrad_enabled() and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0:
                g = quant.fp8_wgrad(dy2, x2)
                if ctx.main_grad is not None:
                    ctx.main_grad.add_(g)
                else:
                    dw = g.to(w.dtype)
            elif ctx.main_grad is not None:
                linear_wgrad(dy2, x2, out=ctx.main_grad, accumulate=True)
            else:
                dw = linear_wgrad(dy2, x2, out_dtype=torch.float32).to(w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db, None, None


def fp8_linear(x, w, bias, main_grad, cache: dict):
    shp = x.shape
    y = _Fp8LinearFn.apply(x.reshape(-1, shp[-1]), w, bias, main_grad, cache)
    return y.reshape(*shp[:-1], w.shape[0])
