"""Optimizer-side kernels on flat buffers: fused AdamW on the fp32 master shard (writes the bf16 parameter in the
same pass), squared-L2 norm, scaled cast/accumulate.  PyTorch fallbacks implement the same arithmetic on CPU."""
from __future__ import annotations

import torch

from . import _lib

LAUNCHES = {"optim": 0}


def adam_step(master, m, v, grad, param, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=None,
              scale_val: float = 1.0):
    """AdamW (decoupled weight decay, bias-corrected) over flat 1-D buffers, in place.

    ``grad`` may be fp32 or bf16; ``param`` (bf16, optional) receives the rounded master weights;
    ``grad_scale`` is an optional 1-element device tensor multiplied into every gradient (clip coefficient)."""
    n = master.numel()
    if _lib.use_native(master) and grad.dtype in (torch.float32, torch.bfloat16):
        LAUNCHES["optim"] += 1
        # the kernel rounds the master weights to bf16 parameters; parameters of another dtype (fp32 models) are
        # refreshed from the master weights afterwards
        fused_param = param if (param is not None and param.dtype == torch.bfloat16) else None
        _lib.check(_lib.kernels().gk_adam(_lib.ptr(master), _lib.ptr(m), _lib.ptr(v), _lib.ptr(grad),
                                          int(grad.dtype == torch.float32), _lib.ptr(fused_param), n, float(lr),
                                          float(beta1), float(beta2), float(eps), float(weight_decay), int(step),
                                          _lib.ptr(grad_scale), float(scale_val), _lib.stream_ptr()), "adam")
        if param is not None and fused_param is None:
            param.copy_(master.to(param.dtype))
        return
    g = grad.float() * scale_val
    if grad_scale is not None:
        g = g * grad_scale.float()
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    upd = (m / bc1) / ((v / bc2).sqrt() + eps) + weight_decay * master
    master.add_(upd, alpha=-lr)
    if param is not None:
        param.copy_(master.to(param.dtype))


def sumsq(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[0] += sum(x**2)`` (fp32 accumulation); returns ``out``."""
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    if _lib.use_native(x) and x.dtype in (torch.float32, torch.bfloat16) and x.is_contiguous():
        LAUNCHES["optim"] += 1
        _lib.check(_lib.kernels().gk_sumsq(_lib.ptr(x), int(x.dtype == torch.float32), x.numel(), _lib.ptr(out),
                                           _lib.stream_ptr()), "sumsq")
        return out
    out += x.float().pow(2).sum()
    return out


def axpy_cast(src: torch.Tensor, dst: torch.Tensor, scale: float = 1.0, accumulate: bool = False):
    """``dst (+)= scale * src`` with dtype conversion (bf16 <-> fp32)."""
    if _lib.use_native(src) and src.is_contiguous() and dst.is_contiguous() and \
            src.dtype in (torch.float32, torch.bfloat16) and dst.dtype in (torch.float32, torch.bfloat16):
        LAUNCHES["optim"] += 1
        _lib.check(_lib.kernels().gk_axpy_cast(_lib.ptr(src), int(src.dtype == torch.float32), _lib.ptr(dst),
                                               int(dst.dtype == torch.float32), src.numel(), float(scale),
                                               int(accumulate), _lib.stream_ptr()), "axpy_cast")
        return dst
    if accumulate:
        dst.add_((src.float() * scale).to(dst.dtype))
    else:
        dst.copy_((src.float() * scale).to(dst.dtype))
    return dst
