"""Muon: SGD-momentum whose 2-D updates are orthogonalised by a quintic Newton-Schulz iteration
(gpatch_v4/core/muon_optimizer.py:18-160).  Non-matrix parameters (and any the caller marks) fall back to AdamW.

The iteration is five small GEMM triples per matrix in bf16; on a GPU they run on the tcgen05 GEMM
(``ops.gemm.gemm``), batched over parameters of equal shape by the caller when it matters.
"""
from __future__ import annotations

import math
from typing import Iterable, List

import torch

from ..ops import _lib
from ..ops.gemm import gemm

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def _mm_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a @ b^T."""
    if _lib.use_native(a) and a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0:
        return gemm(a.contiguous(), b.contiguous())
    return a @ b.t()


def newton_schulz5(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Approximate ``U V^T`` of ``G = U S V^T`` (singular values pushed towards 1), computed in bf16."""
    assert G.dim() == 2
    a, b, c = NS_COEFFS
    X = G.to(torch.bfloat16)
    transposed = G.shape[0] > G.shape[1]
    if transposed:
        X = X.t().contiguous()
    X = X / (X.norm() + 1e-7)
    for _ in range(steps):
        A = _mm_nt(X, X)                       # X X^T
        B = b * A + c * _mm_nt(A, A)           # A is symmetric: A A^T = A A
        X = a * X + _mm_nt(B, X.t().contiguous())  # B X
    return X.t() if transposed else X


class Muon(torch.optim.Optimizer):
    def __init__(self, muon_params: Iterable[torch.nn.Parameter], adamw_params: Iterable[torch.nn.Parameter] = (),
                 lr: float = 1e-3, wd: float = 0.1, momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 5,
                 adamw_betas=(0.9, 0.95), adamw_eps: float = 1e-8, extra_scale_factor: float = 0.2):
        groups: List[dict] = []
        mp = list(muon_params)
        ap = list(adamw_params)
        if mp:
            groups.append(dict(params=mp, use_muon=True, lr=lr, wd=wd, momentum=momentum, nesterov=nesterov,
                               ns_steps=ns_steps))
        if ap:
            groups.append(dict(params=ap, use_muon=False, lr=lr, wd=wd, betas=adamw_betas, eps=adamw_eps))
        super().__init__(groups, {})
        self.extra_scale_factor = extra_scale_factor

    def adjusted_lr(self, lr: float, shape) -> float:
        return lr * self.extra_scale_factor * math.sqrt(max(shape[0], shape[1]))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            lr, wd = g["lr"], g["wd"]
            for p in g["params"]:
                grad = getattr(p, "main_grad", None)
                grad = grad if grad is not None else p.grad
                if grad is None:
                    continue
                st = self.state[p]
                if g["use_muon"]:
                    g2 = grad.reshape(grad.shape[0], -1).float()
                    if "momentum_buffer" not in st:
                        st["momentum_buffer"] = torch.zeros_like(g2)
                    buf = st["momentum_buffer"]
                    buf.mul_(g["momentum"]).add_(g2)
                    upd = g2.add(buf, alpha=g["momentum"]) if g["nesterov"] else buf
                    u = newton_schulz5(upd, g["ns_steps"]).reshape(p.shape)
                    p.mul_(1 - lr * wd)
                    p.add_(u.to(p.dtype), alpha=-self.adjusted_lr(lr, g2.shape))
                else:
                    if "step" not in st:
                        st["step"] = 0
                        st["m"] = torch.zeros_like(grad, dtype=torch.float32)
                        st["v"] = torch.zeros_like(grad, dtype=torch.float32)
                    st["step"] += 1
                    b1, b2 = g["betas"]
                    gf = grad.float()
                    st["m"].lerp_(gf, 1 - b1)
                    st["v"].mul_(b2).addcmul_(gf, gf, value=1 - b2)
                    bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                    upd = (st["m"] / bc1) / ((st["v"] / bc2).sqrt() + g["eps"])
                    p.mul_(1 - lr * wd)
                    p.add_(upd.to(p.dtype), alpha=-lr)
        return loss


def split_muon_params(model: torch.nn.Module):
    """2-D hidden-layer matrices go to Muon; embeddings, the output head, gains and biases go to AdamW."""
    muon, adam = [], []
    for n, p in model.named_parameters():
        if not p.requires_grad:
            continue
        if p.dim() == 2 and "embedding" not in n and "output_layer" not in n and "router" not in n:
            muon.append(p)
        else:
            adam.append(p)
    return muon, adam
