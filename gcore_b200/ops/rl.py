"""RL objective kernels: the GRPO / PPO-clip token loss with k3 KL (forward value and d/dlogp in one pass) and the
GAE reverse scan.  Definitions: gpatch_v4/training_backend/loss/ppo_loss.py:232-346, gpatch_v4/utils/ppo_utils.py:
151-193, gpatch_v4/core/advantage_impl.py:394-444."""
from __future__ import annotations

import torch

from . import _lib

LAUNCHES = {"rl": 0}
STAT_NAMES = ("pg_loss", "kl", "weight", "clipfrac", "ratio", "approx_kl")


def grpo_token_loss_ref(logp, old_lp, ref_lp, adv, *, clip_low, clip_high, dual_clip_c=0.0, kl_beta=0.0,
                        ratio_clamp=0.0, kl_clamp=0.0):
    """Differentiable PyTorch definition: returns ``(per-token loss, per-token kl, ratio, clipped mask)``."""
    old = logp.detach() if old_lp is None else old_lp
    d = logp - old
    if ratio_clamp and ratio_clamp > 0:
        d = d.clamp(-ratio_clamp, ratio_clamp)
    ratio = torch.exp(d)
    l1 = -adv * ratio
    l2 = -adv * ratio.clamp(1 - clip_low, 1 + clip_high)
    L = torch.maximum(l1, l2)
    clipped = l2 > l1
    if dual_clip_c and dual_clip_c > 0:
        l3 = -adv * dual_clip_c
        use3 = (adv < 0) & (l3 < L)
        L = torch.where(use3, l3.detach() + 0 * L, L)
        clipped = clipped | use3
    kl = torch.zeros_like(logp)
    if kl_beta and ref_lp is not None:
        dr = ref_lp - logp
        kl = torch.exp(dr) - dr - 1
        if kl_clamp and kl_clamp > 0:
            kl = kl.clamp(max=kl_clamp)
    return L + kl_beta * kl, kl, ratio, clipped


class _GrpoLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logp, old_lp, ref_lp, adv, weight, cfg):
        n = logp.numel()
        dlogp = torch.empty_like(logp)
        stats = torch.zeros(8, dtype=torch.float32, device=logp.device)
        LAUNCHES["rl"] += 1
        _lib.check(_lib.kernels().gk_grpo_loss(
            _lib.ptr(logp), _lib.ptr(old_lp), _lib.ptr(ref_lp), _lib.ptr(adv), _lib.ptr(weight), n,
            cfg["clip_low"], cfg["clip_high"], cfg["dual_clip_c"], cfg["kl_beta"], cfg["ratio_clamp"],
            cfg["kl_clamp"], None, _lib.ptr(dlogp), _lib.ptr(stats), _lib.stream_ptr()), "grpo_loss")
        ctx.save_for_backward(dlogp)
        loss = stats[0] + cfg["kl_beta"] * stats[1]
        ctx.mark_non_differentiable(stats)
        return loss, stats

    @staticmethod
    def backward(ctx, g, _gs):
        (dlogp,) = ctx.saved_tensors
        return dlogp * g, None, None, None, None, None


def grpo_loss(logp, old_lp, ref_lp, adv, weight, *, clip_low=0.2, clip_high=0.2, dual_clip_c=0.0, kl_beta=0.0,
              ratio_clamp=0.0, kl_clamp=0.0):
    """``loss = sum_t weight_t * (L_clip(t) + kl_beta * k3(t))`` over flat fp32 tensors.

    ``weight`` carries both the response mask and the normaliser (1/#tokens for per-token loss, 1/(len_i * #seqs) for
    per-sequence means).  Returns ``(loss, stats)`` with ``stats`` = weighted sums named by ``STAT_NAMES``."""
    cfg = dict(clip_low=float(clip_low), clip_high=float(clip_high), dual_clip_c=float(dual_clip_c or 0.0),
               kl_beta=float(kl_beta or 0.0), ratio_clamp=float(ratio_clamp or 0.0), kl_clamp=float(kl_clamp or 0.0))
    if _lib.use_native(logp) and logp.dtype == torch.float32:
        flat = lambda t: None if t is None else t.reshape(-1).contiguous().float()
        return _GrpoLossFn.apply(flat(logp), flat(old_lp), flat(ref_lp), flat(adv), flat(weight), cfg)
    tl, kl, ratio, clipped = grpo_token_loss_ref(logp, old_lp, ref_lp, adv, **cfg)
    w = weight
    pg = tl - cfg["kl_beta"] * kl
    old = logp.detach() if old_lp is None else old_lp
    stats = torch.stack([(w * pg).sum(), (w * kl).sum(), w.sum(), (w * clipped.float()).sum(), (w * ratio).sum(),
                         (w * (old - logp)).sum(), w.sum() * 0, w.sum() * 0]).detach()
    return (w * tl).sum(), stats


def gae(rewards, values, mask, gamma: float, lam: float):
    """Generalised advantage estimation over ``[B, S]``; masked-out tokens are skipped (their slot carries the next
    valid value / advantage).  Returns ``(advantages, returns)``."""
    B, S = rewards.shape
    adv = torch.zeros_like(rewards, dtype=torch.float32)
    ret = torch.zeros_like(rewards, dtype=torch.float32)
    if _lib.use_native(rewards):
        r, v, mk = rewards.float().contiguous(), values.float().contiguous(), mask.float().contiguous()
        LAUNCHES["rl"] += 1
        _lib.check(_lib.kernels().gk_gae(_lib.ptr(r), _lib.ptr(v), _lib.ptr(mk), _lib.ptr(adv), _lib.ptr(ret), B, S,
                                         float(gamma), float(lam), _lib.stream_ptr()), "gae")
        return adv, ret
    next_v = torch.zeros(B, dtype=torch.float32, device=rewards.device)
    last = torch.zeros(B, dtype=torch.float32, device=rewards.device)
    rf, vf, mf = rewards.float(), values.float(), mask.float()
    for t in range(S - 1, -1, -1):
        on = mf[:, t] > 0
        delta = rf[:, t] + gamma * next_v - vf[:, t]
        new_last = delta + gamma * lam * last
        last = torch.where(on, new_last, last)
        next_v = torch.where(on, vf[:, t], next_v)
        adv[:, t] = torch.where(on, last, torch.zeros_like(last))
        ret[:, t] = torch.where(on, last + vf[:, t], torch.zeros_like(last))
    return adv, ret
