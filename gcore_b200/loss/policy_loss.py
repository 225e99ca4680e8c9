"""Policy-gradient objectives on packed per-token tensors, behind a name registry.

Semantics follow the reference's loss registry (gpatch_v4/training_backend/loss/registry.py:10-106 and
ppo_loss.py:232-863): ``grpo`` (PPO clip with asymmetric / dual clip), ``gspo`` (sequence-level importance ratio with
token-level gradient), ``cispo`` (clipped, detached IS weight on a REINFORCE term), ``sapo`` (soft sigmoid gate),
``vespo`` (smooth sequence-level kernel), ``opd`` / ``reinforce``.  Every loss returns per-token values; the caller
applies KL-to-reference, the entropy bonus, off-policy correction weights and the aggregation weights.

All tensors are flat ``[T]`` fp32 on the log-prob axis; ``seq_ids`` maps a token to its sequence for the
sequence-level variants (packing-safe, unlike a ``[B, S]`` reduction over the last dim).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, Optional

import torch

from ..ops import rl as rl_ops

_REGISTRY: Dict[str, Callable] = {}


def register_loss(name: str):
    def deco(fn):
        if name in _REGISTRY:
            raise KeyError(f"loss '{name}' already registered")
        _REGISTRY[name] = fn
        return fn
    return deco


def get_loss(name: str) -> Callable:
    if name not in _REGISTRY:
        raise KeyError(f"unknown loss '{name}'; registered: {sorted(_REGISTRY)}")
    return _REGISTRY[name]


def registered_losses():
    return sorted(_REGISTRY)


@dataclass
class LossInput:
    logp: torch.Tensor                      # current policy, requires grad
    old_logp: Optional[torch.Tensor]        # behaviour policy under the trainer (None -> logp.detach())
    ref_logp: Optional[torch.Tensor]
    rollout_logp: Optional[torch.Tensor]    # behaviour policy as reported by the rollout engine
    advantages: torch.Tensor
    mask: torch.Tensor
    seq_ids: torch.Tensor                   # [T] int
    num_seqs: int
    entropy: Optional[torch.Tensor] = None
    old_entropy: Optional[torch.Tensor] = None


@dataclass
class LossOutput:
    token_loss: torch.Tensor
    ratios: torch.Tensor
    metrics: Dict[str, torch.Tensor] = field(default_factory=dict)


_CP_GROUP = None


def set_context_parallel_group(group):
    """Per-sequence sums span the ranks of this group when the tokens of a sequence are sharded over it."""
    global _CP_GROUP
    _CP_GROUP = group


class _SumOverCP(torch.autograd.Function):
    """Sum over the context-parallel ranks; every rank's loss depends on the total, so the gradient is summed too."""

    @staticmethod
    def forward(ctx, x, group):
        import torch.distributed as dist
        ctx.group = group
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def _seg_sum(x, seq_ids, n):
    out = torch.zeros(n, dtype=x.dtype, device=x.device)
    out = out.index_add_(0, seq_ids.long(), x)
    if _CP_GROUP is not None:
        out = _SumOverCP.apply(out, _CP_GROUP)
    return out


def _token_ratio(cfg, logp, old):
    d = logp - old
    if cfg.ppo_logps_ratio_clamp is not None:
        d = d.clamp(-cfg.ppo_logps_ratio_clamp, cfg.ppo_logps_ratio_clamp)
    return torch.exp(d)


def _frac(flag, mask):
    n = mask.sum()
    return torch.stack([(flag.float() * mask).sum(), n])


@register_loss("grpo")
def grpo_loss(cfg, li: LossInput) -> LossOutput:
    old = li.logp.detach() if li.old_logp is None else li.old_logp
    tl, _, ratio, clipped = rl_ops.grpo_token_loss_ref(
        li.logp, old, None, li.advantages, clip_low=cfg.clip_low, clip_high=cfg.clip_high,
        dual_clip_c=cfg.ppo_dual_clip_ratio_c or 0.0, kl_beta=0.0, ratio_clamp=cfg.ppo_logps_ratio_clamp or 0.0)
    return LossOutput(tl, ratio.detach(), {"ppo_ratio_clamped_frac": _frac(clipped, li.mask)})


@register_loss("gspo")
def gspo_loss(cfg, li: LossInput) -> LossOutput:
    """Sequence importance ratio = exp(mean_t(logp - old)); the gradient still flows through every token."""
    old = li.logp.detach() if li.old_logp is None else li.old_logp
    d = (li.logp - old) * li.mask
    lens = _seg_sum(li.mask, li.seq_ids, li.num_seqs).clamp_min(1.0)
    seq_mean = _seg_sum(d, li.seq_ids, li.num_seqs) / lens
    log_ratio = li.logp - li.logp.detach() + seq_mean.detach()[li.seq_ids.long()]
    ratio = torch.exp(log_ratio.clamp(max=10.0))
    l1 = -li.advantages * ratio
    l2 = -li.advantages * ratio.clamp(1 - cfg.clip_low, 1 + cfg.clip_high)
    return LossOutput(torch.maximum(l1, l2), ratio.detach(), {"ppo_ratio_clamped_frac": _frac(l2 > l1, li.mask)})


@register_loss("cispo")
def cispo_loss(cfg, li: LossInput) -> LossOutput:
    old = li.logp.detach() if li.old_logp is None else li.old_logp
    ratio = _token_ratio(cfg, li.logp, old)
    clipped = ratio.clamp(1 - cfg.clip_low, 1 + cfg.clip_high)
    tl = -clipped.detach() * li.advantages * li.logp
    return LossOutput(tl, ratio.detach(), {"cispo/clipfrac": _frac(clipped.detach() != ratio.detach(), li.mask)})


@register_loss("sapo")
def sapo_loss(cfg, li: LossInput) -> LossOutput:
    old = li.logp.detach() if li.old_logp is None else li.old_logp
    ratio = _token_ratio(cfg, li.logp, old)
    tau = torch.where(li.advantages > 0, torch.full_like(ratio, cfg.sapo_tau_pos),
                      torch.full_like(ratio, cfg.sapo_tau_neg))
    sg = torch.sigmoid(tau * (ratio - 1.0))
    gate = (4.0 / tau) * sg
    kern = 4.0 * sg.detach() * (1 - sg.detach())
    return LossOutput(-li.advantages * gate, ratio.detach(),
                      {"sapo/strong_attenuation_frac": _frac(kern < 0.5, li.mask)})


@register_loss("vespo")
def vespo_loss(cfg, li: LossInput) -> LossOutput:
    """REINFORCE scaled by phi(W) = W^c1 * exp(c2 * (1 - W)), W = product of token ratios (policy lag times
    train / rollout mismatch) over the sequence; phi is detached."""
    assert li.old_logp is not None and li.rollout_logp is not None, "vespo needs prev and rollout log-probs"
    clampv = cfg.ppo_logps_ratio_clamp or 20.0
    with torch.no_grad():
        tlr = (li.logp - li.old_logp).clamp(-clampv, clampv)
        tis = (li.old_logp - li.rollout_logp).clamp(-clampv, clampv)
        seq_log_w = _seg_sum((tlr + tis) * li.mask, li.seq_ids, li.num_seqs).clamp(-clampv, clampv)
        w = seq_log_w.exp()
        lens = _seg_sum(li.mask, li.seq_ids, li.num_seqs).clamp_min(1.0)
        seq_adv = _seg_sum(li.advantages * li.mask, li.seq_ids, li.num_seqs) / lens
        pos = (seq_adv >= 0).float()
        c1 = pos * getattr(cfg, "vespo_c1_pos", 1.0) + (1 - pos) * getattr(cfg, "vespo_c1_neg", 1.0)
        c2 = (pos * getattr(cfg, "vespo_c2_pos", 1.0) + (1 - pos) * getattr(cfg, "vespo_c2_neg", 1.0)).clamp_min(1e-4)
        phi = torch.nan_to_num(torch.exp(c2 + c1 * torch.log(w.clamp_min(1e-8)) - c2 * w), 0.0, 0.0, 0.0)
        ratio = tlr.exp()
    tl = -phi[li.seq_ids.long()] * li.advantages * li.logp
    return LossOutput(tl, ratio, {"vespo/phi_mean": torch.stack([phi.sum(), phi.new_tensor(float(phi.numel()))])})


@register_loss("steer")
def steer_loss(cfg, li: LossInput) -> LossOutput:
    """A base surrogate (``steer_policy_method``) whose tokens are down-weighted by how much their update is estimated
    to move the policy entropy: ``metric = |A / p_old * p (1 - p) * (ln p + H)|``, weight ``exp(-k * metric)`` clipped
    to ``[w_min, 1]`` with ``k`` chosen so that the largest metric of the batch gets ``w_min``
    (gpatch_v4/training_backend/loss/ppo_loss.py:253-290, 872)."""
    base = get_loss(cfg.steer_policy_method)(cfg, li)
    H = li.old_entropy if li.old_entropy is not None else li.entropy
    if H is None:
        raise ValueError("loss_func=steer needs per-token entropies (they are computed when it is selected)")
    w_min = float(cfg.steer_token_weight_min)
    with torch.no_grad():
        old = li.logp.detach() if li.old_logp is None else li.old_logp
        p = li.logp.detach().float().exp().clamp(1e-8, 1.0 - 1e-8)
        metric = (li.advantages.float() / old.float().exp().clamp(1e-8, 1.0) * p * (1.0 - p) *
                  (p.log() + H.detach().float())).abs()
        valid = li.mask > 0
        top = metric[valid].max() if bool(valid.any()) else metric.new_zeros(())
        k = -math.log(w_min) / torch.clamp(top, min=0.02) if w_min < 1.0 else metric.new_zeros(())
        w = torch.exp(-k * metric).clamp(w_min, 1.0) * li.mask
    m = dict(base.metrics)
    m["steer/token_weight_mean"] = torch.stack([w.sum(), li.mask.sum()])
    m["steer/token_weight_lt_0_95_frac"] = _frac((w < 0.95) & valid, li.mask)
    return LossOutput(base.token_loss * w, base.ratios, m)


def discounted_future_sum(x: torch.Tensor, seq_ids: torch.Tensor, gamma: float, chunk: int = 512) -> torch.Tensor:
    """``out[t] = sum_{j >= t, same sequence} gamma^(j - t) x[j]`` over packed sequences.  Every sequence is walked
    from its end in chunks; inside a chunk the sum is a reversed cumulative sum of ``x * gamma^k`` divided by
    ``gamma^k`` in fp64 (exact for chunk lengths whose ``gamma^-k`` stays finite), the tail enters as a carry."""
    out = torch.zeros_like(x, dtype=torch.float64)
    ids = seq_ids.long()
    T = x.numel()
    if T == 0:
        return out.to(x.dtype)
    change = torch.nonzero(ids[1:] != ids[:-1]).flatten() + 1
    bounds = [0] + change.tolist() + [T]
    xd = x.double()
    for s0, s1 in zip(bounds[:-1], bounds[1:]):
        carry = xd.new_zeros(())
        for b in range(s1, s0, -chunk):
            a = max(s0, b - chunk)
            k = torch.arange(b - a, device=x.device, dtype=torch.float64)
            w = torch.pow(xd.new_tensor(gamma), k)
            local = torch.flip(torch.cumsum(torch.flip(xd[a:b] * w, [0]), 0), [0]) / w
            out[a:b] = local + carry * torch.pow(xd.new_tensor(gamma), (b - a) - k)
            carry = out[a]
    return out.to(x.dtype)


@register_loss("fipo")
def fipo_loss(cfg, li: LossInput) -> LossOutput:
    """Clipped surrogate whose advantages are scaled by an influence weight: the exponential of the discounted sum of
    the later tokens' log-ratios (``gamma = 2^(-1 / fipo_decay_rate)``), clipped to ``1 +- fipo_clip_ratio`` (or
    ``[1, 1 + ratio]``); tokens with a negative advantage and a ratio above ``fipo_safety_thresh`` keep at most weight 1;
    sequences with more than one dual-clipped token are dropped
    (gpatch_v4/training_backend/loss_factory.py:1966-2240)."""
    old = li.logp.detach() if li.old_logp is None else li.old_logp
    ratio = _token_ratio(cfg, li.logp, old)
    with torch.no_grad():
        gamma = 2.0 ** (-1.0 / float(cfg.fipo_decay_rate))
        fut = discounted_future_sum((li.logp.detach() - old) * li.mask, li.seq_ids, gamma, int(cfg.fipo_chunk_size))
        hi = 1.0 + cfg.fipo_clip_ratio
        lo = 1.0 if cfg.fipo_clip_high_only else 1.0 - cfg.fipo_clip_ratio
        raw = torch.exp(fut.clamp(max=20.0))
        iw = raw.clamp(lo, hi)
        risky = (li.advantages < 0) & (ratio.detach() > cfg.fipo_safety_thresh)
        iw = torch.where(risky, iw.clamp(0.8, 1.0), iw)
    adv = li.advantages * iw
    l1 = -adv * ratio
    l2 = -adv * ratio.clamp(1 - cfg.clip_low, 1 + cfg.clip_high)
    clip_max = torch.maximum(l1, l2)
    tl = clip_max
    metrics = {"ppo_ratio_clamped_frac": _frac(l2 > l1, li.mask),
               "fipo/influence_weights_mean": torch.stack([(iw * li.mask).sum(), li.mask.sum()]),
               "fipo/clip_frac_total": _frac((raw > hi) | (raw < lo), li.mask)}
    c = cfg.ppo_dual_clip_ratio_c
    if c:
        l3 = -adv * c
        dual = (adv < 0) & (l3 < clip_max)
        tl = torch.where(adv < 0, torch.minimum(l3, clip_max), clip_max)
        n_dual = _seg_sum((dual.float() * li.mask).detach(), li.seq_ids, li.num_seqs)
        keep = (n_dual <= 1).to(tl.dtype)[li.seq_ids.long()]
        tl = tl * keep
        metrics["fipo/dropped_seq_frac"] = torch.stack([(n_dual > 1).float().sum(),
                                                        (_seg_sum(li.mask, li.seq_ids, li.num_seqs) > 0).float().sum()])
    return LossOutput(tl, ratio.detach(), metrics)


def _centered_cov(cfg, li: LossInput):
    """Per-token ``(A - mean A) * (log p - mean log p)`` over the valid tokens of the micro-batch (detached)."""
    valid = li.mask > 0
    n = li.mask.sum().clamp_min(1.0)
    a = li.advantages.detach().float()
    lp = li.logp.detach().float()
    cov = (a - (a * li.mask).sum() / n) * (lp - (lp * li.mask).sum() / n)
    return cov, valid


@register_loss("clip_cov")
def clip_cov_loss(cfg, li: LossInput) -> LossOutput:
    """Clipped surrogate in which a random ``clip_cov_ratio`` share of the valid tokens whose advantage / log-prob
    covariance lies in ``(clip_cov_lb, clip_cov_ub)`` (and which the ratio clip left alone) gets no gradient: the
    high-covariance tokens are the ones that collapse the entropy (gpatch_v4/training_backend/loss/ppo_loss.py:142-167)."""
    old = li.logp.detach() if li.old_logp is None else li.old_logp
    ratio = _token_ratio(cfg, li.logp, old)
    l1 = -li.advantages * ratio
    l2 = -li.advantages * ratio.clamp(1 - cfg.clip_low, 1 + cfg.clip_high)
    with torch.no_grad():
        cov, valid = _centered_cov(cfg, li)
        cand = valid & ~(l2 > l1) & (cov < cfg.clip_cov_ub) & (cov > cfg.clip_cov_lb)
        idx = torch.nonzero(cand).flatten()
        n_drop = max(int(cfg.clip_cov_ratio * float(li.mask.sum())), 1)
        keep = torch.ones_like(li.mask)
        if idx.numel() > 0:
            pick = idx[torch.randperm(idx.numel(), device=idx.device)[:min(n_drop, idx.numel())]]
            keep[pick] = 0
    tl = torch.maximum(l1, l2) * keep
    return LossOutput(tl, ratio.detach(), {"ppo_ratio_clamped_frac": _frac(l2 > l1, li.mask),
                                           "clip_cov_frac": _frac(keep == 0, li.mask),
                                           "cov_mean": torch.stack([(cov * li.mask).sum(), li.mask.sum()])})


@register_loss("kl_cov")
def kl_cov_loss(cfg, li: LossInput) -> LossOutput:
    """Clipped surrogate plus ``kl_cov_coef * |log p - log p_old|`` on the ``kl_cov_ratio`` share of valid tokens
    with the largest advantage / log-prob covariance (gpatch_v4/training_backend/loss/ppo_loss.py:169-210)."""
    old = li.logp.detach() if li.old_logp is None else li.old_logp
    ratio = _token_ratio(cfg, li.logp, old)
    l1 = -li.advantages * ratio
    l2 = -li.advantages * ratio.clamp(1 - cfg.clip_low, 1 + cfg.clip_high)
    d = li.logp - old
    if cfg.ppo_logps_ratio_clamp is not None:
        d = d.clamp(-cfg.ppo_logps_ratio_clamp, cfg.ppo_logps_ratio_clamp)
    abs_kl = d.abs()
    tl = torch.maximum(l1, l2)
    with torch.no_grad():
        cov, valid = _centered_cov(cfg, li)
        sel = torch.zeros_like(valid)
        n_valid = int(valid.sum())
        if n_valid > 0 and cfg.kl_cov_ratio > 0:
            k = max(1, int(n_valid * cfg.kl_cov_ratio))
            top = torch.topk(cov.masked_fill(~valid, float("-inf")), k).indices
            sel[top] = True
    tl = torch.where(sel, tl + cfg.kl_cov_coef * abs_kl, tl)
    return LossOutput(tl, ratio.detach(), {"ppo_ratio_clamped_frac": _frac(l2 > l1, li.mask),
                                           "ppo_abs_kl": torch.stack([(abs_kl.detach() * li.mask).sum(), li.mask.sum()]),
                                           "kl_cov_frac": _frac(sel, li.mask),
                                           "cov_mean": torch.stack([(cov * li.mask).sum(), li.mask.sum()])})


@register_loss("reinforce")
def reinforce_loss(cfg, li: LossInput) -> LossOutput:
    return LossOutput(-li.advantages * li.logp, torch.ones_like(li.logp), {})


@register_loss("opd")
def opd_loss(cfg, li: LossInput) -> LossOutput:
    """On-policy distillation: advantages already hold (teacher - student) log-prob gaps; clip like grpo."""
    return grpo_loss(cfg, li)


# ------------------------------------------------------------------------------------------------ shared terms
def kl_penalty(logp, ref_logp, kind: str = "k3", clamp: Optional[float] = None):
    """Estimators of KL(pi || ref) from samples of pi (gpatch_v4/utils/ppo_utils.py:151-193)."""
    d = ref_logp - logp
    if kind == "k1":
        kl = -d
    elif kind == "k2":
        kl = 0.5 * d * d
    else:
        kl = torch.exp(d) - d - 1
    if clamp is not None and clamp > 0:
        kl = kl.clamp(max=clamp) if kind == "k3" else kl.clamp(-clamp, clamp)
    return kl


def offpolicy_correction(cfg, old_logp, rollout_logp, mask, seq_ids, num_seqs):
    """Train-vs-rollout importance weights (gpatch_v4/core/correction_helper.py:238-420).
    Returns ``(weights [T] detached, metrics)``; ``weights`` multiply the actor loss."""
    with torch.no_grad():
        lr = (old_logp - rollout_logp).clamp(-20.0, 20.0)
        if cfg.offpolicy_correction_level == "token":
            w = lr.exp()
        else:
            lens = _seg_sum(mask, seq_ids, num_seqs).clamp_min(1.0)
            s = _seg_sum(lr * mask, seq_ids, num_seqs)
            if cfg.offpolicy_correction_level == "geometric":
                s = s / lens
            w = s.clamp(-20.0, 20.0).exp()[seq_ids.long()]
        upper = cfg.offpolicy_correction_upper
        lower = cfg.offpolicy_correction_lower if cfg.offpolicy_correction_lower is not None else 1.0 / upper
        mode = cfg.offpolicy_correction
        metrics = {"tis/weight_mean": torch.stack([(w * mask).sum(), mask.sum()]),
                   "tis/out_of_range_frac": _frac((w > upper) | (w < lower), mask)}
        if mode == "none":
            out = torch.ones_like(w)
        elif mode == "truncate":
            out = w.clamp(max=upper)
        elif mode == "clip":
            out = w.clamp(lower, upper)
        elif mode == "mask":
            out = torch.where((w >= lower) & (w <= upper), torch.ones_like(w), torch.zeros_like(w))
        elif mode == "icepop":
            out = torch.where((w >= lower) & (w <= upper), w, torch.zeros_like(w))
        elif mode == "kpop":
            # drop whole sequences whose geometric-mean weight leaves the band
            lens = _seg_sum(mask, seq_ids, num_seqs).clamp_min(1.0)
            g = (_seg_sum(lr * mask, seq_ids, num_seqs) / lens).exp()
            keep = ((g >= lower) & (g <= upper)).float()
            out = w.clamp(max=upper) * keep[seq_ids.long()]
        else:
            raise ValueError(mode)
        veto = cfg.offpolicy_correction_veto
        if veto is not None:
            bad = _seg_sum(((w < veto).float() * mask), seq_ids, num_seqs) > 0
            out = out * (~bad).float()[seq_ids.long()]
            metrics["tis/veto_frac"] = torch.stack([bad.float().sum(), bad.new_tensor(float(num_seqs)).float()])
    return out, metrics


def aggregation_weights(mask, seq_ids, num_seqs, per_token: bool, denom: float):
    """Weights ``w`` such that ``sum(w * token_loss)`` is this micro-batch's share of the global loss.
    per-token: ``mask / global_token_count``; else per-sequence masked means over ``global_alive_sequences``
    (gpatch_v4/training_backend/loss/utils.py:8-55, megatron_backend/mixin.py:1949-1983)."""
    if per_token:
        return mask / max(denom, 1.0)
    lens = _seg_sum(mask, seq_ids, num_seqs).clamp_min(1.0)
    return mask / lens[seq_ids.long()] / max(denom, 1.0)


def square_averaging_weights(mask, seq_ids, num_seqs, denom: float):
    """Weights of the square-averaging cross-entropy: a token of a sequence with N answer tokens counts 1 / sqrt(N),
    normalised by the global sum of sqrt(N) over sequences (``denom``), so that short answers are not drowned by
    long ones (gpatch_v4/training_backend/loss_factory.py:3199-3290)."""
    lens = _seg_sum(mask, seq_ids, num_seqs).clamp_min(1.0)
    return mask / lens.sqrt()[seq_ids.long()] / max(denom, 1.0)


def value_loss(values, old_values, returns, mask_w, clip: Optional[float]):
    """0.5 * max((clip(V) - R)^2, (V - R)^2) (gpatch_v4/training_backend/loss_factory.py:3355-3371)."""
    l1 = (values - returns) ** 2
    if clip is not None and clip > 0:
        vc = old_values + (values - old_values).clamp(-clip, clip)
        l1 = torch.maximum(l1, (vc - returns) ** 2)
    return 0.5 * (l1 * mask_w).sum()


def dpo_loss(pol_chosen, pol_rejected, ref_chosen, ref_rejected, beta: float, label_smoothing: float = 0.0,
             reference_free: bool = False):
    """Sequence log-prob sums -> DPO loss and reward accuracies."""
    pi = pol_chosen - pol_rejected
    ref = torch.zeros_like(pi) if reference_free else ref_chosen - ref_rejected
    logits = beta * (pi - ref)
    loss = -(torch.nn.functional.logsigmoid(logits) * (1 - label_smoothing)
             + torch.nn.functional.logsigmoid(-logits) * label_smoothing)
    return loss.mean(), {"dpo/reward_acc": (logits > 0).float().mean().detach(),
                         "dpo/margin": logits.detach().mean() / max(beta, 1e-12)}


def rm_bt_loss(score_chosen, score_rejected, margin: float = 0.0):
    """Bradley-Terry pairwise reward-model loss."""
    d = score_chosen - score_rejected - margin
    return -torch.nn.functional.logsigmoid(d).mean(), {"rm/acc": (d > 0).float().mean().detach()}
