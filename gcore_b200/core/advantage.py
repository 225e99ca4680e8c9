"""Advantage estimators behind a registry (``ppo.advantage_type``), operating on a list of per-sample dicts.

Definitions follow gpatch_v4/core/advantage_impl.py:37-873 and advantage_helper.py:204-676:
  grpo      A_i = (r_i - mean_g) / (std_g + eps), unbiased std over the prompt group, invalid samples excluded
            (empty group: mean 0 / std 1), broadcast over response tokens, returns = advantages
  gdpo      per-reward-head group normalisation, weighted sum, optional batch-norm over the batch
  ppo       GAE over per-token rewards with a critic's values (skipping masked tokens), returns = A + V
  reinforce r_i - mean(batch)
  identity  A = r
  on_policy_distill   per-token (teacher logp - student logp)
plus global whitening, clipping and a KL-to-reference penalty folded into per-token rewards.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

_REGISTRY: Dict[str, Callable] = {}


def register_advantage(name):
    def deco(fn):
        _REGISTRY[name] = fn
        return fn
    return deco


def get_advantage_fn(name: str) -> Callable:
    if name not in _REGISTRY:
        raise KeyError(f"unknown advantage_type '{name}'; registered: {sorted(_REGISTRY)}")
    return _REGISTRY[name]


def group_normalize(rewards: torch.Tensor, group_ids: torch.Tensor, sample_mask: Optional[torch.Tensor],
                    eps: float, norm_by_std: bool = True) -> torch.Tensor:
    """rewards [N]; group_ids [N] int; returns advantages [N] (0 for invalid samples)."""
    r = rewards.float()
    valid = torch.ones_like(r, dtype=torch.bool) if sample_mask is None else sample_mask.bool()
    G = int(group_ids.max().item()) + 1 if group_ids.numel() else 0
    gid = group_ids.long()
    vf = valid.float()
    cnt = torch.zeros(G).index_add_(0, gid, vf)
    s = torch.zeros(G).index_add_(0, gid, r * vf)
    mean = torch.where(cnt > 0, s / cnt.clamp_min(1), torch.zeros(G))
    dev = (r - mean[gid]) * vf
    ss = torch.zeros(G).index_add_(0, gid, dev * dev)
    std = torch.where(cnt > 1, (ss / (cnt - 1).clamp_min(1)).sqrt(), torch.ones(G))
    std = torch.where(cnt > 0, std, torch.ones(G))
    if norm_by_std:
        if bool(((cnt == 1) & True).any()):
            single = (cnt == 1)
            # a lone valid sample has no spread to normalise by
            std = torch.where(single, torch.ones(G), std)
        adv = dev / (std[gid] + eps)
    else:
        adv = dev
    return adv * vf


def _broadcast_over_tokens(samples: List[dict], adv: torch.Tensor, key="advantages"):
    for s, a in zip(samples, adv.tolist()):
        m = torch.as_tensor(s["mask"], dtype=torch.float32)
        s[key] = m * a
        s["returns"] = s[key].clone()


@register_advantage("grpo")
def grpo_advantage(samples: List[dict], cfg, **_):
    r = torch.tensor([float(torch.as_tensor(s["rewards"]).sum()) for s in samples])
    gid = torch.tensor([int(s["group_id"]) for s in samples])
    sm = torch.tensor([bool(s.get("sample_mask", True)) for s in samples])
    adv = group_normalize(r, gid, sm, cfg.grpo_advantage_epsilon, cfg.norm_adv_by_std_in_grpo)
    _broadcast_over_tokens(samples, adv)
    return samples


@register_advantage("gdpo")
def gdpo_advantage(samples: List[dict], cfg, **_):
    """Each reward head is group-normalised on its own, then heads are mixed with ``gdpo_reward_weights``."""
    heads = sorted({k for s in samples for k in (s.get("reward_dict") or {})})
    gid = torch.tensor([int(s["group_id"]) for s in samples])
    sm = torch.tensor([bool(s.get("sample_mask", True)) for s in samples])
    if not heads:
        return grpo_advantage(samples, cfg)
    total = torch.zeros(len(samples))
    for h in heads:
        r = torch.tensor([float(s["reward_dict"].get(h, 0.0)) for s in samples])
        total += cfg.gdpo_reward_weights.get(h, 1.0) * group_normalize(r, gid, sm, cfg.grpo_advantage_epsilon, True)
    valid = sm.float()
    n = valid.sum().clamp_min(1)
    mean = (total * valid).sum() / n
    var = (((total - mean) * valid) ** 2).sum() / n
    total = (total - mean) / (var.sqrt() + cfg.grpo_advantage_epsilon) * valid
    for s, a in zip(samples, total.tolist()):
        s["pre_bn_advantages"] = a
    _broadcast_over_tokens(samples, total)
    return samples


def _gdpo_combined(samples: List[dict], cfg):
    """Sum over reward heads of weight x (group-normalised head reward); None without per-head rewards."""
    heads = sorted({k for s in samples for k in (s.get("reward_dict") or {})})
    if not heads:
        return None
    gid = torch.tensor([int(s["group_id"]) for s in samples])
    sm = torch.tensor([bool(s.get("sample_mask", True)) for s in samples])
    total = torch.zeros(len(samples))
    for h in heads:
        r = torch.tensor([float(s["reward_dict"].get(h, 0.0)) for s in samples])
        total += cfg.gdpo_reward_weights.get(h, 1.0) * group_normalize(r, gid, sm, cfg.grpo_advantage_epsilon, True)
    return total, sm


def _sample_bn(total, sm, eps, group=None):
    """(x - mean) / (std + eps) over the valid samples - of all data-parallel ranks when ``group`` is given - with the
    unbiased standard deviation (1 for a single sample)."""
    valid = sm.float()
    st = torch.stack([(total * valid).sum(), (total * total * valid).sum(), valid.sum()]).double()
    if group is not None:
        import torch.distributed as dist
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
            t = st.to(dev)
            dist.all_reduce(t, group=group)
            st = t.cpu()
    n = float(st[2])
    mean = float(st[0]) / max(n, 1.0)
    std = math.sqrt(max(float(st[1]) - n * mean * mean, 0.0) / (n - 1.0)) if n > 1 else 1.0
    return (total - mean) / (std + eps) * valid, {"gdpo/bn_mean": mean, "gdpo/bn_std": std}


def _gdpo_variant(samples, cfg, bn: bool, dp_group):
    got = _gdpo_combined(samples, cfg)
    if got is None:
        return grpo_advantage(samples, cfg)
    total, sm = got
    for s, a in zip(samples, total.tolist()):
        s["pre_bn_advantages"] = a
    if bn:
        total, stats = _sample_bn(total, sm, cfg.grpo_advantage_epsilon, dp_group)
        for s in samples:
            s["advantage_stats"] = stats
    else:
        total = total * sm.float()
    _broadcast_over_tokens(samples, total)
    return samples


@register_advantage("gdpo_sample_bn")
def gdpo_sample_bn_advantage(samples: List[dict], cfg, dp_group=None, **_):
    """gdpo followed by a batch norm over the valid samples of the whole data-parallel batch."""
    return _gdpo_variant(samples, cfg, True, dp_group)


@register_advantage("group_gdpo")
def group_gdpo_advantage(samples: List[dict], cfg, **_):
    """Per-head group normalisation and mixing only (no batch statistics)."""
    return _gdpo_variant(samples, cfg, False, None)


@register_advantage("group_gdpo_sample_bn")
def group_gdpo_sample_bn_advantage(samples: List[dict], cfg, **_):
    """The batch norm uses this rank's samples only."""
    return _gdpo_variant(samples, cfg, True, None)


@register_advantage("reinforce")
def reinforce_advantage(samples: List[dict], cfg, **_):
    r = torch.tensor([float(torch.as_tensor(s["rewards"]).sum()) for s in samples])
    _broadcast_over_tokens(samples, r - r.mean())
    return samples


@register_advantage("identity")
def identity_advantage(samples: List[dict], cfg, **_):
    r = torch.tensor([float(torch.as_tensor(s["rewards"]).sum()) for s in samples])
    _broadcast_over_tokens(samples, r)
    return samples


@register_advantage("on_policy_distill")
def opd_advantage(samples: List[dict], cfg, **_):
    for s in samples:
        m = torch.as_tensor(s["mask"], dtype=torch.float32)
        s["advantages"] = (torch.as_tensor(s["teacher_logprobs"]).float() -
                           torch.as_tensor(s["logprobs"]).float()) * m
        s["returns"] = s["advantages"].clone()
    return samples


register_advantage("g_opd")(opd_advantage)


@register_advantage("ppo")
def gae_advantage(samples: List[dict], cfg, **_):
    """Sequence reward lands on the last response token; optional per-token rewards and KL penalty are added."""
    from ..ops.rl import gae
    S = max(len(s["mask"]) for s in samples)
    B = len(samples)
    R, V, M = torch.zeros(B, S), torch.zeros(B, S), torch.zeros(B, S)
    for i, s in enumerate(samples):
        m = torch.as_tensor(s["mask"], dtype=torch.float32)
        n = m.numel()
        M[i, :n] = m
        V[i, :n] = torch.as_tensor(s["values"], dtype=torch.float32)[:n]
        if s.get("per_token_rewards") is not None:
            R[i, :n] = torch.as_tensor(s["per_token_rewards"], dtype=torch.float32)[:n]
        nz = m.nonzero()
        if nz.numel():
            R[i, int(nz[-1])] += float(torch.as_tensor(s["rewards"]).sum())
        if cfg.ppo_initial_policy_kl_penalty and s.get("ref_logprobs") is not None:
            kl = torch.as_tensor(s["logprobs"]).float() - torch.as_tensor(s["ref_logprobs"]).float()
            R[i, :n] -= cfg.ppo_initial_policy_kl_penalty * kl[:n] * m
    adv, ret = gae(R, V, M, cfg.ppo_discount_factor, cfg.ppo_gae_lambda)
    for i, s in enumerate(samples):
        n = len(s["mask"])
        s["advantages"] = adv[i, :n].clone()
        s["returns"] = ret[i, :n].clone()
    return samples


def whiten_advantages(samples: List[dict], group=None, eps: float = 1e-8):
    """Global masked whitening with statistics reduced over the data-parallel group
    (gpatch_v4/utils/training_utils.py:2096-2166)."""
    tot = torch.zeros(3, dtype=torch.float64)
    for s in samples:
        a, m = s["advantages"].double(), torch.as_tensor(s["mask"], dtype=torch.float64)
        tot += torch.stack([(a * m).sum(), (a * a * m).sum(), m.sum()])
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        t = tot.float()
        if dist.get_backend(group) == "nccl":
            t = t.cuda()
        dist.all_reduce(t, group=group)
        tot = t.cpu().double()
    n = tot[2].clamp_min(1)
    mean = tot[0] / n
    var = (tot[1] / n - mean * mean).clamp_min(0)
    for s in samples:
        m = torch.as_tensor(s["mask"], dtype=torch.float32)
        s["original_advantages"] = s["advantages"].clone()
        s["advantages"] = ((s["advantages"] - float(mean)) / (float(var.sqrt()) + eps)) * m
    return samples


def clip_advantages(samples: List[dict], low: float, high: float):
    for s in samples:
        s["advantages"] = s["advantages"].clamp(low, high)
    return samples


def compute_advantages(samples: List[dict], ppo_cfg, dp_group=None, custom_fn: Optional[Callable] = None):
    for s in samples:
        if "mask" not in s:
            from .packing import response_mask
            s["mask"] = response_mask(int(s["prompt_length"]), len(s["tokens"]))
    fn = custom_fn if custom_fn is not None else get_advantage_fn(ppo_cfg.advantage_type)
    try:
        samples = fn(samples, ppo_cfg, dp_group=dp_group)
    except TypeError:   # plug-in functions with the two-argument signature
        samples = fn(samples, ppo_cfg)
    if ppo_cfg.whiten_advantages:
        samples = whiten_advantages(samples, dp_group)
    if ppo_cfg.advantage_clip:
        samples = clip_advantages(samples, ppo_cfg.advantage_clip_low, ppo_cfg.advantage_clip_high)
    if ppo_cfg.mask_negative_samples:
        for s in samples:
            if float(s["advantages"].sum()) < 0:
                s["advantages"] = torch.zeros_like(s["advantages"])
    return samples
