"""Example of a user-supplied policy loss (``ppo.loss_func_py_path`` / ``loss_func_py_name``): the clipped GRPO
surrogate in which tokens with a positive advantage get a wider upper clip when the policy is still uncertain about
them (log-prob below a threshold) - exploration where the reward says "more of this" (the role of the reference's
tasks/math_rl_v4/epo_grpo_loss.py).  Called as ``fn(ppo_cfg, loss_input)`` per micro-batch; returns a ``LossOutput``
with the per-token loss (the engine applies mask, aggregation weights, KL to the reference and the entropy bonus)."""
import torch

from gcore_b200.loss.policy_loss import LossInput, LossOutput

UNCERTAIN_LOGP = -2.0     # tokens the policy gives less than e^-2 are "uncertain"
EXTRA_CLIP_HIGH = 0.2


def uncertainty_widened_clip_loss(cfg, li: LossInput) -> LossOutput:
    old = li.logp.detach() if li.old_logp is None else li.old_logp
    ratio = torch.exp((li.logp - old).clamp(-20.0, 20.0))
    widen = ((li.advantages > 0) & (old < UNCERTAIN_LOGP)).to(ratio.dtype)
    hi = 1.0 + cfg.clip_high + EXTRA_CLIP_HIGH * widen
    lo = torch.full_like(ratio, 1.0 - cfg.clip_low)
    clipped = torch.minimum(torch.maximum(ratio, lo), hi)
    l1, l2 = -li.advantages * ratio, -li.advantages * clipped
    loss = torch.maximum(l1, l2)
    m = li.mask
    n = m.sum().clamp_min(1.0)
    return LossOutput(loss, ratio.detach(), {
        "ppo_ratio_clamped_frac": torch.stack([((l2 > l1).to(m.dtype) * m).sum(), n]),
        "widened_clip_frac": torch.stack([(widen * m).sum(), n])})
