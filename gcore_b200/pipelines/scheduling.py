"""Flow-matching schedules and the stochastic sampler step whose transition density makes a denoising trajectory a
sequence of actions with log-probabilities (DanceGRPO-style; gpatch_v4/extended_pipeline/mixin.py:17-191).

Notation: ``sigma`` runs from 1 (noise) to 0 (image); the model predicts the velocity ``v = noise - x0`` at
``x_sigma = (1 - sigma) x0 + sigma noise``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def sd3_time_shift(shift: float, t: torch.Tensor) -> torch.Tensor:
    return (shift * t) / (1 + (shift - 1) * t)


def sigma_schedule(shift: float, sampling_steps: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (sigmas [steps + 1] from 1 to 0 after the SD3 shift, integer timesteps = sigma * 1000)."""
    s = sd3_time_shift(shift, torch.linspace(1, 0, sampling_steps + 1))
    return s, (s * 1000).to(torch.long)


def gaussian_log_prob(sample: torch.Tensor, mean: torch.Tensor, std: float) -> torch.Tensor:
    """Per-sample log density of ``sample`` under N(mean, std^2), averaged over all non-batch dimensions."""
    lp = (-((sample.detach().float() - mean.float()) ** 2) / (2 * std ** 2) - math.log(std)
          - 0.5 * math.log(2 * math.pi))
    return lp.mean(dim=tuple(range(1, lp.ndim)))


def sde_step(model_output: torch.Tensor, latents: torch.Tensor, sigmas: torch.Tensor, index: int, eta: float,
             prev_sample: Optional[torch.Tensor] = None, noise: Optional[torch.Tensor] = None,
             generator: Optional[torch.Generator] = None):
    """One reverse step ``sigma[index] -> sigma[index + 1]`` of the stochastic sampler.

    Mean = Euler step of the probability-flow ODE plus the score correction ``-0.5 eta^2 score dsigma``; standard
    deviation ``eta sqrt(sigma[index] - sigma[index + 1])``.  With ``prev_sample`` given nothing is drawn: the
    function returns the log-probability of that transition under the current model (the training pass).
    Returns ``(prev_sample, predicted x0, log_prob [B], noise)``.
    """
    v = model_output.float()
    assert latents.dtype == torch.float32
    sigma = float(sigmas[index])
    dsigma = float(sigmas[index + 1]) - sigma
    mean = latents + dsigma * v
    x0 = latents - sigma * v
    std = eta * math.sqrt(sigma - float(sigmas[index + 1]))
    score = -(latents - x0 * (1 - sigma)) / sigma ** 2
    mean = mean + (-0.5 * eta ** 2 * score) * dsigma
    if prev_sample is None:
        if noise is None:
            if generator is None:
                noise = torch.randn_like(mean)
            else:   # drawn where the generator lives, so a seeded rollout does not depend on the compute device
                noise = torch.randn(mean.shape, generator=generator, device=generator.device).to(mean.device)
        prev_sample = mean + noise * std
    return prev_sample, x0, gaussian_log_prob(prev_sample, mean, std), noise


def ode_step(model_output: torch.Tensor, latents: torch.Tensor, sigmas: torch.Tensor, index: int) -> torch.Tensor:
    return latents + (float(sigmas[index + 1]) - float(sigmas[index])) * model_output.float()


def clipped_policy_loss(advantages, logp, old_logp, eps_low: float, eps_high: float, adv_clip=(-5.0, 5.0)):
    """PPO-clip on per-transition log-probabilities; returns (mean loss, detached mean ratio)."""
    adv = advantages.clamp(adv_clip[0], adv_clip[1])
    ratio = torch.exp(logp - old_logp)
    loss = torch.maximum(-adv * ratio, -adv * ratio.clamp(1 - eps_low, 1 + eps_high)).mean()
    return loss, ratio.detach().mean()


def flow_matching_target(x0: torch.Tensor, noise: torch.Tensor, sigma: torch.Tensor):
    """-> (noisy sample at ``sigma``, velocity target) for the supervised flow-matching loss."""
    s = sigma.view(-1, *([1] * (x0.ndim - 1))).to(x0.dtype)
    return (1 - s) * x0 + s * noise, noise - x0


def sample_training_sigmas(n: int, shift: float, generator=None, device="cpu", scheme: str = "logit_normal"):
    """Training-time noise levels in (0, 1): logit-normal (SD3) or uniform, followed by the time shift."""
    if scheme == "logit_normal":
        u = torch.sigmoid(torch.randn(n, generator=generator))
    else:
        u = torch.rand(n, generator=generator)
    return sd3_time_shift(shift, u).clamp(1e-4, 1 - 1e-4).to(device)
