"""Unified understanding + generation model and its pipeline: one decoder whose layers hold two sets of weights - an
understanding expert applied to text tokens and a generation expert applied to latent-image tokens - sharing one
attention over the packed sequence (text is causal; the latent tokens of an image see the text before them and each
other).  Trained with next-token cross-entropy on the text and the flow-matching loss on the latents, sampled as a
text-conditioned flow (with classifier-free guidance and its renormalisation), and tuned with GRPO over the
stochastic sampler like the diffusion pipelines.

Behavioural model: Bagel (gpatch_v4/extended_pipeline/pipeline_bagel.py:46-926; loss assembly :196-246: ``ce`` summed
over text tokens and divided by the global text-token count, ``mse`` averaged over channels, summed over latent tokens
and divided by the global latent-token count, weighted by ``ce_weight`` / ``mse_weight``; guidance merge with
``cfg_renorm_type`` global / channel :526-546).
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..models.dit import (ByteTokenizer, LatentAutoencoder, Linear, RMSNorm, latent_image_ids, pack_latents,
                          timestep_embedding, unpack_latents)
from .base import ExtendedPipeline, unbind_to_list
from .scheduling import (clipped_policy_loss, flow_matching_target, sample_training_sigmas, sde_step,
                         sigma_schedule)


class _Expert(nn.Module):
    def __init__(self, d, heads, ffn):
        super().__init__()
        self.ln1, self.ln2 = RMSNorm(d), RMSNorm(d)
        self.qkv, self.proj = Linear(d, 3 * d), Linear(d, d)
        self.fc1, self.fc2 = Linear(d, 2 * ffn, bias=False), Linear(ffn, d, bias=False)


class MoTLayer(nn.Module):
    """Mixture-of-transformers layer: per-token choice of expert weights, one shared attention."""

    def __init__(self, d, heads, ffn):
        super().__init__()
        self.d, self.h = d, heads
        self.und, self.gen = _Expert(d, heads, ffn), _Expert(d, heads, ffn)

    def _route(self, x, is_gen, fn_und, fn_gen):
        out = torch.empty(*x.shape[:-1], fn_und.weight.shape[0], dtype=x.dtype, device=x.device)
        if (~is_gen).any():
            out[~is_gen] = fn_und(x[~is_gen])
        if is_gen.any():
            out[is_gen] = fn_gen(x[is_gen])
        return out

    def forward(self, x, is_gen, mask, rope):
        """x [T, d] packed tokens of one sample; is_gen [T] bool; mask [T, T] bool (True = may attend)."""
        T, d = x.shape
        H, D = self.h, d // self.h
        h1 = torch.where(is_gen[:, None], self.gen.ln1(x), self.und.ln1(x))
        qkv = self._route(h1, is_gen, self.und.qkv, self.gen.qkv).view(T, 3, H, D)
        q, k, v = qkv.unbind(1)
        cos, sin = rope
        q, k = _rope1d(q, cos, sin), _rope1d(k, cos, sin)
        a = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
                                           attn_mask=mask[None, None])[0].transpose(0, 1).reshape(T, d)
        x = x + self._route(a, is_gen, self.und.proj, self.gen.proj)
        h2 = torch.where(is_gen[:, None], self.gen.ln2(x), self.und.ln2(x))
        gu = self._route(h2, is_gen, self.und.fc1, self.gen.fc1)
        g, u = gu.chunk(2, -1)
        return x + self._route(F.silu(g) * u, is_gen, self.und.fc2, self.gen.fc2)


def _rope1d(x, cos, sin):
    xf = x.float()
    a, b = xf[..., ::2], xf[..., 1::2]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.stack([a * c - b * s, a * s + b * c], -1).reshape(x.shape).to(x.dtype)


class BagelModel(nn.Module):
    def __init__(self, vocab, d, layers, heads, latent_dim, max_latent_side=64):
        super().__init__()
        self.d, self.heads = d, heads
        self.embed = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList(MoTLayer(d, heads, 2 * d) for _ in range(layers))
        self.norm_und, self.norm_gen = RMSNorm(d), RMSNorm(d)
        self.lm_head = Linear(d, vocab, bias=False)
        self.vae2llm, self.llm2vae = Linear(latent_dim, d), Linear(d, latent_dim, zero=True)
        self.time_in = nn.Sequential(Linear(256, d), nn.SiLU(), Linear(d, d))
        self.latent_pos = nn.Embedding(max_latent_side * max_latent_side, d)
        self.max_latent_side = max_latent_side

    def forward(self, text_ids, latents=None, sigma=None, latent_hw=None):
        """One sample: ``text_ids`` [Tt]; optional noisy ``latents`` [N, C] at noise level ``sigma`` (scalar tensor)
        placed after the text.  Returns (text logits [Tt, V], velocity [N, C] or None)."""
        x = self.embed(text_ids)
        Tt = x.shape[0]
        is_gen = torch.zeros(Tt, dtype=torch.bool, device=x.device)
        pos = torch.arange(Tt, device=x.device)
        if latents is not None:
            N = latents.shape[0]
            h, w = latent_hw
            rows = torch.arange(h, device=x.device)[:, None].expand(h, w).reshape(-1)
            cols = torch.arange(w, device=x.device)[None, :].expand(h, w).reshape(-1)
            lx = (self.vae2llm(latents.to(x.dtype)) + self.time_in(timestep_embedding(sigma.reshape(1), 256).to(x.dtype))
                  + self.latent_pos(rows * self.max_latent_side + cols))
            x = torch.cat([x, lx], 0)
            is_gen = torch.cat([is_gen, torch.ones(N, dtype=torch.bool, device=x.device)])
            pos = torch.cat([pos, torch.full((N,), Tt, device=x.device)])   # an image occupies one rope position
        T = x.shape[0]
        mask = torch.tril(torch.ones(T, T, dtype=torch.bool, device=x.device))
        if latents is not None:
            mask[Tt:, Tt:] = True          # latent tokens of the image attend to each other in both directions
        D = self.d // self.heads
        inv = 10000.0 ** (-torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D)
        ang = pos.float()[:, None] * inv[None]
        rope = (ang.cos(), ang.sin())
        for layer in self.layers:
            x = layer(x, is_gen, mask, rope)
        logits = self.lm_head(self.norm_und(x[:Tt]))
        vel = self.llm2vae(self.norm_gen(x[Tt:])) if latents is not None else None
        return logits, vel


class BagelPipeline(ExtendedPipeline):
    # ------------------------------------------------------------------ construction
    def setup_pipeline(self) -> int:
        cfg, mc, t = self.config, self.config.model, self.config.training
        torch.manual_seed(t.seed)
        self.tokenizer = ByteTokenizer()
        self.latent_dim = mc.latent_channels * 4
        self.model = BagelModel(mc.lm_vocab_size, mc.lm_hidden_size, mc.lm_layers, mc.lm_heads,
                                self.latent_dim).to(self.device)
        self.vae = LatentAutoencoder(mc.latent_channels, mc.vae_base_channels, mc.vae_factor).to(self.device).eval()
        for p in self.vae.parameters():
            p.requires_grad_(False)
        if dist.is_initialized() and dist.get_world_size() > 1:
            for p in self.model.parameters():
                dist.broadcast(p.data, src=0)
        self.build_optimizer(self.model)
        self.sigma_schedule, self.timesteps = sigma_schedule(t.shift, t.sampling_steps)
        self.sampling_steps = t.sampling_steps
        ck = cfg.checkpoint
        if ck.load_ckpt_path or (t.save_interval and ck.save_ckpt_path):
            return self.load_checkpoint(ck.load_ckpt_path or ck.save_ckpt_path)
        return 0

    def latent_hw(self):
        t, f = self.config.training, self.config.model.vae_factor
        return t.height // f // 2, t.width // f // 2     # packed 2 x 2 patches

    def encode_prompt(self, prompt: List[str], **kw):
        ids, mask = self.tokenizer(prompt, self.config.model.text_max_length)
        return [ids[i][mask[i]].to(self.device) for i in range(len(prompt))]

    def merge_uncond_predict(self, v_uncond, v_cond, scale: float, renorm: str = "global", renorm_min: float = 0.0):
        v = v_uncond + scale * (v_cond - v_uncond)
        dims = (0, 1) if renorm == "global" else (-1,)
        ratio = (torch.norm(v_cond, dim=dims, keepdim=True) / (torch.norm(v, dim=dims, keepdim=True) + 1e-8))
        return v * ratio.clamp(min=renorm_min, max=1.0)

    def _velocity(self, text_ids, latents, sigma):
        _, v = self.model(text_ids, latents, torch.as_tensor(sigma, device=self.device, dtype=torch.float32),
                          self.latent_hw())
        return v

    # ------------------------------------------------------------------ rollout
    @torch.no_grad()
    def __call__(self, prompt: List[str] = None, generator: Optional[torch.Generator] = None, **kw):
        t = self.config.training
        texts = self.encode_prompt(prompt)
        h, w = self.latent_hw()
        self.model.eval()
        uncond = torch.tensor([self.tokenizer.eos_id], device=self.device)
        rb = {k: [] for k in ("images", "text_ids", "latents", "next_latents", "log_probs", "timesteps")}
        steps = self.sampling_steps - 1
        for ids in texts:
            x = torch.randn(1, h * w, self.latent_dim, generator=generator).to(self.device)
            traj, lps, x0 = [x], [], x
            for si in range(self.sampling_steps):
                sig = float(self.sigma_schedule[si])
                v = self._velocity(ids, x[0], sig)
                if t.guidance_scale > 1:
                    v = self.merge_uncond_predict(self._velocity(uncond, x[0], sig), v, t.guidance_scale)
                x, x0, lp, _ = sde_step(v[None], x, self.sigma_schedule, si, t.eta, generator=generator)
                traj.append(x)
                lps.append(lp)
            tr = torch.cat(traj, 0)
            rb["images"].append(self.decode_to_images(x0)[0])
            rb["text_ids"].append(ids.cpu())
            rb["latents"].append(tr[:steps].cpu())
            rb["next_latents"].append(tr[1:steps + 1].cpu())
            rb["log_probs"].append(torch.cat(lps)[:steps].cpu())
            rb["timesteps"].append(self.timesteps[:steps].clone())
        return rb, {"images": rb["images"], "prompt": list(prompt)}

    @torch.no_grad()
    def decode_to_images(self, packed):
        h, w = self.latent_hw()
        return self.vae.decode(unpack_latents(packed.float(), 2 * h, 2 * w)).cpu()

    # ------------------------------------------------------------------ GRPO update
    def ppo_train_step(self, rollout_batches: List[Dict[str, Any]]) -> Dict[str, float]:
        t, ppo = self.config.training, self.config.ppo
        eps_lo = ppo.ppo_clip_ratio_low if ppo.ppo_clip_ratio_low is not None else ppo.ppo_ratio_eps
        eps_hi = ppo.ppo_clip_ratio_high if ppo.ppo_clip_ratio_high is not None else ppo.ppo_ratio_eps
        gas = t.train_gas_wo_timestep
        self.model.train()
        self.optimizer.zero_grad(set_to_none=True)
        out = {"policy/loss": [], "policy/ppo_ratio": [], "policy/grad_norm": []}
        uncond = torch.tensor([self.tokenizer.eos_id], device=self.device)
        for mi, d in enumerate(rollout_batches):
            ids = d["text_ids"].to(self.device)
            train_steps = max(int(d["timesteps"].shape[0] * t.timestep_fraction), 1)
            adv = torch.as_tensor(d["advantages"], device=self.device, dtype=torch.float32).reshape(1)
            for ti in range(train_steps):
                x = d["latents"][ti].to(self.device).float()
                nxt = d["next_latents"][ti].to(self.device).float()
                idx = int(d["perms"][ti])
                sig = float(self.sigma_schedule[idx])
                v = self._velocity(ids, x, sig)
                if t.guidance_scale > 1:
                    with torch.no_grad():
                        vu = self._velocity(uncond, x, sig)
                    v = self.merge_uncond_predict(vu, v, t.guidance_scale)
                lp = sde_step(v[None], x[None], self.sigma_schedule, idx, t.eta, prev_sample=nxt[None])[2]
                loss, ratio = clipped_policy_loss(adv, lp, d["log_probs"][ti:ti + 1].to(self.device).float(), eps_lo,
                                                  eps_hi, (ppo.adv_clip_min, ppo.adv_clip_max))
                (loss / (gas * train_steps)).backward()
                l, r = self.reduce_mean(loss.detach() / (gas * train_steps), ratio)
                out["policy/loss"].append(l)
                out["policy/ppo_ratio"].append(r)
            if (mi + 1) % gas == 0 or mi == len(rollout_batches) - 1:
                out["policy/grad_norm"].append(self.optimizer_step(self.model))
        return {k: sum(v) / max(len(v), 1) for k, v in out.items()}

    # ------------------------------------------------------------------ supervised step (text CE + flow MSE)
    def sft_train_step(self, rollout_batches: List[Dict[str, Any]]) -> Dict[str, float]:
        """Samples: ``caption`` (+ optional ``pixel_values`` to generate, optional ``answer`` text to predict).  Both
        losses are normalised by the global token counts of their kind."""
        t = self.config.training
        self.model.train()
        self.optimizer.zero_grad(set_to_none=True)
        n_ce = sum(max(len(self._text(m)) - 1, 0) for m in rollout_batches)
        n_mse = sum(self.latent_hw()[0] * self.latent_hw()[1] for m in rollout_batches if "pixel_values" in m)
        tot = torch.tensor([float(n_ce), float(n_mse)])
        world = 1
        if dist.is_initialized() and dist.get_world_size() > 1:
            world = dist.get_world_size()
            tt = tot.to(self.device) if dist.get_backend() == "nccl" else tot
            dist.all_reduce(tt)
            tot = tt.cpu()
        ce_sum, mse_sum = 0.0, 0.0
        for m in rollout_batches:
            ids = self._text(m).to(self.device)
            lat = sig = None
            if "pixel_values" in m:
                with torch.no_grad():
                    x0 = pack_latents(self.vae.encode(torch.as_tensor(m["pixel_values"])[None].to(self.device).float()))[0]
                sig = sample_training_sigmas(1, t.shift, device=self.device, scheme=t.noise_scheme)
                lat, target = flow_matching_target(x0[None], torch.randn_like(x0[None]), sig)
                lat, target = lat[0], target[0]
            logits, v = self.model(ids, lat, sig[0] if sig is not None else None, self.latent_hw())
            loss = 0.0
            if ids.numel() > 1:
                ce = F.cross_entropy(logits[:-1].float(), ids[1:], reduction="sum") * world / max(float(tot[0]), 1.0)
                loss = loss + t.ce_loss_weight * ce
                ce_sum += float(ce.detach())
            if v is not None:
                mse = (v.float() - target.float()).pow(2).mean(-1).sum() * world / max(float(tot[1]), 1.0)
                loss = loss + t.mse_loss_weight * mse
                mse_sum += float(mse.detach())
            loss.backward()
        norm = self.optimizer_step(self.model)
        ce_m, mse_m = self.reduce_mean(ce_sum, mse_sum)
        return {"ce": ce_m, "mse": mse_m, "grad_norm": norm, "train_loss": t.ce_loss_weight * ce_m +
                t.mse_loss_weight * mse_m}

    def _text(self, m):
        txt = m["caption"] + (m.get("answer") or "")
        ids, mask = self.tokenizer([txt], self.config.model.text_max_length)
        return ids[0][mask[0]]
