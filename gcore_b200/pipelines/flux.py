"""Text-to-image pipeline over the rectified-flow transformer: rollouts with per-step log-probabilities for GRPO,
the clipped policy update over a random subset of each trajectory's steps, and the supervised flow-matching step.

Behavioural model: ``FluxPipeline`` (gpatch_v4/extended_pipeline/pipeline_flux.py:32-584): ``__call__`` returns the
rollout batch ``{encoder_hidden_states, pooled_prompt_embeds, text_ids, image_ids, latents, next_latents, log_probs,
timesteps}`` (per-sample lists, trajectories without their last step) plus the reward request ``{images, prompt}``;
``ppo_train_step`` re-evaluates the stored transitions (``sde_step`` with ``prev_sample`` given) and applies the
clipped loss scaled by ``1 / (gas * train_timesteps)``.
"""
from __future__ import annotations

from contextlib import nullcontext
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..models.dit import (ByteTokenizer, DiTConfig, LatentAutoencoder, MMDiT, TextEncoder, latent_image_ids,
                          pack_latents, unpack_latents)
from .base import ExtendedPipeline, unbind_to_list
from .scheduling import (clipped_policy_loss, flow_matching_target, sample_training_sigmas, sde_step,
                         sigma_schedule)


class FluxPipeline(ExtendedPipeline):
    cond_images = False   # subclasses that condition on a source image set this

    # ------------------------------------------------------------------ construction
    def setup_pipeline(self) -> int:
        cfg, mc, t = self.config, self.config.model, self.config.training
        torch.manual_seed(t.seed)
        tcfg = dict(mc.transformer)
        tcfg.setdefault("in_channels", mc.latent_channels * 4)
        self.dit_cfg = DiTConfig(**tcfg)
        dt = self._dtype()
        self.model = MMDiT(self.dit_cfg).to(self.device, dt)
        self.model.gradient_checkpointing = t.gradient_checkpointing
        self.tokenizer = ByteTokenizer()
        self.text_encoder = TextEncoder(self.dit_cfg.text_dim, self.dit_cfg.pooled_dim, mc.text_layers).to(self.device)
        self.vae = LatentAutoencoder(mc.latent_channels, mc.vae_base_channels, mc.vae_factor).to(self.device)
        for mod, frozen in ((self.text_encoder, mc.freeze_text_encoder), (self.vae, mc.freeze_vae)):
            if frozen:
                mod.eval()
                for p in mod.parameters():
                    p.requires_grad_(False)
        if mc.state_dict_path:
            sd = torch.load(mc.state_dict_path, map_location=self.device, weights_only=False)
            self.model.load_state_dict(sd.get("transformer", sd))
            if "text_encoder" in sd:
                self.text_encoder.load_state_dict(sd["text_encoder"])
            if "vae" in sd:
                self.vae.load_state_dict(sd["vae"])
        if dist.is_initialized() and dist.get_world_size() > 1:
            for p in self.model.parameters():   # identical initial weights on every data-parallel rank
                dist.broadcast(p.data, src=0)
        self.build_optimizer(self.model)
        self.num_channels_latents = mc.latent_channels
        self.setup_scheduler_and_timesteps()
        ck = cfg.checkpoint
        if cfg.training.save_interval and ck.save_ckpt_path:
            return self.load_checkpoint(ck.save_ckpt_path)
        if ck.load_ckpt_path:
            return self.load_checkpoint(ck.load_ckpt_path)
        return 0

    def setup_scheduler_and_timesteps(self):
        t = self.config.training
        self.sampling_steps = t.sampling_steps
        self.sigma_schedule, self.timesteps = sigma_schedule(t.shift, t.sampling_steps)

    def _autocast(self):
        if self.config.training.use_torch_autocast and self.device.type == "cuda":
            return torch.autocast("cuda", torch.bfloat16)
        return nullcontext()

    # ------------------------------------------------------------------ text / latents
    @torch.no_grad()
    def encode_prompt(self, prompt: List[str], **kw):
        """-> (prompt_embeds [B, Nt, Dt], pooled [B, Dp], text_ids [Nt, 3])."""
        ids, mask = self.tokenizer(prompt, self.config.model.text_max_length)
        emb, pooled = self.text_encoder(ids.to(self.device), mask.to(self.device))
        text_ids = torch.zeros(emb.shape[1], 3, device=self.device)
        return emb, pooled, text_ids

    def latent_hw(self):
        t, f = self.config.training, self.config.model.vae_factor
        return t.height // f, t.width // f

    def prepare_latents(self, batch_size: int, generator: Optional[torch.Generator] = None,
                        same_per_group: int = 0):
        """Packed Gaussian start latents (fp32) and their position ids.  ``same_per_group = n``: the n samples of a
        prompt start from the same noise (``create_same_rng_for_same_prompt`` of the reference's rollout)."""
        H, W = self.latent_hw()
        C = self.num_channels_latents
        n = batch_size // same_per_group if same_per_group else batch_size
        z = torch.randn(n, C, H, W, generator=generator)
        if same_per_group:
            z = z.repeat_interleave(same_per_group, 0)
        return pack_latents(z).to(self.device, torch.float32), latent_image_ids(H, W, self.device)

    @torch.no_grad()
    def decode_to_images(self, packed: torch.Tensor) -> torch.Tensor:
        H, W = self.latent_hw()
        return self.vae.decode(unpack_latents(packed.float(), H, W)).cpu()

    def offload_encoder(self):
        self.text_encoder.to("cpu")

    def onload_encoder(self):
        self.text_encoder.to(self.device)

    # ------------------------------------------------------------------ model call
    def _velocity(self, latents, timestep_int, prompt_embeds, pooled, text_ids, img_ids, guidance=None, cond=None):
        """``cond = (tokens [B, Nc, C], ids [Nc, 3])`` are appended behind the noisy tokens (edit pipelines)."""
        x = latents.to(self._dtype())
        ids = img_ids
        if cond is not None:
            x = torch.cat([x, cond[0].to(x.dtype)], 1)
            ids = torch.cat([img_ids, cond[1]], 0)
        with self._autocast():
            v = self.model(hidden_states=x, encoder_hidden_states=prompt_embeds, timestep=timestep_int.float() / 1000,
                           pooled_projections=pooled, img_ids=ids, txt_ids=text_ids, guidance=guidance)
        return v[:, :latents.shape[1]]

    def _guidance(self, n):
        if not self.dit_cfg.guidance_embeds:
            return None
        return torch.full((n,), self.config.training.guidance_scale, device=self.device, dtype=torch.float32)

    # ------------------------------------------------------------------ rollout
    @torch.no_grad()
    def __call__(self, prompt: List[str] = None, prompt_embeds=None, pooled_prompt_embeds=None, text_ids=None,
                 generator: Optional[torch.Generator] = None, cond=None, **kw):
        """One stochastic trajectory per entry of ``prompt`` (callers repeat prompts ``sampling_repeat_n`` times).
        Returns ``(rollout batch, reward request)``."""
        t = self.config.training
        if prompt_embeds is None:
            prompt_embeds, pooled_prompt_embeds, text_ids = self.encode_prompt(prompt)
        B = prompt_embeds.shape[0]
        latents, img_ids = self.prepare_latents(B, generator, t.sampling_repeat_n if t.same_noise_for_same_prompt
                                                and B % t.sampling_repeat_n == 0 else 0)
        self.setup_scheduler_and_timesteps()
        self.model.eval()
        guidance = self._guidance(B)
        all_latents, all_lp = [latents], []
        mbs = t.rollout_model_mbs or B
        x0 = latents
        for si in range(self.sampling_steps):
            ts = torch.full((B,), int(self.timesteps[si]), device=self.device, dtype=torch.long)
            v = torch.cat([self._velocity(latents[a:a + mbs], ts[a:a + mbs], prompt_embeds[a:a + mbs],
                                          pooled_prompt_embeds[a:a + mbs], text_ids, img_ids,
                                          None if guidance is None else guidance[a:a + mbs],
                                          None if cond is None else (cond[0][a:a + mbs], cond[1]))
                           for a in range(0, B, mbs)])
            latents, x0, lp, _ = sde_step(v, latents, self.sigma_schedule, si, t.eta, generator=generator)
            all_latents.append(latents)
            all_lp.append(lp)
        traj = torch.stack(all_latents, 1)             # [B, steps + 1, N, C]
        lps = torch.stack(all_lp, 1)                   # [B, steps]
        images = self.decode_to_images(x0)             # the last step's clean prediction, as the reference decodes
        # the last transition is dropped: its standard deviation shrinks to 0 with the final sigma step
        steps = self.sampling_steps - 1
        rb = {
            "images": unbind_to_list(images),
            "encoder_hidden_states": unbind_to_list(prompt_embeds.cpu()),
            "pooled_prompt_embeds": unbind_to_list(pooled_prompt_embeds.cpu()),
            "text_ids": [text_ids.cpu() for _ in range(B)],
            "image_ids": [img_ids.cpu() for _ in range(B)],
            "latents": unbind_to_list(traj[:, :steps].cpu()),
            "next_latents": unbind_to_list(traj[:, 1:steps + 1].cpu()),
            "log_probs": unbind_to_list(lps[:, :steps].cpu()),
            "timesteps": [self.timesteps[:steps].clone() for _ in range(B)],
        }
        if cond is not None:
            rb["cond_latents"] = unbind_to_list(cond[0].cpu())
            rb["cond_ids"] = [cond[1].cpu() for _ in range(B)]
        return rb, {"images": rb["images"], "prompt": list(prompt) if prompt is not None else None}

    # ------------------------------------------------------------------ GRPO update
    def prepare_data_for_training(self, micro: List[Dict[str, Any]]):
        keys = ["encoder_hidden_states", "pooled_prompt_embeds", "text_ids", "image_ids", "latents", "next_latents",
                "log_probs", "timesteps", "advantages", "perms"]
        if "cond_latents" in micro[0]:
            keys += ["cond_latents", "cond_ids"]
        return {k: torch.stack([torch.as_tensor(d[k]) for d in micro]).to(self.device, non_blocking=True) for k in keys}

    def ppo_train_step(self, rollout_batches: List[Dict[str, Any]]) -> Dict[str, float]:
        """``rollout_batches``: per-sample dicts (one trajectory each) with ``advantages`` and ``perms`` filled in.
        Micro-batches of ``train_mbs`` trajectories; an optimizer step every ``train_gas_wo_timestep`` micro-batches."""
        t, ppo = self.config.training, self.config.ppo
        gas = t.train_gas_wo_timestep
        self.model.train()
        self.optimizer.zero_grad(set_to_none=True)
        eps_lo = ppo.ppo_clip_ratio_low if ppo.ppo_clip_ratio_low is not None else ppo.ppo_ratio_eps
        eps_hi = ppo.ppo_clip_ratio_high if ppo.ppo_clip_ratio_high is not None else ppo.ppo_ratio_eps
        metrics: Dict[str, List[float]] = {"policy/loss": [], "policy/ppo_ratio": [], "policy/grad_norm": []}
        micros = [rollout_batches[i:i + t.train_mbs] for i in range(0, len(rollout_batches), t.train_mbs)]
        for mi, micro in enumerate(micros):
            d = self.prepare_data_for_training(micro)
            n = d["latents"].shape[0]
            guidance = self._guidance(n)
            train_steps = max(int(d["timesteps"].shape[1] * t.timestep_fraction), 1)
            cond = (d["cond_latents"], d["cond_ids"][0]) if "cond_latents" in d else None
            for ti in range(train_steps):
                x, nxt = d["latents"][:, ti].float(), d["next_latents"][:, ti].float()
                v = self._velocity(x, d["timesteps"][:, ti], d["encoder_hidden_states"], d["pooled_prompt_embeds"],
                                   d["text_ids"][0], d["image_ids"][0], guidance, cond)
                lp = torch.cat([sde_step(v[i:i + 1], x[i:i + 1], self.sigma_schedule, int(d["perms"][i, ti]), t.eta,
                                         prev_sample=nxt[i:i + 1])[2] for i in range(n)])
                loss, ratio = clipped_policy_loss(d["advantages"].float().reshape(-1), lp, d["log_probs"][:, ti].float(),
                                                  eps_lo, eps_hi, (ppo.adv_clip_min, ppo.adv_clip_max))
                (loss / (gas * train_steps)).backward()
                l, r = self.reduce_mean(loss.detach() / (gas * train_steps), ratio)
                metrics["policy/loss"].append(l)
                metrics["policy/ppo_ratio"].append(r)
            if (mi + 1) % gas == 0 or mi == len(micros) - 1:
                metrics["policy/grad_norm"].append(self.optimizer_step(self.model))
        return {k: sum(v) / max(len(v), 1) for k, v in metrics.items()}

    # ------------------------------------------------------------------ supervised flow matching
    def encode_images(self, images: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            return pack_latents(self.vae.encode(images.to(self.device).float()))

    def sft_train_step(self, rollout_batches: List[Dict[str, Any]]) -> Dict[str, float]:
        """``rollout_batches``: dicts with ``caption`` (str) and ``pixel_values`` [3, H, W] in [-1, 1] (edit pipelines:
        also ``source_pixel_values``).  Loss: mean squared error against the velocity target at a random noise
        level."""
        t = self.config.training
        self.model.train()
        gas = max(t.gradient_accumulation_steps, 1)
        micros = [rollout_batches[i:i + t.train_mbs] for i in range(0, len(rollout_batches), t.train_mbs)]
        losses, norms = [], []
        for mi, micro in enumerate(micros):
            emb, pooled, text_ids = self.encode_prompt([m["caption"] for m in micro])
            x0 = self.encode_images(torch.stack([torch.as_tensor(m["pixel_values"]) for m in micro]))
            cond = self._cond_from_batch(micro)
            sig = sample_training_sigmas(x0.shape[0], t.shift, device=self.device, scheme=t.noise_scheme)
            xt, target = flow_matching_target(x0, torch.randn_like(x0), sig)
            H, W = self.latent_hw()
            v = self._velocity(xt, sig * 1000, emb, pooled, text_ids, latent_image_ids(H, W, self.device),
                               self._guidance(x0.shape[0]), cond)
            loss = torch.nn.functional.mse_loss(v.float(), target.float())
            (loss / gas).backward()
            losses.append(self.reduce_mean(loss.detach())[0])
            if (mi + 1) % gas == 0 or mi == len(micros) - 1:
                norms.append(self.optimizer_step(self.model))
        return {"train_loss": sum(losses) / len(losses), "grad_norm": sum(norms) / max(len(norms), 1)}

    def _cond_from_batch(self, micro):
        return None
