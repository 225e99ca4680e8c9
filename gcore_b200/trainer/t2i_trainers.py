"""Trainers of the image-generation family.

* ``T2iGrpoTrainer``  - rollout (n trajectories per prompt) -> rewards (rule function and / or reward models, mixed by
  weight) -> group-normalised advantages -> clipped update over a random subset of every trajectory's steps
  (gpatch_v4/actor/t2i_grpo_train_actor.py:229-313,435-460, trainer/t2i_grpo_trainer.py).
* ``T2iDpoTrainer``   - Diffusion-DPO on (caption, preferred image, rejected image): both images share noise and
  noise level, the implicit reward is the drop in denoising error against a frozen reference copy; ``train_method:
  sft`` trains the plain flow-matching loss on the preferred image (trainer/t2i_dpo_trainer.py:78-151).
* ``T2iEditSftTrainer`` - supervised edit triples (trainer/t2i_edit_sft_trainer.py).
* ``BagelTrainer``    - unified model: text cross-entropy + flow loss, periodic validation, EMA, checkpoints
  (trainer/omni_base_trainer.py:297-554).

Data comes from ``data.py_path`` / ``data.fn_name`` (``fn(config, dp_rank, dp_size) -> iterable of batches``) or, when
none is configured, from the synthetic sets below (coloured-rectangle images with captions naming the colour), which
give a learnable signal without any download.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, Iterator, List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..configs.base import import_from_path
from ..pipelines import get_pipeline
from ..pipelines.scheduling import flow_matching_target, sample_training_sigmas
from ..utils.logging_utils import get_logger

COLOURS = {"red": (1.0, -1.0, -1.0), "green": (-1.0, 1.0, -1.0), "blue": (-1.0, -1.0, 1.0),
           "white": (1.0, 1.0, 1.0), "black": (-1.0, -1.0, -1.0), "yellow": (1.0, 1.0, -1.0)}


def _dp():
    if dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def synthetic_image(colour: str, h: int, w: int, g: torch.Generator) -> torch.Tensor:
    img = torch.full((3, h, w), -0.2) + 0.05 * torch.randn(3, h, w, generator=g)
    y0, x0 = int(torch.randint(0, h // 2, (1,), generator=g)), int(torch.randint(0, w // 2, (1,), generator=g))
    c = torch.tensor(COLOURS[colour])[:, None, None]
    img[:, y0:y0 + h // 2, x0:x0 + w // 2] = c
    return img.clamp(-1, 1)


def synthetic_t2i_batches(config, kind: str, rank: int, world: int) -> Iterator[List[dict]]:
    """kind: prompts | pairs (caption, image) | prefs (caption, chosen, rejected) | edits (caption, source, target)."""
    t = config.training
    g = torch.Generator().manual_seed(t.seed * 7919 + rank)
    names = sorted(COLOURS)
    per_rank = max(t.rollout_gbs // world, 1) if kind == "prompts" else max(t.train_gbs_wo_timestep // world, 1)
    while True:
        batch = []
        for _ in range(per_rank):
            a, b = (names[int(i)] for i in torch.randperm(len(names), generator=g)[:2])
            cap = f"a {a} square"
            if kind == "prompts":
                batch.append({"caption": cap, "colour": a})
            elif kind == "pairs":
                batch.append({"caption": cap, "pixel_values": synthetic_image(a, t.height, t.width, g)})
            elif kind == "prefs":
                batch.append({"caption": cap, "pixel_values": synthetic_image(a, t.height, t.width, g),
                              "rejected_pixel_values": synthetic_image(b, t.height, t.width, g)})
            else:
                batch.append({"caption": f"make it {a}", "source_pixel_values": synthetic_image(b, t.height, t.width, g),
                              "pixel_values": synthetic_image(a, t.height, t.width, g)})
        yield batch


def colour_reward(images: List[torch.Tensor], prompts: List[str], **_) -> torch.Tensor:
    """Rule reward of the synthetic task: how close the image's mean colour is to the colour the caption names."""
    out = []
    for img, p in zip(images, prompts):
        target = next((torch.tensor(c) for n, c in COLOURS.items() if n in p), torch.zeros(3))
        out.append(-float((img.float().mean((1, 2)) - target).pow(2).mean()))
    return torch.tensor(out)


class _Base:
    kind = "pairs"

    def __init__(self, config, data_fn: Optional[Callable] = None):
        self.cfg = config
        self.log = get_logger(type(self).__name__)
        self.pipe = get_pipeline(config.model.pipeline)(config)
        self.data_fn = data_fn
        self.history: List[Dict[str, float]] = []

    def setup(self):
        self.step = self.pipe.setup_pipeline()
        rank, world = _dp()
        fn = self.data_fn
        if fn is None and self.cfg.data.py_path:
            fn = import_from_path(self.cfg.data.py_path, self.cfg.data.fn_name or "build_dataset")
        self.batches = iter(fn(self.cfg, rank, world)) if fn is not None else \
            synthetic_t2i_batches(self.cfg, self.kind, rank, world)
        return self

    def maybe_save(self):
        t, ck = self.cfg.training, self.cfg.checkpoint
        if t.save_interval and ck.save_ckpt_path and self.step % t.save_interval == 0:
            self.pipe.save_checkpoint(ck.save_ckpt_path, self.step)

    def total_steps(self):
        return self.cfg.training.total_training_step

    def generation_validation(self) -> Dict[str, float]:
        """Every ``training.eval_interval`` steps, when ``data.eval_data_path`` names validation cases: generate them
        with the current weights and score caption / image similarity (``validation/runner.py``)."""
        path = getattr(self.cfg.data, "eval_data_path", None)
        ev = self.cfg.training.eval_interval
        if not (path and ev and (self.step + 1) % ev == 0 and callable(getattr(self.pipe, "__call__", None))):
            return {}
        if getattr(self, "_val_runner", None) is None:
            from ..validation import ValidationRunner
            root = os.path.join(self.cfg.checkpoint.save_ckpt_path or self.cfg.report.log_dir or ".", "val_results")
            self._val_runner = ValidationRunner(self.pipe, data_path=path, save_dir=root)
        return self._val_runner.run(self.step + 1)[0]

    def run(self):
        while self.step < self.total_steps():
            m = self.train_one_step()
            m.update(self.generation_validation())
            self.step += 1
            self.history.append(m)
            if _dp()[0] == 0:
                self.log.info(f"step {self.step} " + " ".join(f"{k}={v:.5g}" for k, v in m.items()))
            self.maybe_save()
        return self.history


class T2iGrpoTrainer(_Base):
    kind = "prompts"

    def __init__(self, config, data_fn=None, reward_fns: Optional[Dict[str, Callable]] = None):
        super().__init__(config, data_fn)
        self.reward_fns = reward_fns

    def setup(self):
        super().setup()
        if self.reward_fns is None:
            b = self.cfg.bt_rm
            if b.rule_py_path:
                self.reward_fns = {"rule": import_from_path(b.rule_py_path, b.rule_fn_name or "reward_fn")}
            else:
                self.reward_fns = {"colour": colour_reward}
        return self

    def total_steps(self):
        return self.cfg.training.total_ppo_step

    def calculate_advantage(self, rewards: Dict[str, torch.Tensor], n: int) -> torch.Tensor:
        """Every reward is normalised inside its prompt group ((r - mean) / (std + eps), unbiased std), then the
        normalised rewards are mixed by ``ppo.reward_weights`` (actor/t2i_grpo_train_actor.py:229-313)."""
        eps = self.cfg.ppo.grpo_advantage_epsilon
        w = self.cfg.ppo.reward_weights
        total = None
        for name, r in rewards.items():
            g = r.float().view(-1, n)
            a = (g - g.mean(1, keepdim=True)) / (g.std(1, keepdim=True, unbiased=True) + eps) if n > 1 else g * 0
            a = a.reshape(-1) * float(w.get(name, 1.0))
            total = a if total is None else total + a
        return total

    def rollout(self, batch: List[dict]):
        t = self.cfg.training
        n = t.sampling_repeat_n
        prompts = [b["caption"] for b in batch for _ in range(n)]
        g = torch.Generator().manual_seed(t.seed + 1000003 * self.step + _dp()[0])
        kw = {}
        if getattr(self.pipe, "cond_images", False):
            kw["image"] = torch.stack([torch.as_tensor(b["source_pixel_values"]) for b in batch for _ in range(n)])
        rb, req = self.pipe(prompt=prompts, generator=g, **kw)
        rewards = {k: torch.as_tensor(fn(req["images"], req["prompt"]), dtype=torch.float32)
                   for k, fn in self.reward_fns.items()}
        adv = self.calculate_advantage(rewards, n)
        rb["advantages"] = [a for a in adv]
        rb = self.pipe.permute_timesteps(rb, g)
        keys = [k for k in rb if k != "images"]
        samples = [{k: rb[k][i] for k in keys} for i in range(len(prompts))]
        return samples, rewards

    def train_one_step(self) -> Dict[str, float]:
        samples, rewards = self.rollout(next(self.batches))
        m = self.pipe.ppo_train_step(samples)
        for k, r in rewards.items():
            m[f"rollout-rewards/{k}"] = self.pipe.reduce_mean(r.mean())[0]
        return m


class T2iDpoTrainer(_Base):
    kind = "prefs"

    def setup(self):
        super().setup()
        if self.cfg.training.train_method == "dpo":
            self.ref = self.pipe.frozen_copy(self.pipe.model)
        return self

    def _errors(self, model, xt, target, sig, emb, pooled, text_ids):
        from ..models.dit import latent_image_ids
        H, W = self.pipe.latent_hw()
        saved, self.pipe.model = self.pipe.model, model
        try:
            v = self.pipe._velocity(xt, sig * 1000, emb, pooled, text_ids, latent_image_ids(H, W, self.pipe.device),
                                    self.pipe._guidance(xt.shape[0]))
        finally:
            self.pipe.model = saved
        return (v.float() - target.float()).pow(2).mean(dim=(1, 2))

    def train_one_step(self) -> Dict[str, float]:
        t, pipe = self.cfg.training, self.pipe
        batch = next(self.batches)
        if t.train_method == "sft":
            return pipe.sft_train_step(batch)
        pipe.model.train()
        pipe.optimizer.zero_grad(set_to_none=True)
        gas = max(t.gradient_accumulation_steps, 1)
        micros = [batch[i:i + t.train_mbs] for i in range(0, len(batch), t.train_mbs)]
        acc = {"train_loss": [], "model_mse": [], "ref_mse": [], "implicit_acc": []}
        for micro in micros:
            emb, pooled, text_ids = pipe.encode_prompt([m["caption"] for m in micro])
            xw = pipe.encode_images(torch.stack([torch.as_tensor(m["pixel_values"]) for m in micro]))
            xl = pipe.encode_images(torch.stack([torch.as_tensor(m["rejected_pixel_values"]) for m in micro]))
            n = xw.shape[0]
            # the preferred and the rejected image of a pair share the noise and the noise level
            sig = sample_training_sigmas(n, t.shift, device=pipe.device, scheme=t.noise_scheme)
            noise = torch.randn_like(xw)
            xt_w, tg_w = flow_matching_target(xw, noise, sig)
            xt_l, tg_l = flow_matching_target(xl, noise, sig)
            xt, tg = torch.cat([xt_w, xt_l]), torch.cat([tg_w, tg_l])
            e2, p2, s2 = torch.cat([emb, emb]), torch.cat([pooled, pooled]), torch.cat([sig, sig])
            err = self._errors(pipe.model, xt, tg, s2, e2, p2, text_ids)
            with torch.no_grad():
                ref_err = self._errors(self.ref, xt, tg, s2, e2, p2, text_ids)
            model_diff = err[:n] - err[n:]
            ref_diff = ref_err[:n] - ref_err[n:]
            inside = -0.5 * self.cfg.dpo.beta_dpo * (model_diff - ref_diff)
            loss = -F.logsigmoid(inside).mean()
            (loss / (gas * len(micros))).backward()
            vals = pipe.reduce_mean(loss.detach(), err.detach().mean(), ref_err.mean(), (inside > 0).float().mean())
            for k, v in zip(acc, vals):
                acc[k].append(v)
        out = {k: sum(v) / len(v) for k, v in acc.items()}
        out["grad_norm"] = pipe.optimizer_step(pipe.model)
        return out


class T2iEditSftTrainer(_Base):
    kind = "edits"

    def train_one_step(self) -> Dict[str, float]:
        return self.pipe.sft_train_step(next(self.batches))


class BagelTrainer(_Base):
    """Supervised training of the unified model with the shared loop's hooks: validation every ``eval_interval``
    steps (flow loss on held-out pairs at fixed noise levels) and EMA / checkpoint handling in the pipeline."""
    kind = "pairs"

    def validate(self) -> Dict[str, float]:
        pipe, t = self.pipe, self.cfg.training
        rank, world = _dp()
        held = next(synthetic_t2i_batches(self.cfg, "pairs", rank + 10007, world))
        pipe.model.eval()
        tot, cnt = 0.0, 0
        from ..models.dit import pack_latents
        with torch.no_grad():
            for m in held:
                ids = pipe._text(m).to(pipe.device)
                x0 = pack_latents(pipe.vae.encode(torch.as_tensor(m["pixel_values"])[None].to(pipe.device).float()))
                for s in (0.25, 0.5, 0.75):
                    sig = torch.tensor([s], device=pipe.device)
                    g = torch.Generator().manual_seed(17)
                    xt, tg = flow_matching_target(x0, torch.randn(x0.shape, generator=g).to(pipe.device), sig)
                    _, v = pipe.model(ids, xt[0], sig[0], pipe.latent_hw())
                    tot += float((v.float() - tg[0].float()).pow(2).mean())
                    cnt += 1
        return {"valid/mse": pipe.reduce_mean(tot / max(cnt, 1))[0]}

    def train_one_step(self) -> Dict[str, float]:
        m = self.pipe.sft_train_step(next(self.batches))
        ev = self.cfg.training.eval_interval
        if ev and (self.step + 1) % ev == 0:
            m.update(self.validate())
        return m
