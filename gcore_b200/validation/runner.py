"""Validation during text-to-image training: a fixed list of cases is generated with the current weights (and with
the EMA weights when they exist), every image is scored against its caption and, for edit cases, against its source
image, results and metrics are written below ``<save dir>/step_XXXXXXX/`` and the aggregated metrics return to the
trainer's log.

Behaviour follows the reference's runner (gpatch_v4/validation/runner_base.py:20-302): cases come from a jsonl file
(or the first jsonl file of a directory) and are grouped into phases by ``task_type``; the case list is padded to a
multiple of the job size and sharded by rank; module train / eval modes are snapshotted and restored around the run;
rank 0 writes ``metrics.json``.  The similarity scorer (clip_metrics.py:8-100) is a CLIP model loaded from a local
directory when one is configured and loadable; otherwise the pipeline's own text encoder and a fixed random-projection
image embedder give a (much weaker, but deterministic and dependency-free) text-image / image-image similarity, so
that the plumbing and the trend over training can still be followed.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

PHASE_ORDER = ("t2i", "edit")


def snapshot_modes(module: torch.nn.Module) -> Dict[str, bool]:
    return {n: m.training for n, m in module.named_modules()}


def restore_modes(module: torch.nn.Module, snap: Dict[str, bool]):
    for n, m in module.named_modules():
        if n in snap:
            m.training = snap[n]


class EmbeddingMetrics:
    """Cosine similarity of caption and image embeddings (``text_image_score``) and of two images
    (``image_image_score``)."""

    def __init__(self, pipe=None, clip_path: Optional[str] = None, device="cpu", dim: int = 256, seed: int = 1234):
        self.pipe, self.clip_path, self.device, self.dim, self.seed = pipe, clip_path, torch.device(device), dim, seed
        self._clip = None
        self._proj = None

    def _load_clip(self):
        if self._clip is not None or not self.clip_path or not os.path.isdir(self.clip_path):
            return self._clip
        try:
            from transformers import CLIPModel, CLIPProcessor
            self._clip = (CLIPModel.from_pretrained(self.clip_path).to(self.device).eval(),
                          CLIPProcessor.from_pretrained(self.clip_path))
        except Exception:  # noqa: BLE001 - no usable checkpoint: the built-in embedder takes over
            self._clip = None
        return self._clip

    def _image_embed(self, img: torch.Tensor) -> torch.Tensor:
        """Built-in image embedder: 8 x 8 average-pooled pixels and their channel statistics through a fixed random
        projection."""
        x = img.float().to(self.device)
        if x.dim() == 3 and x.shape[0] not in (1, 3) and x.shape[-1] in (1, 3):
            x = x.permute(2, 0, 1)
        feat = torch.cat([F.adaptive_avg_pool2d(x[None], 8).reshape(-1), x.mean((1, 2)), x.std((1, 2))])
        if self._proj is None or self._proj.shape[1] != feat.numel():
            g = torch.Generator().manual_seed(self.seed)
            self._proj = (torch.randn(self.dim, feat.numel(), generator=g) / math.sqrt(feat.numel())).to(self.device)
        return F.normalize(self._proj @ feat, dim=0)

    def _text_embed(self, text: str) -> torch.Tensor:
        if self.pipe is not None:
            with torch.no_grad():
                _, pooled, _ = self.pipe.encode_prompt([text])
            e = pooled[0].float().to(self.device)
        else:
            g = torch.Generator().manual_seed(abs(hash(text)) % (1 << 31))
            e = torch.randn(self.dim, generator=g).to(self.device)
        if e.numel() != self.dim:
            g = torch.Generator().manual_seed(self.seed + 1)
            w = (torch.randn(self.dim, e.numel(), generator=g) / math.sqrt(e.numel())).to(self.device)
            e = w @ e
        return F.normalize(e, dim=0)

    @torch.no_grad()
    def text_image_score(self, text: str, image: torch.Tensor) -> float:
        clip = self._load_clip()
        if clip is not None:
            model, proc = clip
            from PIL import Image
            pil = Image.fromarray((image.clamp(0, 1).permute(1, 2, 0).cpu().numpy() * 255).astype("uint8"))
            out = model(**{k: v.to(self.device) for k, v in proc(text=[text], images=[pil], return_tensors="pt",
                                                                 padding=True, truncation=True, max_length=77).items()})
            return float(F.normalize(out.text_embeds, dim=-1) @ F.normalize(out.image_embeds, dim=-1).T)
        return float(self._text_embed(text) @ self._image_embed(image))

    @torch.no_grad()
    def image_image_score(self, a: torch.Tensor, b: torch.Tensor) -> float:
        return float(self._image_embed(a) @ self._image_embed(b))

    def cleanup(self):
        self._clip = None


class ValidationRunner:
    """``run(step)`` -> ``(metrics, save_root)``.  ``cases``: list of dicts with ``prompt`` and optionally
    ``task_type`` (``t2i`` | ``edit``) and ``source_image`` (tensor [3, H, W] for edit cases)."""

    def __init__(self, pipe, data_path: Optional[str] = None, save_dir: str = "val_results", cases: Optional[list] = None,
                 clip_path: Optional[str] = None, extra_reward=None):
        self.pipe, self.save_dir, self.extra_reward = pipe, save_dir, extra_reward
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.groups = self._group(cases if cases is not None else self._load(data_path))
        self.metrics_model = EmbeddingMetrics(pipe, clip_path, device=getattr(pipe, "device", "cpu"))

    @staticmethod
    def _load(path) -> list:
        if not path:
            return []
        if os.path.isdir(path):
            names = sorted(n for n in os.listdir(path) if n.endswith(".jsonl"))
            if not names:
                return []
            path = os.path.join(path, names[0])
        if not os.path.isfile(path):
            return []
        return [json.loads(line) for line in open(path, encoding="utf-8") if line.strip()]

    @staticmethod
    def _group(cases) -> Dict[str, list]:
        g = {p: [] for p in PHASE_ORDER}
        for c in cases:
            g["edit" if c.get("task_type") == "edit" else "t2i"].append(c)
        return {k: v for k, v in g.items() if v}

    def _shard(self, cases):
        n = math.ceil(len(cases) / self.world) * self.world
        padded = cases + [None] * (n - len(cases))      # every rank runs the same number of generations
        per = n // self.world
        return padded[self.rank * per:(self.rank + 1) * per]

    def run(self, step: int):
        if not self.groups:
            return {}, ""
        root = os.path.join(self.save_dir, f"step_{step:07d}")
        os.makedirs(root, exist_ok=True)
        metrics: Dict[str, float] = {}
        models = [("train", None)]
        ema = getattr(self.pipe, "ema", None)
        if ema is not None:
            models.append(("ema", ema))
        for tag, ema_state in models:
            snap = snapshot_modes(self.pipe.model)
            backup = None
            if ema_state is not None:   # evaluate the averaged weights, then put the live ones back
                backup = {k: v.detach().clone() for k, v in self.pipe.model.state_dict().items()}
                ema_state.copy_to(self.pipe.model)
            self.pipe.model.eval()
            try:
                for phase in PHASE_ORDER:
                    if phase in self.groups:
                        metrics.update(self._run_phase(self.groups[phase], phase, tag, os.path.join(root, tag)))
            finally:
                if backup is not None:
                    self.pipe.model.load_state_dict(backup)
                restore_modes(self.pipe.model, snap)
        if self.rank == 0:
            json.dump(metrics, open(os.path.join(root, "metrics.json"), "w"), indent=2)
        self.metrics_model.cleanup()
        if self.world > 1:
            dist.barrier()
        return metrics, root

    @torch.no_grad()
    def _run_phase(self, cases, phase: str, tag: str, out_dir: str) -> Dict[str, float]:
        os.makedirs(out_dir, exist_ok=True)
        mine = self._shard(cases)
        rows = []
        g = torch.Generator(device="cpu").manual_seed(4242)
        for k, case in enumerate(mine):
            live = case if case is not None else cases[0]    # padding cases generate too, but are not scored
            prompt = live["prompt"]
            kw = {}
            if phase == "edit" and live.get("source_image") is not None and hasattr(self.pipe, "encode_condition"):
                kw["cond"] = self.pipe.encode_condition(torch.as_tensor(live["source_image"])[None])
            rb, _ = self.pipe(prompt=[prompt], generator=g, **kw)
            img = rb["images"][0].float().cpu()
            if case is None:
                continue
            row = {"phase": phase, "prompt": prompt, "text_image": self.metrics_model.text_image_score(prompt, img)}
            if phase == "edit" and case.get("source_image") is not None:
                row["image_image"] = self.metrics_model.image_image_score(img, torch.as_tensor(case["source_image"]))
            if self.extra_reward is not None:
                row["reward"] = float(self.extra_reward([img], [prompt])[0])
            torch.save(img, os.path.join(out_dir, f"{phase}_r{self.rank}_{k}.pt"))
            rows.append(row)
        allrows = [rows]
        if self.world > 1:
            allrows = [None] * self.world
            dist.all_gather_object(allrows, rows)
        flat = [r for part in allrows for r in part]
        out = {}
        for key in ("text_image", "image_image", "reward"):
            vals = [r[key] for r in flat if key in r]
            if vals:
                out[f"val/{tag}/{phase}/{key}"] = sum(vals) / len(vals)
        out[f"val/{tag}/{phase}/cases"] = float(len(flat))
        return out
