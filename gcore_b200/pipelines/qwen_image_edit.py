"""Instruction-guided image editing: the source image's latent tokens ride behind the noisy tokens of the image being
generated, tagged by their own position ids (image index 1), and only the first block of outputs is the velocity.

Behavioural model: ``QwenImageEditPipeline`` / Flux-Kontext (gpatch_v4/extended_pipeline/pipeline_qwen_image_edit.py):
same rollout batch as the text-to-image pipeline plus the conditioning latents, same GRPO update, and the supervised
edit step (``train_t2i_edit_sft``) on (instruction, source image, edited image) triples.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..models.dit import latent_image_ids, pack_latents
from .flux import FluxPipeline


class QwenImageEditPipeline(FluxPipeline):
    cond_images = True

    def encode_condition(self, source_images: torch.Tensor):
        """[B, 3, H, W] in [-1, 1] -> (latent tokens [B, N, C], ids [N, 3] with image index 1)."""
        with torch.no_grad():
            lat = self.vae.encode(source_images.to(self.device).float())
        H, W = lat.shape[-2:]
        return pack_latents(lat), latent_image_ids(H, W, self.device, index=1)

    @torch.no_grad()
    def __call__(self, prompt: List[str] = None, image: Optional[torch.Tensor] = None, **kw):
        assert image is not None, "the edit pipeline needs the source image of every prompt"
        return super().__call__(prompt=prompt, cond=self.encode_condition(image), **kw)

    def _cond_from_batch(self, micro):
        src = torch.stack([torch.as_tensor(m["source_pixel_values"]) for m in micro])
        return self.encode_condition(src)
