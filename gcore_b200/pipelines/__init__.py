"""Image-generation pipelines for reinforcement learning, preference training and supervised fine-tuning of
rectified-flow models (the reference's ``extended_pipeline`` package: Flux, Qwen-Image-Edit, Bagel;
gpatch_v4/extended_pipeline/__init__.py)."""
from .base import ExtendedPipeline
from .flux import FluxPipeline
from .qwen_image_edit import QwenImageEditPipeline
from .bagel import BagelPipeline

PIPELINES = {"flux": FluxPipeline, "flux_kontext": QwenImageEditPipeline, "qwen_image_edit": QwenImageEditPipeline,
             "bagel": BagelPipeline}


def get_pipeline(name: str):
    if name not in PIPELINES:
        raise KeyError(f"unknown pipeline {name!r}; known: {sorted(PIPELINES)}")
    return PIPELINES[name]
