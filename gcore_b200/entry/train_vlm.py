"""Vision-language entry points (the reference's VLM SFT and VLM GRPO mains): ``+task.vlm.mode=sft`` (default) trains
on (image, prompt, response) rows, ``+task.vlm.mode=grpo`` samples responses to image prompts with the colocated
rollout engine and runs GRPO.  The policy needs ``policy.vision_config`` and ``policy.image_token_id``.

Data (``data.train_data_path``, indexed jsonl): ``{"tokens": [...], "prompt_length": n, "image_grid": [h, w],
"pixel_patches": <path of a torch-saved [h*w, patch_dim] tensor, or nested lists>}`` where ``tokens`` holds
``h*w / spatial_merge**2`` copies of the image token id per image; without a path synthetic rows are drawn (image
brightness encodes the answer token).

``torchrun ... -m gcore_b200.entry.train_vlm --config vlm.yaml +task.vlm.mode=grpo``"""
import sys

import torch

from ..configs.config import RlConfig
from ..data.datasets import IndexedJsonlDataset
from ..engine import get_training_engine
from ..trainer.grpo_trainer import GrpoTrainer
from ..utils.logging_utils import get_logger
from .common import finalize, init_runtime, load


def _patches(x):
    return torch.load(x, map_location="cpu") if isinstance(x, str) else torch.as_tensor(x, dtype=torch.float32)


def vlm_rows(cfg, vc, image_token_id: int, vocab: int, batch: int, seed: int = 0):
    """Yields lists of rows ``{"tokens", "prompt_length", "pixel_patches", "image_grid"}``."""
    path = cfg.data.train_data_path
    if path:
        ds = IndexedJsonlDataset(path)
        for i in range(0, len(ds) - batch + 1, batch):
            yield [dict(tokens=torch.tensor(r["tokens"]), prompt_length=int(r["prompt_length"]),
                        pixel_patches=_patches(r["pixel_patches"]), image_grid=tuple(r["image_grid"]))
                   for r in (ds[j] for j in range(i, i + batch))]
        return
    g = torch.Generator().manual_seed(seed)
    s = vc.spatial_merge
    lo = min(20, vocab - 12)
    while True:
        rows = []
        for k in range(batch):
            h, w = (2 * s, 2 * s) if k % 2 == 0 else (s, 3 * s)
            label = lo + int(torch.randint(0, 10, (1,), generator=g))
            img = torch.randn(h * w, vc.patch_dim, generator=g) * 0.1 + (label - lo - 5) * 0.2
            prompt = [3] + [image_token_id] * (h * w // (s * s)) + [4]
            rows.append(dict(tokens=torch.tensor(prompt + [label]), prompt_length=len(prompt), pixel_patches=img,
                             image_grid=(h, w)))
        yield rows


def main(argv=None):
    cfg = load(RlConfig, argv)
    init_runtime(cfg)
    opt = dict((cfg.task or {}).get("vlm", {}) or {})
    mode = opt.get("mode", "sft")
    log = get_logger("vlm")
    total = cfg.training.exit_step or cfg.training.total_ppo_step or 0
    history = []
    if mode == "sft":
        cfg.policy.without_ref = True
        eng = get_training_engine(cfg.policy, cfg.optimizer, cfg.training, None)
        eng.setup_model_and_get_optimizer(seed=cfg.training.seed)
        assert hasattr(eng.model, "vision"), "policy.vision_config is empty: not a vision-language policy"
        rows = vlm_rows(cfg, eng.model.vc, eng.model.image_token_id, eng.model_cfg.vocab_size,
                        max(cfg.training.train_gbs, 1), cfg.training.seed)
        for step, batch in zip(range(total), rows):
            for r in batch:
                m = torch.zeros(r["tokens"].numel())
                m[r["prompt_length"] - 1:-1] = 1.0
                r["loss_mask"] = m
            metrics = eng.finetune_step(batch)
            history.append(metrics)
            log.info(f"step {step} lm_loss {metrics['lm_loss']:.4f}")
    else:
        tr = GrpoTrainer(cfg).setup()
        model = tr.policy.model
        assert hasattr(model, "vision"), "policy.vision_config is empty: not a vision-language policy"
        rows = vlm_rows(cfg, model.vc, model.image_token_id, tr.policy.model_cfg.vocab_size,
                        max(cfg.training.rollout_gbs, 1), cfg.training.seed)
        for step, batch in zip(range(total), rows):
            prompts = [dict(tokens=r["tokens"][:r["prompt_length"]].tolist(), pixel_patches=r["pixel_patches"],
                            image_grid=r["image_grid"]) for r in batch]
            metrics = tr.step(prompts)
            history.append(metrics)
            log.info(f"ppo_step {step} reward {metrics['rollout-rewards/mean']:.4f}")
    finalize()
    return history


if __name__ == "__main__":
    main()
    sys.exit(0)
