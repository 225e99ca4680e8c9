"""DPO entry point (``gpatch_v4/entry/train_lm_dpo.py``): pairs of (chosen, rejected) token sequences from an indexed
jsonl file (``data.train_data_path`` lines: {"prompt": [...], "chosen": [...], "rejected": [...]}) or synthetic pairs."""
import sys

import torch

from ..configs.config import DpoConfig
from ..data.datasets import IndexedJsonlDataset
from ..engine import get_training_engine
from ..trainer.preference_trainers import dpo_step
from ..utils.logging_utils import get_logger
from .common import finalize, init_runtime, load


def pair_batches(cfg, vocab: int, seed: int = 0):
    path = cfg.data.train_data_path
    bs = max(cfg.training.train_gbs, 1)
    if path:
        ds = IndexedJsonlDataset(path)
        for i in range(0, len(ds) - bs + 1, bs):
            rows = [ds[j] for j in range(i, i + bs)]
            mk = lambda r, k: {"tokens": torch.tensor(r["prompt"] + r[k]), "prompt_length": len(r["prompt"])}  # noqa: E731
            yield [mk(r, "chosen") for r in rows], [mk(r, "rejected") for r in rows]
    else:
        g = torch.Generator().manual_seed(seed)
        while True:
            mk = lambda: {"tokens": torch.randint(3, vocab, (48,), generator=g), "prompt_length": 16}  # noqa: E731
            yield [mk() for _ in range(bs)], [mk() for _ in range(bs)]


def main(argv=None):
    cfg = load(DpoConfig, argv)
    init_runtime(cfg)
    eng = get_training_engine(cfg.policy, cfg.optimizer, cfg.training, cfg.ppo)
    eng.setup_model_and_get_optimizer(seed=cfg.training.seed, with_ref=not cfg.reference_free)
    log = get_logger("dpo")
    total = cfg.training.exit_step or cfg.training.total_ppo_step or 0
    for step, (chosen, rejected) in enumerate(pair_batches(cfg, eng.model_cfg.vocab_size, cfg.training.seed)):
        if step >= total:
            break
        m = dpo_step(eng, chosen, rejected, beta=cfg.dpo_beta, label_smoothing=cfg.dpo_label_smoothing,
                     reference_free=cfg.reference_free, sft_coef=cfg.dpo_sft_loss_coef)
        log.info(f"step {step} " + " ".join(f"{k}={v:.4f}" for k, v in m.items()))
    finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
