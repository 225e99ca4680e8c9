"""Embedding-model training entry point (the reference's embedding main): (query, positive) pairs from an indexed
jsonl file (``{"query": [...], "positive": [...]}`` token-id lists) or synthetic pairs; in-batch-negative InfoNCE on
the pooled final hidden states.

``torchrun ... -m gcore_b200.entry.train_lm_embedding --config emb.yaml +task.embedding.temperature=0.05``"""
import sys

import torch

from ..configs.config import FinetuneConfig
from ..data.datasets import IndexedJsonlDataset
from ..engine import get_training_engine
from ..trainer.preference_trainers import embedding_step
from ..utils.logging_utils import get_logger
from .common import finalize, init_runtime, load


def pair_batches(cfg, vocab: int, seed: int = 0):
    path, bs = cfg.data.train_data_path, max(cfg.training.train_gbs, 1)
    if path:
        ds = IndexedJsonlDataset(path)
        for i in range(0, len(ds) - bs + 1, bs):
            rows = [ds[j] for j in range(i, i + bs)]
            yield ([{"tokens": torch.tensor(r["query"])} for r in rows],
                   [{"tokens": torch.tensor(r["positive"])} for r in rows])
    else:
        g = torch.Generator().manual_seed(seed)
        while True:  # a positive shares its topic token block with its query
            topics = torch.randint(3, vocab, (bs, 6), generator=g)
            mk = lambda t: {"tokens": torch.cat([t, torch.randint(3, vocab, (4,), generator=g)])}  # noqa: E731
            yield [mk(t) for t in topics], [mk(t) for t in topics]


def main(argv=None):
    cfg = load(FinetuneConfig, argv)
    init_runtime(cfg)
    cfg.policy.without_ref = True
    eng = get_training_engine(cfg.policy, cfg.optimizer, cfg.training, None)
    eng.setup_model_and_get_optimizer(seed=cfg.training.seed)
    opt = dict((cfg.task or {}).get("embedding", {}) or {})
    log = get_logger("embedding")
    total = cfg.training.exit_step or cfg.training.total_training_step or 0
    history = []
    for step, (q, p) in enumerate(pair_batches(cfg, eng.model_cfg.vocab_size, cfg.training.seed)):
        if step >= total:
            break
        m = embedding_step(eng, q, p, float(opt.get("temperature", 0.05)), opt.get("pooling", "last"),
                           bool(opt.get("grad_cache", False)))
        history.append(m)
        log.info(f"step {step} " + " ".join(f"{k}={v:.4f}" for k, v in m.items()))
    finalize()
    return history


if __name__ == "__main__":
    main()
    sys.exit(0)
