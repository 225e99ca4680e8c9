"""Pre-training entry point (``gpatch_v4/entry/train_lm_pretrain.py``): rows of ``training.seq_length`` tokens cut
from a token stream (``data.train_data_path``: indexed jsonl of ``{"tokens": [...]}`` documents) or synthetic rows,
loss on every token, same engine / checkpoint / resume path as SFT.

``torchrun ... -m gcore_b200.entry.train_lm_pretrain --config pretrain.yaml training.exit_step=1000``"""
import sys

from ..configs.config import FinetuneConfig
from ..data.datasets import pretrain_dataset_fn
from ..trainer.finetune_trainer import FinetuneTrainer
from .common import finalize, init_runtime, load


def main(argv=None):
    cfg = load(FinetuneConfig, argv)
    init_runtime(cfg)
    trainer = FinetuneTrainer(cfg, dataset_fn=pretrain_dataset_fn).setup()
    history = trainer.train_loop()
    trainer.save()
    finalize()
    return history


if __name__ == "__main__":
    main()
    sys.exit(0)
