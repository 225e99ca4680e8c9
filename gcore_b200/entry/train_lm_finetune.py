"""SFT entry point (``gpatch_v4/entry/train_lm_finetune.py``):
``torchrun ... -m gcore_b200.entry.train_lm_finetune --config sft.yaml training.exit_step=100``"""
import sys

from ..configs.config import FinetuneConfig
from ..trainer.finetune_trainer import FinetuneTrainer
from .common import finalize, init_runtime, load


def main(argv=None):
    cfg = load(FinetuneConfig, argv)
    init_runtime(cfg)
    trainer = FinetuneTrainer(cfg).setup()
    trainer.train_loop()
    trainer.save()
    finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
