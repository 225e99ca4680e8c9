"""Supervised instruction-guided image editing (``gpatch_v4/entry/train_t2i_edit_sft.py``).
``torchrun ... -m gcore_b200.entry.train_t2i_edit_sft --config t2i.yaml training.sampling_steps=8``"""
import sys

from ..configs.config import T2iConfig
from ..trainer.t2i_trainers import T2iEditSftTrainer
from .t2i_common import finalize_t2i, init_t2i_runtime
from .common import load


def main(argv=None):
    cfg = load(T2iConfig, argv)
    cfg.model.pipeline = "qwen_image_edit"
    init_t2i_runtime(cfg)
    trainer = T2iEditSftTrainer(cfg).setup()
    hist = trainer.run()
    finalize_t2i()
    return hist


if __name__ == "__main__":
    sys.exit(0 if main() is not None else 1)
