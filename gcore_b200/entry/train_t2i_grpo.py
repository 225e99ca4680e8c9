"""Text-to-image GRPO (``gpatch_v4/entry/train_t2i_grpo.py``): rollouts of the stochastic flow sampler, rule / model
rewards, clipped update over trajectory steps.
``torchrun ... -m gcore_b200.entry.train_t2i_grpo --config t2i.yaml training.sampling_steps=8``"""
import sys

from ..configs.config import T2iConfig
from ..trainer.t2i_trainers import T2iGrpoTrainer
from .t2i_common import finalize_t2i, init_t2i_runtime
from .common import load


def main(argv=None):
    cfg = load(T2iConfig, argv)
    init_t2i_runtime(cfg)
    trainer = T2iGrpoTrainer(cfg).setup()
    hist = trainer.run()
    finalize_t2i()
    return hist


if __name__ == "__main__":
    sys.exit(0 if main() is not None else 1)
