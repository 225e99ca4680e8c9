"""GRPO / PPO entry point (``gpatch_v4/entry/train_lm_grpo.py``):
``torchrun ... -m gcore_b200.entry.train_lm_grpo --config rl.yaml training.total_ppo_step=100``"""
import sys

from ..configs.config import RlConfig
from ..trainer.rl_loop import RlLoop
from .common import finalize, init_runtime, load


def main(argv=None):
    cfg = load(RlConfig, argv)
    init_runtime(cfg)
    RlLoop(cfg).setup().run()
    finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
