"""Bradley-Terry reward-model training entry point (``gpatch_v4/entry/train_lm_reward_model.py``)."""
import sys

from ..configs.config import RewardTrainConfig
from ..engine import get_training_engine
from ..trainer.preference_trainers import rm_step
from ..utils.logging_utils import get_logger
from .common import finalize, init_runtime, load
from .train_lm_dpo import pair_batches


def main(argv=None):
    cfg = load(RewardTrainConfig, argv)
    init_runtime(cfg)
    eng = get_training_engine(cfg.policy, cfg.optimizer, cfg.training, cfg.ppo, value_head=True)
    eng.setup_model_and_get_optimizer(seed=cfg.training.seed, with_ref=False)
    log = get_logger("rm")
    total = cfg.training.exit_step or cfg.training.total_ppo_step or 0
    for step, (chosen, rejected) in enumerate(pair_batches(cfg, eng.model_cfg.vocab_size, cfg.training.seed)):
        if step >= total:
            break
        m = rm_step(eng, chosen, rejected, margin=cfg.rm_margin)
        log.info(f"step {step} " + " ".join(f"{k}={v:.4f}" for k, v in m.items()))
    finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
