"""Single-controller (asynchronous) GRPO entry point (``gpatch_v4/entry/train_lm_grpo_single_ctrl.py``)."""
import sys

from ..configs.config import RlConfig
from ..trainer.rl_loop import RlLoop
from ..trainer.single_ctrl_trainer import GrpoSingleCtrlTrainer
from .common import finalize, init_runtime, load


def main(argv=None):
    cfg = load(RlConfig, argv)
    init_runtime(cfg)
    loop = RlLoop(cfg).setup()  # reuses data / checkpoint plumbing; the controller replaces the generator
    tr = GrpoSingleCtrlTrainer(cfg, loop.prompt_iter)
    tr.tr = loop.trainer
    tr.setup()
    total = cfg.training.exit_step or cfg.training.total_ppo_step or 0
    while tr.tr.ppo_step < total:
        m = tr.step()
        if loop.reporter:
            loop.reporter.log(m, tr.tr.ppo_step)
        if cfg.training.save_interval and tr.tr.ppo_step % cfg.training.save_interval == 0:
            loop.save()
    finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
