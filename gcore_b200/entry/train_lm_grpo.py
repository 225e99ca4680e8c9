"""GRPO / PPO entry point (``gpatch_v4/entry/train_lm_grpo.py``):
``torchrun ... -m gcore_b200.entry.train_lm_grpo --config rl.yaml training.total_ppo_step=100``

``placement_type: disaggregated`` splits the job: the first ``disaggregated_train_gpus`` ranks train, the others serve
rollouts (``rollout/disaggregated.py``); every rank runs this same entry point."""
import os
import sys

from ..configs.config import RlConfig
from ..trainer.rl_loop import RlLoop
from .common import finalize, init_runtime, load


def _main_disaggregated(cfg):
    import torch.distributed as dist
    from ..core import parallel_state as ps
    from ..rollout.disaggregated import RoleLayout, SamplerServer, setup_roles
    d = cfg.policy.dist_config
    ps.init_distributed(None, d.torch_dist_timeout_minutes)
    world = dist.get_world_size()
    n_train = cfg.disaggregated_train_gpus or world // 2
    stp = cfg.sampler.infer_engine_configs[0].dist_config.tensor_model_parallel_size
    layout = RoleLayout(world, n_train, stp)
    role = setup_roles(layout, dict(tp=d.tensor_model_parallel_size, pp=d.pipeline_model_parallel_size,
                                    cp=d.context_parallel_size, ep=d.expert_model_parallel_size))
    ps.set_seed(cfg.training.seed)
    if role == "sampler":
        from ..models.config import build_model_config
        SamplerServer(cfg, build_model_config(cfg.policy.model_arch, cfg.policy.model_config), layout).serve()
        hist = []
    else:
        from ..trainer.disagg_trainer import DisaggGrpoTrainer
        tr = DisaggGrpoTrainer(cfg, layout)
        hist = RlLoop(cfg, trainer=tr).setup().run()
        tr.shutdown()
    dist.barrier()
    dist.destroy_process_group()
    return hist


def main(argv=None):
    cfg = load(RlConfig, argv)
    if cfg.placement_type == "disaggregated" and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        _main_disaggregated(cfg)
        return 0
    init_runtime(cfg)
    RlLoop(cfg).setup().run()
    finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
