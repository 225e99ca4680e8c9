"""gloo worker of the disaggregated-placement test: ``n_train`` trainer ranks (data parallel, optionally tensor
parallel) and the remaining ranks as rollout engines (optionally tensor parallel).  argv: out.json n_train train_tp
sampler_tp."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from gcore_b200.core import parallel_state as ps  # noqa: E402
from gcore_b200.models.config import get_preset  # noqa: E402
from gcore_b200.rollout.disaggregated import RoleLayout, SamplerServer, setup_roles  # noqa: E402
from gcore_b200.rollout.weight_sync import _engine_tensor_map, tensor_digest  # noqa: E402


def main():
    out, n_train, train_tp, sampler_tp = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
    ps.init_distributed("gloo")
    world, rank = dist.get_world_size(), dist.get_rank()
    from test_grpo_cpu import make_cfg, reward_has_small_token
    layout = RoleLayout(world, n_train, sampler_tp)
    role = setup_roles(layout, dict(tp=train_tp))
    cfg = make_cfg()
    cfg.placement_type = "disaggregated"
    cfg.policy.dist_config.tensor_model_parallel_size = train_tp
    cfg.policy.dist_config.sequence_parallel = train_tp > 1
    cfg.policy.sampler_client.update_weight_max_size_mb = 1          # several buckets even for the tiny model
    dp = n_train // train_tp
    cfg.training.rollout_gbs, cfg.training.train_gbs = 4 * dp, 16 * dp
    mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
    torch.manual_seed(0)
    res = {}
    if role == "train":
        from gcore_b200.trainer.disagg_trainer import DisaggGrpoTrainer
        tr = DisaggGrpoTrainer(cfg, layout, model_cfg=mcfg, reward_fn=reward_has_small_token).setup()
        g = torch.Generator().manual_seed(5 + ps.get_data_parallel_rank())
        prompts = [torch.randint(3, 1024, (6 + i,), generator=g).tolist() for i in range(4)]
        ms = [tr.step(prompts) for _ in range(2)]
        tr.shutdown()
        res = {"role": "train", "grad_norm": [m["policy/grad_norm"] for m in ms],
               "tokens": [m["rollout-metrics/total_tokens"] for m in ms], "transfer": tr.last_transfer,
               "digest": {n: tensor_digest(t) for n, t in tr.policy.named_local_weights(merged_lora=True)},
               "tp_rank": ps.get_tensor_model_parallel_rank()}
    else:
        srv = SamplerServer(cfg, mcfg, layout)
        stats = srv.serve()
        res = {"role": "sampler", "stats": stats, "tp_rank": ps.get_tensor_model_parallel_rank(),
               "digest": {n: tensor_digest(t) for n, t in _engine_tensor_map(srv.engine, srv.model).items()}}
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        json.dump(allres, open(out, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
