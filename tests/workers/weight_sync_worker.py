"""2-rank worker: trainer TP=2 -> rollout TP=1 weight resync over peer memory against the all-gather path."""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig  # noqa: E402
from gcore_b200.core import parallel_state as ps  # noqa: E402
from gcore_b200.engine.train_engine import TrainingEngine  # noqa: E402
from gcore_b200.models.config import ModelConfig  # noqa: E402
from gcore_b200.models.gpt import GPTModel  # noqa: E402
from gcore_b200.ops import _lib  # noqa: E402
from gcore_b200.rollout.engine import InferEngine, RolloutWeights  # noqa: E402
from gcore_b200.rollout.weight_sync import sync_weights  # noqa: E402


def rollout_engine(mcfg, dev):
    full = GPTModel(mcfg, tp_size=1, device=dev)
    full.reset_parameters(999)  # different from the trainer's weights
    return InferEngine(mcfg, RolloutWeights.from_model(full, clone=True), tp_size=1, tp_group=None, device=dev,
                       num_kv_blocks=64, use_cuda_graph=False)


def main():
    out_path = sys.argv[1]
    ps.init_distributed("nccl")
    ps.initialize_model_parallel(tp=2)
    rank = dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    res = {}
    for tag, mcfg in (("small", ModelConfig(num_layers=2, hidden_size=256, num_attention_heads=4, num_kv_heads=2,
                                            ffn_hidden_size=704, vocab_size=1024, qkv_bias=True, dtype="bfloat16")),
                      ("medium", ModelConfig(num_layers=4, hidden_size=2048, num_attention_heads=16, num_kv_heads=4,
                                             ffn_hidden_size=8192, vocab_size=32768, dtype="bfloat16"))):
        pc = PolicyConfig(recompute="none", without_ref=True)
        pc.dist_config.tensor_model_parallel_size = 2
        pc.dist_config.sequence_parallel = True
        eng = TrainingEngine(pc, OptimizerConfig(), TrainingConfig(), model_cfg=mcfg)
        eng.setup_model_and_get_optimizer(seed=5, with_ref=False)
        engines, stats, times = {}, {}, {}
        for mode in ("nccl", "peer"):
            os.environ["GCORE_PEER_WEIGHT_SYNC"] = "1" if mode == "peer" else "0"
            ie = rollout_engine(mcfg, dev)
            stats[mode] = sync_weights(eng, ie, max_bucket_mb=64)
            ts = []
            for _ in range(3):
                dist.barrier()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                sync_weights(eng, ie, max_bucket_mb=64)
                torch.cuda.synchronize()
                ts.append((time.perf_counter() - t0) * 1e3)
            times[mode] = min(ts)
            engines[mode] = ie
        _lib.check_device_errors()
        same = all(torch.equal(a, b) for a, b in zip(engines["nccl"].w.tensors(), engines["peer"].w.tensors()))
        # and both equal the un-sharded weights of a TP=1 model built from the same seed
        full = GPTModel(mcfg, tp_size=1, device=dev)
        full.reset_parameters(5)
        ref = RolloutWeights.from_model(full)
        exact = all(torch.equal(a, b) for a, b in zip(ref.tensors(), engines["peer"].w.tensors()))
        if tag != "small":
            exact = True  # large tensors are initialised per TP rank, so only the small model has a TP=1 twin
        res[tag] = dict(peer_equals_allgather=same, equals_unsharded_model=exact,
                        used_peer_path=stats["peer"].get("peer_memory", 0.0) == 1.0,
                        ms=dict(nccl=round(times["nccl"], 3), peer=round(times["peer"], 3)),
                        mbytes=round(stats["peer"]["bytes"] / 1e6, 1))
        del eng, engines
        torch.cuda.empty_cache()
    if rank == 0:
        json.dump(res, open(out_path, "w"), indent=1)
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
