import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gcore_b200.core import parallel_state as ps  # noqa: E402
from test_sft_cpu import build_engine, run_steps  # noqa: E402


def main():
    out = sys.argv[1]
    ps.init_distributed("gloo")
    ps.initialize_model_parallel(tp=1)
    rank, world = dist.get_rank(), dist.get_world_size()
    eng = build_engine()
    losses = run_steps(eng, rank, world, steps=20)
    torch.save(losses, os.path.join(out, f"losses_{rank}.pt"))
    from gcore_b200.checkpoint.torch_dist import load_checkpoint, save_checkpoint
    ckpt = os.path.join(out, "ckpt")
    save_checkpoint(eng, ckpt, step=20)
    before = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    m_before = [sh["m"].clone() for sh in eng.optimizer.shards]
    with torch.no_grad():
        for p in eng.model.parameters():
            p.add_(1.0)
        for sh in eng.optimizer.shards:
            sh["m"].zero_()
    step = load_checkpoint(eng, ckpt)
    ok = step == 20 and all(torch.equal(before[n], p) for n, p in eng.model.named_parameters())
    ok = ok and all(torch.equal(a, sh["m"]) for a, sh in zip(m_before, eng.optimizer.shards))
    torch.save(bool(ok), os.path.join(out, f"reload_ok_{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
