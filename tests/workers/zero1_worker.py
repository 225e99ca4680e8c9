"""2+ rank worker: ZeRO-1 step over peer memory (pull-reduce + AdamW + push) against the NCCL reduce-scatter /
all-gather path, with and without gradient clipping; optional timing of both."""
import json
import os
import sys
import types

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

from gcore_b200.core import parallel_state as ps  # noqa: E402
from gcore_b200.ops import _lib  # noqa: E402
from gcore_b200.parallel.distributed_optimizer import DistributedDataParallel, DistributedOptimizer  # noqa: E402


class Toy(torch.nn.Module):
    def __init__(self, sizes, dev):
        super().__init__()
        g = torch.Generator(device="cpu").manual_seed(3)
        self.ws = torch.nn.ParameterList(
            [torch.nn.Parameter((torch.randn(*s, generator=g) * 0.1).bfloat16().to(dev)) for s in sizes])


def run(fused: bool, sizes, dev, rank, clip, steps=3, bucket=200_000):
    os.environ["GCORE_FUSED_DP"] = "1" if fused else "0"
    model = Toy(sizes, dev)
    ddp = DistributedDataParallel(model, bucket_size=bucket)
    cfg = types.SimpleNamespace(lr=1e-2, min_lr=0.0, lr_warmup_steps=0, lr_warmup_step_frac=None, lr_warmup_init=0.0,
                                lr_decay_steps=None, lr_decay_style="constant", adam_beta1=0.9, adam_beta2=0.95,
                                adam_eps=1e-8, weight_decay=0.01, max_grad_norm=clip)
    opt = DistributedOptimizer(ddp, cfg)
    assert all(b.peer == fused for b in ddp.buffers), [b.peer for b in ddp.buffers]
    norms = []
    for it in range(steps):
        ddp.zero_grad_buffer()
        g = torch.Generator(device="cpu").manual_seed(1000 * rank + it)
        for p in model.ws:
            p.main_grad.copy_(torch.randn(*p.shape, generator=g).to(dev))
        ddp.finish_grad_sync(extra_scale=0.5)
        opt.step()
        norms.append(float(opt.last_grad_norm))
    torch.cuda.synchronize()
    _lib.check_device_errors()
    flat = torch.cat([p.detach().float().reshape(-1) for p in model.ws])
    return flat, norms, ddp, opt, model


def main():
    out_path = sys.argv[1]
    bench = len(sys.argv) > 2 and sys.argv[2] == "bench"
    ps.init_distributed("nccl")
    ps.initialize_model_parallel(tp=1)
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    sizes = [(512, 384), (384,), (1024, 256), (256, 1024), (77, 8)]
    res = {}
    for clip in (1.0, 0.0):
        ref, n_ref, *_ = run(False, sizes, dev, rank, clip)
        got, n_got, *_ = run(True, sizes, dev, rank, clip)
        err = (ref - got).abs().max().item()
        # every rank must hold the same parameters after the push
        gathered = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(gathered, got)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        res[f"clip{clip}"] = dict(match=err < 4e-3, err=err, same_on_all_ranks=same,
                                  norm_match=all(abs(a - b) <= 1e-3 * max(1.0, abs(a)) for a, b in zip(n_ref, n_got)),
                                  norms=[n_ref, n_got])
    if bench:
        big = [(8192, 8192)] * 6  # 403 M parameters
        timing = {}
        for fused in (False, True):
            flat, norms, ddp, opt, model = run(fused, big, dev, rank, 1.0, steps=1, bucket=40_000_000)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ts = []
            for it in range(6):
                dist.barrier()
                torch.cuda.synchronize()
                ev[0].record()
                ddp.finish_grad_sync(extra_scale=1.0)
                opt.step()
                ev[1].record()
                torch.cuda.synchronize()
                ts.append(ev[0].elapsed_time(ev[1]))
            t = torch.tensor(sorted(ts[2:])[len(ts[2:]) // 2], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            timing["fused_ms" if fused else "nccl_ms"] = round(t.item(), 3)
            del flat, ddp, opt, model
            torch.cuda.empty_cache()
        n = sum(a * b for a, b in big)
        # bytes over NVLink per rank: pull (dp-1)/dp of the fp32 gradients of its shard... = n*4*(dp-1)/dp in, n*2*(dp-1)/dp out
        timing["nvlink_roofline_ms"] = round(n * 4 * (world - 1) / world / 770e9 * 1e3, 3)
        timing["hbm_roofline_ms"] = round((n * 4 * 2 + n / world * (12 * 2 + 4) + n * 2) / 6.55e12 * 1e3, 3)
        res["timing"] = timing
    if rank == 0:
        json.dump(res, open(out_path, "w"), indent=1)
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
