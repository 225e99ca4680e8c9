"""2+ rank worker: context-parallel attention over peer memory (K/V pull, dK/dV return) against the single-GPU
kernel on the unsharded packed stream; optional timing against the all-gather / reduce-scatter twin."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

from gcore_b200.core import parallel_state as ps  # noqa: E402
from gcore_b200.ops import _lib  # noqa: E402
from gcore_b200.ops.attention import flash_attn_varlen  # noqa: E402
from gcore_b200.parallel.cp import CPContext, cp_attention  # noqa: E402


def make_docs(T, seed, lo=64, hi=2048):
    g = torch.Generator().manual_seed(seed)
    cu = [0]
    while cu[-1] < T:
        cu.append(min(T, cu[-1] + int(torch.randint(lo, hi + 1, (1,), generator=g))))
    return cu


def close(a, b, tol=2e-2):
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item()
    return bool(err <= tol * max(ref, 1e-3)), err


def case(T, Hq, Hk, D, window, use_sinks, seed, dev, group, fused=True):
    cp, rank = dist.get_world_size(group), dist.get_rank(group)
    s = T // cp
    cu = make_docs(T, seed)
    g = torch.Generator().manual_seed(seed + 1)
    q = (torch.randn(T, Hq, D, generator=g) * 0.5).bfloat16().to(dev)
    k = (torch.randn(T, Hk, D, generator=g) * 0.5).bfloat16().to(dev)
    v = (torch.randn(T, Hk, D, generator=g) * 0.5).bfloat16().to(dev)
    do = (torch.randn(T, Hq, D, generator=g) * 0.1).bfloat16().to(dev)
    sinks = (torch.randn(Hq, generator=g) * 0.5).to(dev) if use_sinks else None
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    mx = max(cu[i + 1] - cu[i] for i in range(len(cu) - 1))
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    sr = sinks.clone().requires_grad_(True) if use_sinks else None
    o_ref = flash_attn_varlen(qr, kr, vr, cu_t, cu_t, mx, mx, causal=True, window=window, sinks=sr)
    o_ref.backward(do)
    sl = slice(rank * s, (rank + 1) * s)
    os.environ["GCORE_FUSED_CP"] = "1" if fused else "0"
    ctx = CPContext(group, cp, rank, cu, s, dev)
    ql, kl, vl = (t[sl].clone().requires_grad_(True) for t in (q, k, v))
    sl_s = sinks.clone().requires_grad_(True) if use_sinks else None
    o = cp_attention(ql, kl, vl, ctx, window, sl_s)
    o.backward(do[sl])
    torch.cuda.synchronize()
    _lib.check_device_errors()
    r = {}
    for name, a, b in (("o", o, o_ref[sl]), ("dq", ql.grad, qr.grad[sl]), ("dk", kl.grad, kr.grad[sl]),
                       ("dv", vl.grad, vr.grad[sl])):
        ok, err = close(a, b)
        r[name], r[name + "_err"] = ok, err
    if use_sinks:
        ds = sl_s.grad.float().clone()
        dist.all_reduce(ds, group=group)
        ok, err = close(ds, sr.grad)
        r["dsinks"], r["dsinks_err"] = ok, err
    return r


def main():
    out_path = sys.argv[1]
    bench = len(sys.argv) > 2 and sys.argv[2] == "bench"
    ps.init_distributed("nccl")
    world, rank = dist.get_world_size(), dist.get_rank()
    ps.initialize_model_parallel(tp=1, cp=world)
    group = ps.get_context_parallel_group()
    dev = torch.device("cuda", torch.cuda.current_device())
    res = {}
    res["full"] = case(4096, 8, 2, 128, 0, False, 1, dev, group)
    res["window_sinks"] = case(4096, 8, 2, 128, 512, True, 2, dev, group)
    res["full_again"] = case(2048, 4, 4, 64, 0, False, 3, dev, group)
    res["nccl_twin"] = case(4096, 8, 2, 128, 512, True, 2, dev, group, fused=False)
    if bench:
        T, Hq, Hk, D = 65536, 16, 4, 128  # one TP=2 shard of the Llama-3-8B long-context configuration
        s = T // world
        g = torch.Generator().manual_seed(5)
        lens = torch.exp(torch.randn(4096, generator=g) * 1.2 + 7).clamp(64, 32768).long().tolist()
        cu = [0]
        for ln in lens:
            if cu[-1] >= T:
                break
            cu.append(min(T, cu[-1] + ln))
        ctx = CPContext(group, world, rank, cu, s, dev)
        timing = {"docs": len(cu) - 1}
        for window in (0, 4096):
            for fused in (True, False):
                os.environ["GCORE_FUSED_CP"] = "1" if fused else "0"
                ts = []
                for it in range(6):
                    q = torch.randn(s, Hq, D, device=dev).bfloat16().requires_grad_(True)
                    k = torch.randn(s, Hk, D, device=dev).bfloat16().requires_grad_(True)
                    v = torch.randn(s, Hk, D, device=dev).bfloat16().requires_grad_(True)
                    do = torch.randn(s, Hq, D, device=dev).bfloat16()
                    dist.barrier()
                    torch.cuda.synchronize()
                    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                    e[0].record()
                    o = cp_attention(q, k, v, ctx, window, None)
                    e[1].record()
                    o.backward(do)
                    e[2].record()
                    torch.cuda.synchronize()
                    ts.append((e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])))
                ts = ts[2:]
                f = torch.tensor([sorted(t[0] for t in ts)[len(ts) // 2], sorted(t[1] for t in ts)[len(ts) // 2]],
                                 device=dev)
                dist.all_reduce(f, op=dist.ReduceOp.MAX)
                timing[f"window{window}_{'peer' if fused else 'nccl'}"] = dict(fwd_ms=round(f[0].item(), 3),
                                                                              bwd_ms=round(f[1].item(), 3))
            p = ctx.plan(window)
            timing[f"window{window}_rows_pulled_last_rank"] = sum(n for r, _, _, n in p.pulls if r != rank)
        res["timing"] = timing
    if rank == 0:
        json.dump(res, open(out_path, "w"), indent=1)
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
