"""2+ rank worker: expert-parallel MoE layer through the peer-memory dispatch / combine kernels against the NCCL
all-to-all path (forward output, input gradient, router-weight gradient, expert weight gradients); optional timing."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

from gcore_b200.core import parallel_state as ps  # noqa: E402
from gcore_b200.models.config import ModelConfig  # noqa: E402
from gcore_b200.models.moe import MoELayer  # noqa: E402
from gcore_b200.ops import _lib  # noqa: E402


def build(cfg, ep, dev, rank):
    torch.manual_seed(11)
    layer = MoELayer(cfg, 0, 1, ep, device=dev)
    E_local = cfg.num_experts // ep
    with torch.no_grad():
        g = torch.Generator(device="cpu").manual_seed(5)
        for name, p in layer.named_parameters():
            if getattr(p, "is_expert", False):
                full = torch.randn(cfg.num_experts, *p.shape[1:], generator=g) * 0.05
                p.copy_(full[rank * E_local:(rank + 1) * E_local].to(p.dtype))
            else:
                p.copy_((torch.randn(*p.shape, generator=g) * 0.05).to(p.dtype))
    return layer


def run(layer, x0, fused):
    os.environ["GCORE_FUSED_EP"] = "1" if fused else "0"
    for p in layer.parameters():
        p.grad = None
    x = x0.clone().requires_grad_(True)
    y, aux = layer(x)
    g = torch.Generator(device="cpu").manual_seed(77 + dist.get_rank())
    dy = (torch.randn(*y.shape, generator=g) * 0.1).to(y.dtype).to(y.device)
    (y.float() * dy.float()).sum().backward()
    torch.cuda.synchronize()
    _lib.check_device_errors()
    grads = {n: p.grad.detach().float().clone() for n, p in layer.named_parameters() if p.grad is not None}
    return y.detach().float(), x.grad.detach().float(), grads


def close(a, b, tol=2e-2):
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    return bool(err <= tol * max(ref, 1e-3)), err, ref


def main():
    out_path = sys.argv[1]
    bench = len(sys.argv) > 2 and sys.argv[2] == "bench"
    ps.init_distributed("nccl")
    world, rank = dist.get_world_size(), dist.get_rank()
    ps.initialize_model_parallel(tp=1, ep=world)
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = ModelConfig(num_layers=1, hidden_size=512, num_attention_heads=4, num_kv_heads=2, ffn_hidden_size=1024,
                      vocab_size=1024, num_experts=8 * world, moe_top_k=4, moe_ffn_hidden_size=256,
                      moe_router_type="softmax", dtype="bfloat16")
    layer = build(cfg, world, dev, rank)
    res = {}
    for it, T in enumerate((300, 1111)):
        g = torch.Generator(device="cpu").manual_seed(1000 * rank + it)
        x0 = torch.randn(T, cfg.hidden_size, generator=g).bfloat16().to(dev)
        y_ref, dx_ref, g_ref = run(layer, x0, False)
        y, dx, gr = run(layer, x0, True)
        r = dict(y=close(y, y_ref)[0], y_err=close(y, y_ref)[1], dx=close(dx, dx_ref)[0], dx_err=close(dx, dx_ref)[1])
        for n in g_ref:
            ok, err, ref = close(gr[n], g_ref[n], 3e-2)
            r["grad_" + n] = ok
            r["grad_" + n + "_err"] = [err, ref]
        res[f"T{T}"] = r
    if bench:
        from gcore_b200.parallel import ep_fused
        cfg2 = ModelConfig(num_layers=1, hidden_size=2048, num_attention_heads=32, num_kv_heads=4,
                           ffn_hidden_size=6144, vocab_size=1024, num_experts=128, moe_top_k=8,
                           moe_ffn_hidden_size=768, moe_router_type="softmax", dtype="bfloat16")
        big = build(cfg2, world, dev, rank)
        T = 8192
        x0 = torch.randn(T, 2048, device=dev).bfloat16()
        timing = {}
        for fused in (False, True):
            os.environ["GCORE_FUSED_EP"] = "1" if fused else "0"
            ts = []
            for it in range(8):
                x = x0.clone().requires_grad_(True)
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                e0.record()
                y, _ = big(x)
                e1.record()
                y.float().sum().backward()
                e2.record()
                torch.cuda.synchronize()
                ts.append((e0.elapsed_time(e1), e1.elapsed_time(e2)))
            ts = ts[3:]
            f = torch.tensor([sorted(t[0] for t in ts)[len(ts) // 2], sorted(t[1] for t in ts)[len(ts) // 2]], device=dev)
            dist.all_reduce(f, op=dist.ReduceOp.MAX)
            timing["fused" if fused else "nccl"] = dict(fwd_ms=round(f[0].item(), 3), bwd_ms=round(f[1].item(), 3))
        # tokens x K rows of H bf16 cross NVLink once in dispatch and once in combine, (ep-1)/ep of them
        bytes_one_way = T * 8 * 2048 * 2 * (world - 1) / world
        timing["nvlink_roofline_ms_dispatch_plus_combine"] = round(2 * bytes_one_way / 770e9 * 1e3, 3)
        res["timing"] = timing
    if rank == 0:
        json.dump(res, open(out_path, "w"), indent=1)
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
