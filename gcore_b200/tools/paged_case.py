"""Runs the paged decode-attention kernel on one shape (for ncu captures and quick timing).

``python -m gcore_b200.tools.paged_case --tokens 64 --heads 28 --kv-heads 4 --ctx 768 --max-ctx 1280 [--graph]``

Without ``--graph`` every launch is a plain launch over rotating K/V caches (more bytes than L2 holds); with it, 24
launches are captured into one CUDA graph and the time per launch under replay is reported.
"""
from __future__ import annotations

import argparse

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--heads", type=int, default=28)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--ctx", type=int, default=768)
    ap.add_argument("--max-ctx", type=int, default=1280)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--graph", action="store_true")
    a = ap.parse_args()
    from gcore_b200.ops import _lib
    from gcore_b200.ops.attention import paged_decode
    dev = torch.device("cuda")
    T, hq, hk, D, bs = a.tokens, a.heads, a.kv_heads, 128, a.block_size
    nblk = T * ((a.max_ctx + bs - 1) // bs)
    copies = 4
    kc = [torch.randn(nblk, bs, hk, D, device=dev).bfloat16() for _ in range(copies)]
    vc = [torch.randn(nblk, bs, hk, D, device=dev).bfloat16() for _ in range(copies)]
    bt = torch.arange(nblk, device=dev, dtype=torch.int32).view(T, -1)
    ctx = torch.full((T,), a.ctx, dtype=torch.int32, device=dev)
    qkv = torch.randn(T, (hq + 2 * hk) * D, device=dev).bfloat16()
    q = qkv.view(T, hq + 2 * hk, D)[:, :hq]
    mb = T * a.ctx * 2 * hk * D * 2 / 1e6
    if a.graph:
        from gcore_b200.tools.decode_bench import graph_time
        us = graph_time([lambda i=i: paged_decode(q, kc[i % copies], vc[i % copies], bt, ctx, a.max_ctx)
                         for i in range(24)])
    else:
        ts = []
        for i in range(a.iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            paged_decode(q, kc[i % copies], vc[i % copies], bt, ctx, a.max_ctx)
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e3)
        us = min(ts[1:]) if len(ts) > 1 else ts[0]
    _lib.check_device_errors()
    print(f"paged decode T={T} H={hq}/{hk} ctx={a.ctx} max={a.max_ctx}: {us:.2f} us per call, {mb:.0f} MB of K/V "
          f"-> {mb / us:.2f} TB/s")


if __name__ == "__main__":
    main()
