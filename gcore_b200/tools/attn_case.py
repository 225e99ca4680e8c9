"""Runs one flash-attention shape a few times (for ncu captures and quick timing).

``python -m gcore_b200.tools.attn_case --batch 2 --seq 2048 --heads 8 --kv-heads 2 [--bwd] [--iters 5]``
"""
from __future__ import annotations

import argparse

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--sdpa", action="store_true", help="time torch SDPA on the same shape instead")
    a = ap.parse_args()
    from gcore_b200.ops import _lib
    from gcore_b200.ops.attention import flash_attn_varlen
    B, L, H, Hk, D = a.batch, a.seq, a.heads, a.kv_heads, a.dim
    T = B * L
    q = torch.randn(T, H, D, device="cuda").bfloat16().requires_grad_(a.bwd)
    k = torch.randn(T, Hk, D, device="cuda").bfloat16().requires_grad_(a.bwd)
    v = torch.randn(T, Hk, D, device="cuda").bfloat16().requires_grad_(a.bwd)
    do = torch.randn(T, H, D, device="cuda").bfloat16()
    cu = torch.arange(0, T + 1, L, dtype=torch.int32, device="cuda")
    flops = 4.0 * B * H * L * L * D / 2 * (3.5 if a.bwd else 1.0)

    def run():
        if a.sdpa:
            qq = q.view(B, L, H, D).transpose(1, 2)
            kk = k.view(B, L, Hk, D).transpose(1, 2).repeat_interleave(H // Hk, 1)
            vv = v.view(B, L, Hk, D).transpose(1, 2).repeat_interleave(H // Hk, 1)
            o = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True)
            if a.bwd:
                o.backward(do.view(B, L, H, D).transpose(1, 2))
            return
        o = flash_attn_varlen(q, k, v, cu, cu, L, L, causal=True)
        if a.bwd:
            o.backward(do)

    ts = []
    for _ in range(a.iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        run()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    _lib.check_device_errors()
    best = min(ts[1:]) if len(ts) > 1 else ts[0]
    print(f"attn B={B} L={L} H={H}/{Hk} D={D} bwd={a.bwd} sdpa={a.sdpa}: ms {[round(t, 4) for t in ts]} "
          f"-> {flops / best / 1e9:.0f} TFLOP/s (causal FLOPs)")


if __name__ == "__main__":
    main()
