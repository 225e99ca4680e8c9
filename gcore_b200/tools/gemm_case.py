"""Runs one GEMM shape a few times (for ncu captures and quick timing).

``python -m gcore_b200.tools.gemm_case --tokens 64 --n 37888 --k 3584 [--iters 5] [--layout fwd|dgrad|wgrad]``
"""
from __future__ import annotations

import argparse

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", "--T", type=int, default=64)
    ap.add_argument("--n", "--N", type=int, default=37888)
    ap.add_argument("--k", "--K", type=int, default=3584)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--layout", default="fwd")
    args = ap.parse_args()
    from gcore_b200.ops import _lib
    from gcore_b200.ops.gemm import linear_dgrad, linear_forward, linear_wgrad
    T, N, K = args.tokens, args.n, args.k
    x = torch.randn(T, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
    dy = torch.randn(T, N, device="cuda").bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn = {"fwd": lambda: linear_forward(x, w), "dgrad": lambda: linear_dgrad(dy, w),
          "wgrad": lambda: linear_wgrad(dy, x)}[args.layout]
    ts = []
    for _ in range(args.iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    _lib.check_device_errors()
    print(f"{args.layout} T={T} N={N} K={K}: ms per call {[round(t, 4) for t in ts]}")


if __name__ == "__main__":
    main()
