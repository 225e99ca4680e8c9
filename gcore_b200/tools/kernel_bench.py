"""Per-kernel timing on one GPU with CUDA events (warm-up, L2 flush between iterations), reported against the
measured roofline denominators in ``MEASURED_PEAKS.json`` when present.

``python -m gcore_b200.tools.kernel_bench [--out file.json] [--quick]``
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                     "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def time_fn(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--quick", action="store_true")
    args = ap.parse_args()
    from gcore_b200.ops import _lib
    from gcore_b200.ops.attention import flash_attn_varlen, paged_decode
    from gcore_b200.ops.gemm import gemm, linear_forward
    tf_peak, bw_peak, src = _peaks()
    res = []

    def rec(name, ms, flops=None, bytes_=None, base_ms=None):
        r = {"name": name, "ms": round(ms, 4)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["frac_of_%s_bf16" % src] = round(flops / ms / 1e9 / tf_peak, 3)
        if bytes_:
            r["gbs"] = round(bytes_ / ms / 1e6, 1)
            r["frac_of_%s_hbm" % src] = round(bytes_ / ms / 1e6 / bw_peak, 3)
        if base_ms:
            r["torch_ms"] = round(base_ms, 4)
            r["speedup_vs_torch"] = round(base_ms / ms, 3)
        res.append(r)
        print(json.dumps(r), flush=True)

    T = 8192
    shapes = [("qkv", 4608, 3584), ("o", 3584, 3584), ("gate_up", 37888, 3584), ("down", 3584, 18944)]
    if args.quick:
        shapes = shapes[:2]
    for name, N, K in shapes:
        x = torch.randn(T, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        dy = torch.randn(T, N, device="cuda").bfloat16()
        fl = 2.0 * T * N * K
        rec(f"gemm_fwd_{name}_T{T}", time_fn(lambda: gemm(x, w)), fl, base_ms=time_fn(lambda: x @ w.t()))
        rec(f"gemm_dgrad_{name}_T{T}", time_fn(lambda: gemm(dy, w, b_mn=True)), fl, base_ms=time_fn(lambda: dy @ w))
        rec(f"gemm_wgrad_{name}_T{T}", time_fn(lambda: gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32)), fl,
            base_ms=time_fn(lambda: dy.t() @ x))
        for Td in (64, 8):
            xd = torch.randn(Td, K, device="cuda").bfloat16()
            rec(f"gemm_decode_{name}_T{Td}", time_fn(lambda: linear_forward(xd, w)), bytes_=2.0 * N * K,
                base_ms=time_fn(lambda: xd @ w.t()))
    # block-scaled fp8 GEMM (1x128 activation scales, 128x128 weight scales) and its quantisers
    from gcore_b200.ops import quant
    for name, N, K in shapes[:3:2] if not args.quick else shapes[:1]:
        x = torch.randn(T, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        aq, as_ = quant.quant_act_1x128(x)
        wq, ws = quant.quant_weight_128x128(w)
        fl = 2.0 * T * N * K
        rec(f"gemm_fp8_blockscaled_{name}_T{T}", time_fn(lambda: quant.gemm_fp8_blockscaled(aq, as_, wq, ws)), fl,
            base_ms=time_fn(lambda: x @ w.t()))
        rec(f"act_quant_1x128_{name}_T{T}", time_fn(lambda: quant.quant_act_1x128(x)), bytes_=3.0 * T * K)
        rec(f"fp8_linear_incl_act_quant_{name}_T{T}",
            time_fn(lambda: quant.gemm_fp8_blockscaled(*quant.quant_act_1x128(x), wq, ws)), fl)
    # attention forward: 8 sequences of 4096, 28 q heads / 4 kv heads, D=128, causal
    Hq, Hk, D, L, B = 28, 4, 128, 4096, 4
    q = torch.randn(B * L, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B * L, Hk, D, device="cuda").bfloat16()
    v = torch.randn(B * L, Hk, D, device="cuda").bfloat16()
    cu = torch.arange(0, (B + 1) * L, L, device="cuda", dtype=torch.int32)
    fl = 4.0 * B * Hq * L * L * D / 2
    with torch.no_grad():
        qs = q.view(B, L, Hq, D).transpose(1, 2)
        ks = k.view(B, L, Hk, D).transpose(1, 2)
        vs = v.view(B, L, Hk, D).transpose(1, 2)
        base = time_fn(lambda: torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True,
                                                                                enable_gqa=True))
        rec("attn_fwd_causal_B4_L4096_H28", time_fn(lambda: flash_attn_varlen(q, k, v, cu, cu, L, L)), fl,
            base_ms=base)
    # paged decode: 64 requests, ctx 1024
    Bd, ctx, bs = 64, 1024, 16
    nb = Bd * ctx // bs
    kc = torch.randn(nb, bs, Hk, D, device="cuda").bfloat16()
    vc = torch.randn(nb, bs, Hk, D, device="cuda").bfloat16()
    bt = torch.randperm(nb, device="cuda").view(Bd, ctx // bs).to(torch.int32)
    cl = torch.full((Bd,), ctx, device="cuda", dtype=torch.int32)
    qd = torch.randn(Bd, Hq, D, device="cuda").bfloat16()
    rec("paged_decode_B64_ctx1024", time_fn(lambda: paged_decode(qd, kc, vc, bt, cl, ctx)),
        bytes_=2.0 * Bd * ctx * Hk * D * 2)
    _lib.check_device_errors()
    if args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        json.dump(res, open(args.out, "w"), indent=1)


if __name__ == "__main__":
    sys.exit(main())
