"""Kernel and phase timing on one GPU with CUDA events (warm-up, inputs or L2 flush larger than L2), reported
against the measured roofline denominators in ``MEASURED_PEAKS.json`` when present.

``python -m gcore_b200.tools.kernel_bench [--out file.json] [--quick]``      the training / decode shape table
``python -m gcore_b200.tools.kernel_bench gemm --tokens 64 --n 37888 --k 3584 [--iters 5] [--layout fwd|dgrad|wgrad]``
``python -m gcore_b200.tools.kernel_bench attn --batch 2 --seq 2048 --heads 8 --kv-heads 2 [--bwd] [--sdpa]``
``python -m gcore_b200.tools.kernel_bench paged --tokens 64 --heads 28 --kv-heads 4 --ctx 768 --max-ctx 1280 [--graph]``
``python -m gcore_b200.tools.kernel_bench decode_chain [--tokens 64] [--tp 1] [--json out.json]``   per-kernel cost
                                                                 of one decoder layer under CUDA-graph replay
``python -m gcore_b200.tools.kernel_bench train_step --model qwen2.5-7b --layers 8 --tokens 8192 --seqlen 1280``
``python -m gcore_b200.tools.kernel_bench ce --tokens 8192 --vocab 152064 --k 3584 [--fused-only]``   vocabulary
                                                                 GEMM with softmax statistics vs the chunked form

The single-shape sub-commands launch one kernel a few times, which also makes them the small cases profilers are
pointed at.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

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


def cmd_table(argv=None):
    """Training and decode shapes of the 7B recipe against the library twin of each kernel."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--quick", action="store_true")
    args = ap.parse_args(argv)
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


def cmd_gemm(argv=None):
    """Runs one GEMM shape a few times (for ncu captures and quick timing)."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", "--T", type=int, default=64)
    ap.add_argument("--n", "--N", type=int, default=37888)
    ap.add_argument("--k", "--K", type=int, default=3584)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--layout", default="fwd")
    ap.add_argument("--two-cta", type=int, default=0, help="1: route large problems to the CTA-pair kernel (A/B)")
    args = ap.parse_args(argv)
    from gcore_b200.ops import _lib
    from gcore_b200.ops import gemm as gemm_mod
    from gcore_b200.ops.gemm import linear_dgrad, linear_forward, linear_wgrad
    gemm_mod.TWO_CTA["enabled"] = bool(args.two_cta)
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


def cmd_attn(argv=None):
    """Runs one flash-attention shape a few times (for ncu captures and quick timing)."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--v-dim", type=int, default=0, help="value head dim when it differs from --dim (192 / 128)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--sdpa", action="store_true", help="time torch SDPA on the same shape instead")
    a = ap.parse_args(argv)
    from gcore_b200.ops import _lib
    from gcore_b200.ops.attention import flash_attn_varlen
    B, L, H, Hk, D = a.batch, a.seq, a.heads, a.kv_heads, a.dim
    T = B * L
    Dv = a.v_dim or D
    q = torch.randn(T, H, D, device="cuda").bfloat16().requires_grad_(a.bwd)
    k = torch.randn(T, Hk, D, device="cuda").bfloat16().requires_grad_(a.bwd)
    v = torch.randn(T, Hk, Dv, device="cuda").bfloat16().requires_grad_(a.bwd)
    do = torch.randn(T, H, Dv, device="cuda").bfloat16()
    cu = torch.arange(0, T + 1, L, dtype=torch.int32, device="cuda")
    # causal: half of (Q K^T + P V) forward; backward adds dP, dV (value width) and dQ, dK (key width) + the recompute
    flops = B * H * L * L * ((D + Dv) + ((2 * D + Dv) + (D + Dv) if a.bwd else 0))

    def run():
        if a.sdpa:
            qq = q.view(B, L, H, D).transpose(1, 2)
            kk = k.view(B, L, Hk, D).transpose(1, 2).repeat_interleave(H // Hk, 1)
            vv = torch.nn.functional.pad(v, (0, D - Dv)).view(B, L, Hk, D).transpose(1, 2).repeat_interleave(H // Hk, 1)
            o = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True)
            if a.bwd:
                o.backward(torch.nn.functional.pad(do, (0, D - Dv)).view(B, L, H, D).transpose(1, 2))
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


def cmd_paged(argv=None):
    """Runs the paged decode-attention kernel on one shape (for ncu captures and quick timing)."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--heads", type=int, default=28)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--ctx", type=int, default=768)
    ap.add_argument("--max-ctx", type=int, default=1280)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--graph", action="store_true")
    a = ap.parse_args(argv)
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


def cmd_mla_decode(argv=None):
    """Times the latent-attention decode kernel on one shape against the eager absorbed form (gather of every
    request's rows + fp32 einsums), reports the share of the measured copy bandwidth the cache rows are read at and
    the tensor throughput of the two contractions."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--heads", type=int, default=128)
    ap.add_argument("--kv-lora", type=int, default=512)
    ap.add_argument("--rope", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--eager", type=int, default=1)
    a = ap.parse_args(argv)
    from gcore_b200.ops import _lib
    from gcore_b200.ops.attention import mla_paged_decode
    dev = torch.device("cuda")
    B, H, C, dr, bs = a.tokens, a.heads, a.kv_lora, a.rope, a.block_size
    per = (a.ctx + bs - 1) // bs
    copies = 3
    caches = [torch.randn(B * per, bs, C + dr, device=dev).bfloat16() * 0.5 for _ in range(copies)]
    bt = torch.arange(B * per, device=dev, dtype=torch.int32).view(B, per)
    ctx = torch.full((B,), a.ctx, dtype=torch.int32, device=dev)
    q_lat = (torch.randn(B, H, C, device=dev) * 0.3).bfloat16()
    q_rope = (torch.randn(B, H, dr, device=dev) * 0.3).bfloat16()
    scale = 1.0 / math.sqrt(192)
    out = torch.empty(B, H, C, device=dev, dtype=torch.bfloat16)

    def timed(fn):
        ts = []
        for i in range(a.iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn(i)
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e3)
        return min(ts[1:]) if len(ts) > 1 else ts[0]

    us = timed(lambda i: mla_paged_decode(q_lat, q_rope, caches[i % copies], bt, ctx, a.ctx, scale, out=out))
    _lib.check_device_errors()
    mb = B * a.ctx * (C + dr) * 2 / 1e6
    gf = 2.0 * B * H * a.ctx * (2 * C + dr) / 1e9
    _, hbm, which = _peaks()
    line = (f"mla decode B={B} H={H} C={C}+{dr} ctx={a.ctx}: {us:.1f} us, {mb:.0f} MB of latent rows -> "
            f"{mb / us:.2f} TB/s ({mb / us * 1e3 / hbm:.2f} of {which} copy), {gf / us * 1e3:.0f} TFLOP/s")
    if a.eager:
        p_all = torch.arange(a.ctx, device=dev)
        idx = bt.long()[:, p_all // bs] * bs + p_all % bs

        def eager(i):
            lat = caches[i % copies].view(-1, C + dr)[idx]
            s = torch.einsum("bhc,blc->bhl", q_lat.float(), lat[..., :C].float())
            s = (s + torch.einsum("bhr,blr->bhl", q_rope.float(), lat[..., C:].float())) * scale
            return torch.einsum("bhl,blc->bhc", torch.softmax(s, -1), lat[..., :C].float())
        ue = timed(eager)
        ref = eager(0)
        got = mla_paged_decode(q_lat, q_rope, caches[0], bt, ctx, a.ctx, scale, out=out).float()
        line += f"; eager absorbed form {ue:.1f} us ({ue / us:.1f}x), max |diff| {float((got - ref).abs().max()):.3e}"
    print(line)


COMMANDS_LATE = {"mla_decode": cmd_mla_decode}


def graph_time(fn_list, reps=5):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for f in fn_list[:2]:
            f()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fn_list:
            f()
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) / len(fn_list))
    return sorted(ts)[len(ts) // 2] * 1e3  # us


def cmd_decode_chain(argv=None):
    """Per-kernel cost of the decode chain under CUDA-graph replay (what a rollout step actually pays per kernel)."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--json", default=None)
    ap.add_argument("--pdl", type=int, default=0, help="launch the native kernels with programmatic dependent launch")
    args = ap.parse_args(argv)
    from gcore_b200.ops import _lib, fused
    from gcore_b200.ops.attention import kv_append_rope, paged_decode, paged_decode_append
    from gcore_b200.ops.gemm import gemm, linear_forward
    dev = torch.device("cuda")
    if args.pdl:
        _lib.kernels().gk_set_pdl(1)
    T, tp = args.tokens, args.tp
    H, F, hq, hk, D = 3584, 18944 // tp, 28 // tp, 4 // tp, 128
    res = {}
    copies = 12
    shapes = {"qkv": ((hq + 2 * hk) * D, H), "o": (H, hq * D), "fc1": (2 * F, H), "fc2": (H, F)}
    for name, (N, K) in shapes.items():
        ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(copies)]
        x = torch.randn(T, K, device=dev).bfloat16()
        res[name + "_default"] = round(graph_time([lambda w=ws[i % copies]: linear_forward(x, w) for i in range(24)]), 2)
        from gcore_b200.ops import gemm as gemm_mod
        gemm_mod._SKINNY[0] = False
        res[name + "_general_kernel"] = round(
            graph_time([lambda w=ws[i % copies]: linear_forward(x, w) for i in range(24)]), 2)
        gemm_mod._SKINNY[0] = True
        bn = 32 if T <= 32 else (64 if T <= 64 else 128)
        for ks in (2, 4):
            if (K // 64) // ks < 2:
                continue
            res[f"{name}_ksplit{ks}"] = round(graph_time(
                [lambda w=ws[i % copies]: gemm(w, x, transposed=True, bn=bn, ksplit=ks) for i in range(24)]), 2)
        res[name + "_torch"] = round(graph_time([lambda w=ws[i % copies]: torch.matmul(x, w.t()) for i in range(24)]), 2)
        res[name + "_MB"] = round(N * K * 2 / 1e6, 1)
        del ws
    # small kernels
    x = torch.randn(T, H, device=dev).bfloat16()
    r = torch.randn(T, H, device=dev).bfloat16()
    g = torch.ones(H, device=dev).bfloat16()
    res["rmsnorm_residual"] = round(graph_time([lambda: fused.rmsnorm(x, g, 1e-6, r) for _ in range(24)]), 2)
    gu = torch.randn(T, 2 * F, device=dev).bfloat16()
    res["swiglu"] = round(graph_time([lambda: fused.swiglu(gu) for _ in range(24)]), 2)
    bs, ctx_len, max_len = 16, 768, 1280
    nblk = T * (max_len // bs)
    kc = [torch.randn(nblk, bs, hk, D, device=dev).bfloat16() for _ in range(4)]
    vc = [torch.randn(nblk, bs, hk, D, device=dev).bfloat16() for _ in range(4)]
    bt = torch.arange(nblk, device=dev, dtype=torch.int32).view(T, -1)
    ctx = torch.full((T,), ctx_len, dtype=torch.int32, device=dev)
    qkv = torch.randn(T, (hq + 2 * hk) * D, device=dev).bfloat16()
    q = qkv.view(T, hq + 2 * hk, D)[:, :hq]
    res["paged_decode_ctx768"] = round(graph_time(
        [lambda i=i: paged_decode(q, kc[i % 4], vc[i % 4], bt, ctx, max_len) for i in range(24)]), 2)
    res["paged_decode_kv_MB"] = round(T * ctx_len * 2 * hk * D * 2 / 1e6, 1)
    pos = torch.full((T,), ctx_len - 1, dtype=torch.int32, device=dev)
    slots = (bt[:, (ctx_len - 1) // bs] * bs + (ctx_len - 1) % bs).to(torch.int32)
    res["kv_append_rope"] = round(graph_time(
        [lambda: kv_append_rope(qkv, pos, slots, kc[0], vc[0], hq, hk, D, 1e6) for _ in range(24)]), 2)
    # rotation + append + attention in one launch (GCORE_FUSED_KV_APPEND=0: the two kernels above in sequence)
    res["paged_decode_append_ctx768"] = round(graph_time(
        [lambda i=i: paged_decode_append(qkv, pos, slots, kc[i % 4], vc[i % 4], bt, ctx, max_len, hq, hk, D, 1e6)
         for i in range(24)]), 2)
    # one decoder layer as the rollout engine chains it (without the all-reduces)
    Hd = H
    wq = (torch.randn((hq + 2 * hk) * D, Hd, device=dev) * 0.02).bfloat16()
    wo = (torch.randn(Hd, hq * D, device=dev) * 0.02).bfloat16()
    w1 = (torch.randn(2 * F, Hd, device=dev) * 0.02).bfloat16()
    w2 = (torch.randn(Hd, F, device=dev) * 0.02).bfloat16()
    layers = [[t.clone() for t in (wq, wo, w1, w2)] for _ in range(6)]

    def layer(i):
        a, b, c, d2 = layers[i % 6]
        h, r2 = fused.rmsnorm(x, g, 1e-6, r)
        qkv2 = linear_forward(h, a)
        o = paged_decode_append(qkv2, pos, slots, kc[i % 4], vc[i % 4], bt, ctx, max_len, hq, hk, D, 1e6)
        y = linear_forward(o.view(T, hq * D), b)
        h2, _ = fused.rmsnorm(y, g, 1e-6, r2)
        return linear_forward(fused.swiglu(linear_forward(h2, c)), d2)

    res["layer_chain_us"] = round(graph_time([lambda i=i: layer(i) for i in range(12)]), 2)
    # the tail of a step: final norm, vocabulary projection (fp32 logits), sampling, state advance
    from gcore_b200.ops.vocab import sample
    V = 152064 // tp
    heads = [(torch.randn(V, H, device=dev) * 0.02).bfloat16() for _ in range(2)]
    seeds = torch.arange(T, device=dev, dtype=torch.int64)
    steps = torch.zeros(T, dtype=torch.int32, device=dev)
    toks = torch.zeros(T, dtype=torch.int64, device=dev)
    ring = torch.zeros(64, T, dtype=torch.int64, device=dev)
    ring_idx = torch.zeros(1, dtype=torch.int64, device=dev)
    res["lm_head_fp32"] = round(graph_time(
        [lambda i=i: linear_forward(x, heads[i % 2], out_dtype=torch.float32) for i in range(8)]), 2)
    res["lm_head_torch_bf16"] = round(graph_time([lambda i=i: torch.matmul(x, heads[i % 2].t()) for i in range(8)]), 2)
    logits = linear_forward(x, heads[0], out_dtype=torch.float32)
    res["sample"] = round(graph_time([lambda: sample(logits, 1.0, seeds, steps) for _ in range(8)]), 2)

    def tail(i):
        hl, _ = fused.rmsnorm(x, g, 1e-6, r)
        tok, lp = sample(linear_forward(hl, heads[i % 2], out_dtype=torch.float32), 1.0, seeds, steps)
        toks.copy_(tok)
        ring.index_copy_(0, ring_idx % 64, tok[None])
        steps.add_(1)
        ring_idx.add_(1)

    res["step_tail_us"] = round(graph_time([lambda i=i: tail(i) for i in range(8)]), 2)
    res["lm_head_MB"] = round(V * H * 2 / 1e6, 1)
    _lib.check_device_errors()
    print(json.dumps(res, indent=1))
    if args.json:
        json.dump(res, open(args.json, "w"), indent=1)


def cmd_train_step(argv=None):
    """Where does a training micro-batch spend its time?  Builds one model shard, runs forward / backward / optimizer on a"""
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--seqlen", type=int, default=1280)
    ap.add_argument("--recompute", default="full")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--profile", action="store_true")
    args = ap.parse_args(argv)
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import get_preset
    from gcore_b200.ops import _lib
    torch.cuda.set_device(0)
    mcfg = get_preset(args.model, num_layers=args.layers)
    eng = TrainingEngine(PolicyConfig(recompute=args.recompute, without_ref=True), OptimizerConfig(),
                         TrainingConfig(), model_cfg=mcfg)
    eng.setup_model_and_get_optimizer(seed=1)
    nseq = max(args.tokens // args.seqlen, 1)
    g = torch.Generator().manual_seed(0)
    samples = [{"tokens": torch.randint(100, 150000, (args.seqlen,), generator=g), "prompt_length": 256}
               for _ in range(nseq)]
    from gcore_b200.core.packing import response_mask
    for s in samples:
        s["mask"] = response_mask(256, args.seqlen)
    mb = eng._pack(samples, list(range(nseq)))

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def one(record=None):
        eng.ddp.zero_grad_buffer()
        t0 = ev()
        hidden, _ = eng._hidden(eng.model, mb)
        t1 = ev()
        lp, _ = eng._logprob_entropy(eng.model, hidden, mb.targets, False)
        loss = -(lp * mb.loss_mask).sum() / mb.loss_mask.sum()
        t2 = ev()
        loss.backward()
        t3 = ev()
        eng.ddp.finish_grad_sync()
        eng.optimizer.step(1e-6)
        t4 = ev()
        torch.cuda.synchronize()
        if record is not None:
            record.append(dict(fwd_layers_ms=t0.elapsed_time(t1), head_fwd_ms=t1.elapsed_time(t2),
                               bwd_ms=t2.elapsed_time(t3), opt_ms=t3.elapsed_time(t4)))

    eng.model.train()
    for _ in range(2):
        one()
    rec = []
    for _ in range(args.iters):
        one(rec)
    mean = {k: round(sum(r[k] for r in rec) / len(rec), 2) for k in rec[0]}
    L, T = args.layers, mb.tokens.numel()
    per_layer = mcfg.num_parameters(include_embedding=False) / mcfg.num_layers * 2 * T
    head = 2 * T * mcfg.hidden_size * mcfg.vocab_size
    mean["fwd_layers_tflops"] = round(per_layer * L / mean["fwd_layers_ms"] / 1e9, 1)
    mean["head_fwd_tflops"] = round(head / mean["head_fwd_ms"] / 1e9, 1)
    passes = 3 if args.recompute == "full" else 2
    mean["bwd_tflops"] = round((per_layer * L * passes + head * 3) / mean["bwd_ms"] / 1e9, 1)
    print(json.dumps(mean))
    if args.profile:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            one()
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=25, max_name_column_width=60))
    _lib.check_device_errors()


COMMANDS = {"table": cmd_table, "gemm": cmd_gemm, "attn": cmd_attn, "paged": cmd_paged,
            "decode_chain": cmd_decode_chain, "train_step": cmd_train_step}


def cmd_ce(argv=None):
    """Log-prob / entropy over the vocabulary: the GEMM with the softmax statistics in its epilogue against the chunked
    form (logits of 4096 tokens through the plain GEMM, one reduction pass) and against the plain GEMM alone."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--vocab", type=int, default=152064)
    ap.add_argument("--k", type=int, default=3584)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--fused-only", action="store_true", help="run only the fused kernel (for ncu captures)")
    args = ap.parse_args(argv)
    from gcore_b200.ops import _lib, vocab
    from gcore_b200.ops.gemm import linear_forward
    T, V, K = args.tokens, args.vocab, args.k
    h = torch.randn(T, K, device="cuda").bfloat16()
    w = (torch.randn(V, K, device="cuda") * 0.02).bfloat16()
    tg = torch.randint(0, V, (T,), device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn):
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        return sorted(ts)[len(ts) // 2]

    def fused():
        with torch.no_grad():
            vocab.FUSED_FWD["enabled"] = True
            return vocab.linear_logprob_entropy(h, w, tg, 1.0)

    def chunked():
        with torch.no_grad():
            vocab.FUSED_FWD["enabled"] = False
            try:
                return vocab.linear_logprob_entropy(h, w, tg, 1.0)
            finally:
                vocab.FUSED_FWD["enabled"] = True

    res = {"T": T, "V": V, "K": K, "fused_ms": round(timed(fused), 4)}
    if not args.fused_only:
        res["chunked_ms"] = round(timed(chunked), 4)
        res["plain_gemm_bf16_logits_ms"] = round(timed(lambda: linear_forward(h, w)), 4)
        res["torch_matmul_ms"] = round(timed(lambda: torch.matmul(h, w.t())), 4)
        a, b = fused(), chunked()
        res["max_abs_diff_logp"] = float((a[0] - b[0]).abs().max())
    fl = 2.0 * T * V * K
    res["fused_tflops"] = round(fl / res["fused_ms"] / 1e9, 1)
    res["partials_bytes"] = int(_lib.kernels().gk_linear_ce_splits(T, V)) * T * 16
    _lib.check_device_errors()
    print(json.dumps(res))


COMMANDS["ce"] = cmd_ce


def cmd_fused(argv=None):
    """The fused compute + collective kernels of rank 0 of 2 on ONE GPU: the peer's buffers and flags are stand-ins in
    local memory, pre-filled at the call epoch, so a single launch runs to completion alone.  Times the kernel at a
    training-sized shape (the bytes that would cross NVLink stay on this GPU: the numbers show the kernel's compute
    and memory behaviour, not link bandwidth) and is the small case profilers are pointed at."""
    import ctypes
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="ag", choices=["ag", "rs", "zero1", "ar_norm", "ep", "peer_copy"])
    ap.add_argument("--rows", type=int, default=4096, help="rows per rank (ag / rs) or tokens (ep)")
    ap.add_argument("--n", type=int, default=4608)
    ap.add_argument("--k", type=int, default=3584)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args(argv)
    from gcore_b200.ops import _lib
    lib = _lib.kernels()
    dev = "cuda"
    err = _lib.ptr(_lib.err_flag(torch.device(dev)))

    def ptrs(*ts):
        return (ctypes.c_ulonglong * len(ts))(*[t.data_ptr() for t in ts])

    def bf(*shape, scale=1.0):
        return (torch.randn(*shape, device=dev) * scale).bfloat16()

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    res = {"kernel": args.kernel}
    state = {"epoch": 0}
    if args.kernel in ("ag", "rs"):
        Tl, N, K, tp = args.rows, args.n, args.k, 2
        w = bf(N, K, scale=0.02)
        if args.kernel == "ag":
            mine = bf(tp * Tl, K)
            peer = torch.zeros_like(mine)
            flags = [torch.zeros(1 << 14, dtype=torch.int32, device=dev) for _ in range(2)]
            flags[0].fill_(1 << 30)                       # the peer's rows "have arrived" for every epoch to come
            y = torch.empty(tp * Tl, N, dtype=torch.bfloat16, device=dev)

            def launch():
                state["epoch"] += 1
                _lib.check(lib.gk_gemm_comm(1, _lib.ptr(mine), K, _lib.ptr(w), K, N, 0, _lib.ptr(y), N, None, tp * Tl, N,
                                            K, 0, tp, Tl, 16, state["epoch"], ptrs(mine, peer, flags[0], flags[1]), K, err,
                                            _lib.stream_ptr()), "ag")
            res.update(flops=2.0 * tp * Tl * N * K, nvlink_bytes=Tl * K * 2)
        else:
            a = bf(tp * Tl, K)
            inbox = torch.zeros(tp, Tl, N, dtype=torch.bfloat16, device=dev)
            peer_inbox = torch.zeros_like(inbox)
            flags = [torch.zeros(1 << 14, dtype=torch.int32, device=dev) for _ in range(2)]
            flags[0].fill_(1 << 30)
            y = torch.empty(Tl, N, dtype=torch.bfloat16, device=dev)

            def launch():
                state["epoch"] += 1
                _lib.check(lib.gk_gemm_comm(2, _lib.ptr(a), K, _lib.ptr(w), K, N, 0, _lib.ptr(y), N, None, tp * Tl, N, K, 0,
                                            tp, Tl, 0, state["epoch"], ptrs(inbox, peer_inbox, flags[0], flags[1]), N, err,
                                            _lib.stream_ptr()), "rs")
            res.update(flops=2.0 * tp * Tl * N * K, nvlink_bytes=Tl * N * 2)
    elif args.kernel == "zero1":
        n = 1 << 28                                            # 268 M parameters in this rank's shard pair
        shard = n // 2
        grads = [torch.randn(n, device=dev) for _ in range(2)]
        params = [torch.zeros(n, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        master, m, v = (torch.zeros(shard, device=dev) for _ in range(3))
        F = ctypes.c_float

        def launch():
            _lib.check(lib.gk_zero1_step(3, ptrs(*grads, *params), 0, 2, 0, shard, None, _lib.ptr(master), _lib.ptr(m),
                                         _lib.ptr(v), F(0.5), None, None, F(1e-4), F(0.9), F(0.95), F(1e-8), F(0.01), 2, 0,
                                         _lib.stream_ptr()), "zero1")
        # per element: 2 x 4 B gradients read, 12 B state read + 12 B written, 2 x 2 B parameters written
        res.update(bytes=shard * (8 + 24 + 4), nvlink_bytes=shard * (4 + 2))
    elif args.kernel == "ar_norm":
        rows, H = 128, args.k
        slot = rows * H
        x0, res_in, gamma = bf(rows, H), bf(rows, H), bf(H)
        ctas = lib.gk_allreduce_ctas()
        inbox = torch.zeros(2, 2, slot, dtype=torch.bfloat16, device=dev)
        flags = torch.full((2, 2, ctas), 1 << 30, dtype=torch.int32, device=dev)   # every epoch already "arrived"
        peer_inbox, peer_flags = torch.zeros_like(inbox), torch.zeros_like(flags)
        st = torch.zeros(4, dtype=torch.int32, device=dev)
        y, ro = torch.empty_like(x0), torch.empty_like(x0)

        def launch():
            _lib.check(lib.gk_allreduce_rmsnorm(_lib.ptr(x0), _lib.ptr(res_in), _lib.ptr(gamma), _lib.ptr(ro), _lib.ptr(y),
                                                rows, H, 1e-6, 0, 2, slot, ptrs(inbox, peer_inbox, flags, peer_flags),
                                                _lib.ptr(st), err, _lib.stream_ptr()), "ar_norm")
        res.update(bytes=rows * H * 2 * 5, nvlink_bytes=rows * H * 2)
    elif args.kernel == "peer_copy":
        rows, cols = 37888, 3584
        src = bf(rows, cols)
        dst = torch.empty(rows, cols // 2, dtype=torch.bfloat16, device=dev)

        def launch():
            _lib.check(lib.gk_peer_copy_2d(_lib.ptr(dst), cols // 2, _lib.ptr(src), cols, rows, cols // 2,
                                           _lib.stream_ptr()), "peer_copy")
        res.update(bytes=rows * cols * 2, nvlink_bytes=rows * cols)
    else:   # ep: push of T x K rows to two "ranks", pull back
        from gcore_b200.parallel.ep_fused import SEG
        T, K, H, E, ep = args.rows, 8, 2048, 128, 2
        El = E // ep
        R_max = T * K + El * SEG
        idx = torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)])
        x = bf(T, H)
        flat = idx.reshape(-1)
        cnt = torch.bincount(flat, minlength=E).int()
        order = torch.argsort(flat, stable=True)
        starts = cnt.long().cumsum(0) - cnt.long()
        pos = torch.empty_like(flat)
        pos[order] = torch.arange(flat.numel(), device=dev) - starts[flat[order]]
        tables = [torch.zeros(2, ep, E, dtype=torch.int32, device=dev) for _ in range(ep)]
        fl = [torch.zeros(2, ep, dtype=torch.int32, device=dev) for _ in range(ep)]
        tables[0][0, 1] = 0
        fl[0][0, 1] = 1
        recv = [torch.zeros(R_max, H, dtype=torch.bfloat16, device=dev) for _ in range(ep)]
        sb = torch.empty(E, dtype=torch.int32, device=dev)
        offs = torch.zeros(El + 1, dtype=torch.int32, device=dev)
        tot = torch.zeros(El, dtype=torch.int32, device=dev)
        dst_row = torch.empty(T * K, dtype=torch.int32, device=dev)
        _lib.check(lib.gk_ep_plan(_lib.ptr(cnt), ptrs(*tables, *fl), 0, ep, E, SEG, R_max, 0, _lib.ptr(sb), _lib.ptr(offs),
                                  _lib.ptr(tot), err, _lib.stream_ptr()), "ep_plan")
        wgt = torch.rand(T * K, device=dev)
        y = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        # int32 copies made once and kept alive: a temporary created inside the call expression would be released (and
        # its block handed to the next temporary) before the asynchronous kernel reads it
        flat_i, pos_i = flat.int().contiguous(), pos.int().contiguous()

        def launch():
            _lib.check(lib.gk_ep_push(_lib.ptr(x), None, _lib.ptr(flat_i), _lib.ptr(pos_i), _lib.ptr(sb),
                                      _lib.ptr(offs), _lib.ptr(tot), ptrs(*recv), _lib.ptr(dst_row), 0, ep, El, SEG, R_max,
                                      K, H, T, _lib.stream_ptr()), "ep_push")
            _lib.check(lib.gk_ep_pull(ptrs(*recv), _lib.ptr(dst_row), _lib.ptr(wgt), _lib.ptr(y), None, ep, K, H, R_max, T,
                                      _lib.stream_ptr()), "ep_pull")
        res.update(bytes=T * K * H * 2 * 4, nvlink_bytes=T * K * H * 2)
    ts = []
    for _ in range(args.iters):
        flush.zero_()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        launch()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    _lib.check_device_errors()
    ms = sorted(ts)[len(ts) // 2]
    res["ms"] = round(ms, 4)
    if "flops" in res:
        res["tflops"] = round(res.pop("flops") / ms / 1e9, 1)
    if "bytes" in res:
        res["local_gbs"] = round(res.pop("bytes") / ms / 1e6, 1)
    res["nvlink_ms_at_770GBs"] = round(res.pop("nvlink_bytes") / 770e6, 4)
    print(json.dumps(res))


COMMANDS["fused"] = cmd_fused
COMMANDS.update(COMMANDS_LATE)


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in COMMANDS:
        return COMMANDS[argv[0]](argv[1:])
    return cmd_table(argv)


if __name__ == "__main__":
    sys.exit(main())
