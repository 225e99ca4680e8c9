"""Per-kernel cost of the decode chain under CUDA-graph replay (what a rollout step actually pays per kernel).

``python -m gcore_b200.tools.decode_bench [--tokens 64] [--tp 1] [--json out.json]``

Each case captures 24 back-to-back launches that rotate over 12 independent weight copies (more bytes than the L2
holds) and reports the replay time divided by 24.
"""
from __future__ import annotations

import argparse
import json

import torch


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--json", default=None)
    ap.add_argument("--pdl", type=int, default=0, help="launch the native kernels with programmatic dependent launch")
    args = ap.parse_args()
    from gcore_b200.ops import _lib, fused
    from gcore_b200.ops.attention import kv_append_rope, paged_decode
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
        kv_append_rope(qkv2, pos, slots, kc[i % 4], vc[i % 4], hq, hk, D, 1e6)
        o = paged_decode(qkv2.view(T, hq + 2 * hk, D)[:, :hq], kc[i % 4], vc[i % 4], bt, ctx, max_len)
        y = linear_forward(o.view(T, hq * D), b)
        h2, _ = fused.rmsnorm(y, g, 1e-6, r2)
        return linear_forward(fused.swiglu(linear_forward(h2, c)), d2)

    res["layer_chain_us"] = round(graph_time([lambda i=i: layer(i) for i in range(12)]), 2)
    _lib.check_device_errors()
    print(json.dumps(res, indent=1))
    if args.json:
        json.dump(res, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
