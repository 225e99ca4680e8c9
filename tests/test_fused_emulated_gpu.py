"""Fused compute + collective kernels on ONE GPU with emulated peers: the buffers and flags a peer would own live in
this GPU's memory, pre-filled with what the peer would have written at the call's epoch, so that the kernel of one
rank runs to completion alone (no kernel ever waits for another launch).  Results are compared with fp32 PyTorch, and
what the kernel pushed to its "peers" is checked in the stand-in buffers.  The real multi-GPU runs are in
test_fused_tp_gpu.py."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from gcore_b200.ops import _lib
    return _lib


def _ptrs(*tensors):
    return (ctypes.c_ulonglong * len(tensors))(*[t.data_ptr() for t in tensors])


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def _err():
    lib = _lib()
    return lib.ptr(lib.err_flag(torch.device("cuda")))


@pytest.mark.parametrize("b_mn", [False, True])
def test_allgather_gemm_rank0_of_2(b_mn):
    lib = _lib()
    torch.manual_seed(0)
    Tl, K, N, tp = 256, 512, 768, 2
    chunks = Tl // 128
    x0, x1 = _bf(Tl, K), _bf(Tl, K)
    w = _bf(N, K, scale=0.05)
    bias = _bf(N)
    wk = w.t().contiguous() if b_mn else w
    mine = torch.zeros(tp * Tl, K, dtype=torch.bfloat16, device="cuda")
    mine[:Tl], mine[Tl:] = x0, x1                                   # rank 1's rows "have arrived"
    my_flags = torch.ones(1024, dtype=torch.int32, device="cuda")   # ... and their flags show epoch 1
    peer = torch.zeros_like(mine)
    peer_flags = torch.zeros(1024, dtype=torch.int32, device="cuda")
    y = torch.empty(tp * Tl, N, dtype=torch.bfloat16, device="cuda")
    rc = lib.kernels().gk_gemm_comm(1, lib.ptr(mine), K, lib.ptr(wk), wk.stride(0), wk.shape[0], int(b_mn), lib.ptr(y),
                                    N, lib.ptr(bias), tp * Tl, N, K, 0, tp, Tl, 2, 1,
                                    _ptrs(mine, peer, my_flags, peer_flags), K, _err(), lib.stream_ptr())
    lib.check(rc, "gemm_comm AG")
    torch.cuda.synchronize()
    lib.check_device_errors()
    ref = torch.cat([x0, x1]).float() @ w.float().t() + bias.float()
    assert torch.allclose(y.float(), ref, atol=0.06, rtol=0.02), (y.float() - ref).abs().max()
    assert torch.equal(peer[:Tl], x0) and not peer[Tl:].any()       # my rows were pushed, nothing else touched
    assert peer_flags[:chunks].tolist() == [1] * chunks             # flags[src = 0][chunk]
    assert not peer_flags[chunks:].any()


def test_gemm_reduce_scatter_rank0_of_2():
    lib = _lib()
    torch.manual_seed(1)
    Tl, K, N, tp = 256, 384, 512, 2
    a = _bf(tp * Tl, K)
    w = _bf(N, K, scale=0.05)
    full = a.float() @ w.float().t()
    peer_part = _bf(Tl, N)                                          # rank 1's partial for my rows
    inbox = torch.zeros(tp, Tl, N, dtype=torch.bfloat16, device="cuda")
    inbox[1] = peer_part
    my_flags = torch.ones(4096, dtype=torch.int32, device="cuda")
    peer_inbox = torch.zeros_like(inbox)
    peer_flags = torch.zeros(4096, dtype=torch.int32, device="cuda")
    y = torch.empty(Tl, N, dtype=torch.bfloat16, device="cuda")
    rc = lib.kernels().gk_gemm_comm(2, lib.ptr(a), K, lib.ptr(w), K, N, 0, lib.ptr(y), N, None, tp * Tl, N, K, 0, tp,
                                    Tl, 0, 1, _ptrs(inbox, peer_inbox, my_flags, peer_flags), N, _err(),
                                    lib.stream_ptr())
    lib.check(rc, "gemm_comm RS")
    torch.cuda.synchronize()
    lib.check_device_errors()
    ref = full[:Tl] + peer_part.float()
    assert torch.allclose(y.float(), ref, atol=0.08, rtol=0.02), (y.float() - ref).abs().max()
    # my partial of the rows rank 1 owns went to slot [src = 0] of its inbox, with one flag per tile
    assert torch.allclose(peer_inbox[0].float(), full[Tl:], atol=0.06, rtol=0.02)
    assert not peer_inbox[1].any()
    n_tiles = (Tl // 128) * ((N + 255) // 256)
    assert int((peer_flags == 1).sum()) == n_tiles and int((peer_flags != 0).sum()) == n_tiles


def _adamw(master, m, v, g, lr, b1, b2, eps, wd, step):
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    upd = (m / (1 - b1 ** step)) / ((v / (1 - b2 ** step)).sqrt() + eps) + wd * master
    return master - lr * upd, m, v


@pytest.mark.parametrize("clip", [False, True])
def test_zero1_two_ranks_sequential(clip):
    """Both ranks' optimizer kernels, one after the other (the kernel itself never waits: ranks are ordered by a
    separate barrier kernel).  Afterwards both parameter buffers hold both updated shards."""
    lib = _lib()
    torch.manual_seed(2)
    n, tp = 8192, 2
    shard = n // tp
    grads = [torch.randn(n, device="cuda") for _ in range(tp)]
    params = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(tp)]
    master0 = torch.randn(n, device="cuda")
    state = [dict(master=master0[r * shard:(r + 1) * shard].clone(), m=torch.zeros(shard, device="cuda"),
                  v=torch.zeros(shard, device="cuda")) for r in range(tp)]
    lr, b1, b2, eps, wd, step, scale = 1e-2, 0.9, 0.95, 1e-8, 0.1, 3, 0.5
    ptrs = _ptrs(*grads, *params)
    gsum = (grads[0] + grads[1]) * scale
    k = lib.kernels()
    F = ctypes.c_float
    if not clip:
        sumsq = torch.zeros(1, device="cuda")
        for r in range(tp):
            st = state[r]
            lib.check(k.gk_zero1_step(3, ptrs, r, tp, r * shard, shard, None, lib.ptr(st["master"]), lib.ptr(st["m"]),
                                      lib.ptr(st["v"]), F(scale), None, lib.ptr(sumsq), F(lr), F(b1), F(b2), F(eps),
                                      F(wd), step, 0, lib.stream_ptr()), "zero1")
        coef = 1.0
    else:
        sumsq = torch.zeros(1, device="cuda")
        reduced = [torch.empty(shard, device="cuda") for _ in range(tp)]
        for r in range(tp):
            st = state[r]
            lib.check(k.gk_zero1_step(1, ptrs, r, tp, r * shard, shard, lib.ptr(reduced[r]), lib.ptr(st["master"]),
                                      lib.ptr(st["m"]), lib.ptr(st["v"]), F(scale), None, lib.ptr(sumsq), F(lr),
                                      F(b1), F(b2), F(eps), F(wd), step, 0, lib.stream_ptr()), "zero1 reduce")
        coef = min(1.0, 1.0 / (float(sumsq.sqrt()) + 1e-6))
        cl = torch.tensor([coef], device="cuda")
        for r in range(tp):
            st = state[r]
            lib.check(k.gk_zero1_step(2, ptrs, r, tp, r * shard, shard, lib.ptr(reduced[r]), lib.ptr(st["master"]),
                                      lib.ptr(st["m"]), lib.ptr(st["v"]), F(scale), lib.ptr(cl), None, F(lr), F(b1),
                                      F(b2), F(eps), F(wd), step, 0, lib.stream_ptr()), "zero1 update")
    torch.cuda.synchronize()
    assert abs(float(sumsq) - float((gsum.double() ** 2).sum())) < 1e-3 * float((gsum.double() ** 2).sum())
    new, _, _ = _adamw(master0, torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), gsum * coef, lr, b1, b2,
                       eps, wd, step)
    assert torch.allclose(torch.cat([s["master"] for s in state]), new, atol=1e-5, rtol=1e-5)
    for r in range(tp):
        assert torch.equal(params[r], new.bfloat16()) or torch.allclose(params[r].float(), new, atol=0.02, rtol=0.01)
    assert torch.equal(params[0], params[1])


def test_zero1_norm_is_bitwise_reproducible():
    lib = _lib()
    torch.manual_seed(3)
    n = 1 << 20
    g = [torch.randn(n, device="cuda"), torch.randn(n, device="cuda")]
    p = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    red = torch.empty(n, device="cuda")
    outs = []
    F = ctypes.c_float
    for _ in range(4):
        ss = torch.zeros(1, device="cuda")
        lib.check(lib.kernels().gk_zero1_step(1, _ptrs(*g, *p), 0, 2, 0, n, lib.ptr(red), None, None, None, F(1.0),
                                              None, lib.ptr(ss), F(0), F(0.9), F(0.95), F(1e-8), F(0), 1, 0,
                                              lib.stream_ptr()), "zero1 norm")
        outs.append(float(ss))
    assert len(set(outs)) == 1, outs


def test_allreduce_oneshot_rank0_of_2():
    lib = _lib()
    torch.manual_seed(4)
    k = lib.kernels()
    ctas = k.gk_allreduce_ctas()
    n, tp, slot = 64 * 3584, 2, 64 * 3584
    x0, x1 = _bf(n), _bf(n)
    inbox = torch.zeros(2, tp, slot, dtype=torch.bfloat16, device="cuda")
    inbox[0, 1] = x1
    flags = torch.zeros(2, tp, ctas, dtype=torch.int32, device="cuda")
    flags[0, 1] = 1
    peer_inbox, peer_flags = torch.zeros_like(inbox), torch.zeros_like(flags)
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.empty_like(x0)
    lib.check(k.gk_allreduce_oneshot(lib.ptr(x0), lib.ptr(out), n, 0, tp, slot, _ptrs(inbox, peer_inbox, flags, peer_flags),
                                     lib.ptr(state), _err(), lib.stream_ptr()), "allreduce")
    torch.cuda.synchronize()
    lib.check_device_errors()
    assert torch.equal(out, (x0.float() + x1.float()).bfloat16())
    assert torch.equal(peer_inbox[0, 0], x0) and not peer_inbox[1].any()
    assert peer_flags[0, 0].tolist() == [1] * ctas
    assert state[:2].tolist() == [1, 0]                              # call counter advanced, ticket reset


@pytest.mark.parametrize("with_res", [True, False])
def test_allreduce_residual_rmsnorm_rank0_of_2(with_res):
    """One kernel = all-reduce, residual add and RMSNorm: the residual stream bit-identical to the three steps done one
    after the other, the normalised output to rounding."""
    lib = _lib()
    from gcore_b200.ops import fused
    torch.manual_seed(7)
    k = lib.kernels()
    ctas = k.gk_allreduce_ctas()
    rows, H, tp = 100, 3584, 2                        # 100 rows over 32 CTAs: uneven, some CTAs own no row
    slot = 128 * H
    x0, x1 = _bf(rows, H), _bf(rows, H)
    res = _bf(rows, H) if with_res else None
    gamma = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    inbox = torch.zeros(2, tp, slot, dtype=torch.bfloat16, device="cuda")
    inbox[0, 1, :rows * H] = x1.reshape(-1)
    flags = torch.zeros(2, tp, ctas, dtype=torch.int32, device="cuda")
    flags[0, 1] = 1
    peer_inbox, peer_flags = torch.zeros_like(inbox), torch.zeros_like(flags)
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    y, res_out = torch.empty_like(x0), torch.empty_like(x0)
    lib.check(k.gk_allreduce_rmsnorm(lib.ptr(x0), lib.ptr(res), lib.ptr(gamma), lib.ptr(res_out), lib.ptr(y), rows, H,
                                     1e-6, 0, tp, slot, _ptrs(inbox, peer_inbox, flags, peer_flags), lib.ptr(state),
                                     _err(), lib.stream_ptr()), "allreduce_rmsnorm")
    torch.cuda.synchronize()
    lib.check_device_errors()
    summed = (x0.float() + x1.float()).bfloat16()
    y_ref, res_ref = fused.rmsnorm(summed, gamma, 1e-6, res)
    assert torch.equal(res_out, res_ref if with_res else summed)
    assert torch.allclose(y.float(), y_ref.float(), atol=2e-2, rtol=1e-2)   # sum of squares added in another order
    assert torch.equal(peer_inbox[0, 0, :rows * H], x0.reshape(-1))
    assert peer_flags[0, 0].tolist() == [1] * ctas                   # CTAs without rows still publish their flag
    assert state[:2].tolist() == [1, 0]


def test_expert_dispatch_combine_two_ranks_sequential():
    """ep_plan / ep_push / ep_pull of both ranks of an expert-parallel pair, run in an order in which no kernel has to
    wait: rank 1's counts are placed in rank 0's table before rank 0 plans; rank 0's plan publishes its counts to
    rank 1 before rank 1 plans."""
    lib = _lib()
    from gcore_b200.parallel.ep_fused import SEG
    torch.manual_seed(5)
    k = lib.kernels()
    ep, E, K, H, T = 2, 8, 2, 256, 96
    El = E // ep
    R_max = 2 * T * K + El * SEG
    idx = [torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(T)]) for _ in range(ep)]
    x = [_bf(T, H) for _ in range(ep)]
    wgt = [torch.rand(T, K, device="cuda") for _ in range(ep)]
    tables = [torch.zeros(2, ep, E, dtype=torch.int32, device="cuda") for _ in range(ep)]
    flags = [torch.zeros(2, ep, dtype=torch.int32, device="cuda") for _ in range(ep)]
    recv = [torch.full((R_max, H), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(ep)]
    cnts = [torch.bincount(i.reshape(-1), minlength=E).int() for i in idx]
    tables[0][0, 1] = cnts[1]
    flags[0][0, 1] = 1
    st = []
    for r in range(ep):
        flat = idx[r].reshape(-1)
        order = torch.argsort(flat, stable=True)
        starts = cnts[r].long().cumsum(0) - cnts[r].long()
        pos = torch.empty_like(flat)
        pos[order] = torch.arange(flat.numel(), device="cuda") - starts[flat[order]]
        s = dict(idx=flat.int(), pos=pos.int(), send_base=torch.empty(E, dtype=torch.int32, device="cuda"),
                 offsets=torch.zeros(El + 1, dtype=torch.int32, device="cuda"),
                 tot=torch.zeros(El, dtype=torch.int32, device="cuda"),
                 dst_row=torch.empty(T * K, dtype=torch.int32, device="cuda"))
        lib.check(k.gk_ep_plan(lib.ptr(cnts[r]), _ptrs(*tables, *flags), r, ep, E, SEG, R_max, 0, lib.ptr(s["send_base"]),
                               lib.ptr(s["offsets"]), lib.ptr(s["tot"]), _err(), lib.stream_ptr()), "ep_plan")
        st.append(s)
    torch.cuda.synchronize()
    lib.check_device_errors()
    tot = cnts[0] + cnts[1]
    for r in range(ep):
        assert st[r]["tot"].tolist() == tot[r * El:(r + 1) * El].tolist()
        offs = st[r]["offsets"].tolist()
        assert offs[0] == 0 and all(o % SEG == 0 for o in offs)
        assert all(offs[e + 1] - offs[e] >= st[r]["tot"][e] for e in range(El))
    for r in range(ep):
        s = st[r]
        lib.check(k.gk_ep_push(lib.ptr(x[r]), None, lib.ptr(s["idx"]), lib.ptr(s["pos"]), lib.ptr(s["send_base"]),
                               lib.ptr(s["offsets"]), lib.ptr(s["tot"]), _ptrs(*recv), lib.ptr(s["dst_row"]), r, ep, El,
                               SEG, R_max, K, H, T, lib.stream_ptr()), "ep_push")
    torch.cuda.synchronize()
    # every expert's segment holds rank 0's rows, then rank 1's, in token order; padding rows are zero
    for d in range(ep):
        offs = st[d]["offsets"].tolist()
        for e in range(El):
            g = d * El + e
            want = torch.cat([x[r][(idx[r] == g).any(-1)] for r in range(ep)])
            got = recv[d][offs[e]:offs[e] + want.shape[0]]
            assert torch.equal(got, want), (d, e)
            assert not recv[d][offs[e] + want.shape[0]:offs[e + 1]].any()
    # "experts": scale every row by (1 + global expert id); then combine
    yout = []
    for d in range(ep):
        offs = st[d]["offsets"].tolist()
        y = recv[d].clone()
        for e in range(El):
            y[offs[e]:offs[e + 1]] = (y[offs[e]:offs[e + 1]].float() * (1 + d * El + e)).bfloat16()
        yout.append(y)
    for r in range(ep):
        out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
        gathered = torch.empty(T * K, H, dtype=torch.bfloat16, device="cuda")
        lib.check(k.gk_ep_pull(_ptrs(*yout), lib.ptr(st[r]["dst_row"]), lib.ptr(wgt[r].reshape(-1).contiguous()),
                               lib.ptr(out), lib.ptr(gathered), ep, K, H, R_max, T, lib.stream_ptr()), "ep_pull")
        torch.cuda.synchronize()
        rows = (x[r].float()[:, None, :] * (1 + idx[r].float())[:, :, None]).bfloat16()        # [T, K, H]
        assert torch.equal(gathered.view(T, K, H), rows)
        ref = (rows.float() * wgt[r][:, :, None]).sum(1)
        assert torch.allclose(out.float(), ref, atol=0.05, rtol=0.01)


def test_peer_copy_2d_and_rows():
    lib = _lib()
    torch.manual_seed(6)
    k = lib.kernels()
    src = _bf(300, 512)
    dst = torch.zeros(300, 256, dtype=torch.bfloat16, device="cuda")
    lib.check(k.gk_peer_copy_2d(lib.ptr(dst[:, 64:]), 256, lib.ptr(src[:, 128:]), 512, 300, 192, lib.stream_ptr()),
              "peer_copy_2d")
    torch.cuda.synchronize()
    assert torch.equal(dst[:, 64:], src[:, 128:320]) and not dst[:, :64].any()
    # gather of three "peers'" segments into one flat buffer; the gap stays zero
    a, b, c = _bf(4096), _bf(4096), _bf(4096)
    out = torch.full((8192,), 3.0, dtype=torch.bfloat16, device="cuda")
    segs = (ctypes.c_ulonglong * 9)(a.data_ptr(), 0, 2048, b.data_ptr() + 2 * 1024, 2048, 4096, c.data_ptr(), 6144, 8192)
    lib.check(k.gk_peer_rows(lib.ptr(out), 8192, 3, segs, lib.stream_ptr()), "peer_rows")
    torch.cuda.synchronize()
    assert torch.equal(out[:2048], a[:2048]) and torch.equal(out[2048:4096], b[1024:3072])
    assert not out[4096:6144].any() and torch.equal(out[6144:], c[:2048])
    # overlapping segments are summed in segment order with fp32 accumulation (the return path of partial dK / dV)
    segs = (ctypes.c_ulonglong * 6)(a.data_ptr(), 0, 4096, b.data_ptr(), 1024, 4096)
    out2 = torch.empty(4096, dtype=torch.bfloat16, device="cuda")
    lib.check(k.gk_peer_rows(lib.ptr(out2), 4096, 2, segs, lib.stream_ptr()), "peer_rows")
    torch.cuda.synchronize()
    assert torch.equal(out2[:1024], a[:1024])
    assert torch.equal(out2[1024:], (a[1024:].float() + b[:3072].float()).bfloat16())
