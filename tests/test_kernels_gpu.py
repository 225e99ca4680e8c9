"""GPU numerics of every hand-written kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(dtype)


def _close(a, b, rtol=2e-2, atol=2e-2):
    """Three criteria: (1) the largest error against the largest reference magnitude, (2) element by element,
    ``|a - b| <= atol + rtol * |b|`` with at most one element in 10^4 beyond it (a kernel that is wrong on the small
    elements only passes (1) but not this one), (3) the relative RMS error of the whole tensor."""
    a, b = a.float(), b.float()
    if a.numel() == 0:
        return
    diff = (a - b).abs()
    err = diff.max().item()
    ref = b.abs().max().item()
    assert err <= atol + rtol * ref, f"max err {err} vs ref magnitude {ref}"
    bad = (diff > atol + rtol * b.abs()).float().mean().item()
    assert bad <= 1e-4, f"{bad:.2e} of the elements are outside atol {atol} + rtol {rtol} * |ref|"
    rms = (diff.norm() / b.norm().clamp_min(1e-20)).item()
    assert rms <= max(4 * rtol, 2e-2) or diff.norm().item() <= atol * math.sqrt(a.numel()), \
        f"relative RMS error {rms:.3e}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (300, 200, 136), (1000, 3584, 1024), (64, 96, 64)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    from gcore_b200.ops.gemm import gemm
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a 16-byte aligned leading dimension")
    torch.manual_seed(0)
    A = _rand(M, K, scale=0.5)
    B = _rand(N, K, scale=0.5)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    ref = A.float() @ B.float().t()
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    _close(out, ref, rtol=1e-2, atol=1e-2 * math.sqrt(K))
    out32 = gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    _close(out32, ref, rtol=2e-3, atol=2e-3 * math.sqrt(K))


@pytest.mark.parametrize("bn", [32, 64, 128, 256])
def test_gemm_tile_widths_bias_accumulate(bn):
    from gcore_b200.ops.gemm import gemm
    torch.manual_seed(1)
    M, N, K = 384, 520, 320
    A, B = _rand(M, K, scale=0.5), _rand(N, K, scale=0.5)
    bias = _rand(N)
    C0 = torch.randn(M, N, device=DEV, dtype=torch.float32)
    out = C0.clone()
    gemm(A, B, out=out, bias=bias, alpha=0.5, accumulate=True, bn=bn)
    ref = C0 + 0.5 * (A.float() @ B.float().t()) + bias.float()[None]
    _close(out, ref, rtol=2e-3, atol=2e-2)


@pytest.mark.parametrize("T", [1, 5, 32, 64, 100, 128])
def test_gemm_decode_swap_ab_splitk(T):
    from gcore_b200.ops.gemm import linear_forward
    torch.manual_seed(2)
    K, N = 3584, 4608
    x, w, bias = _rand(T, K, scale=0.3), _rand(N, K, scale=0.05), _rand(N)
    ref = x.float() @ w.float().t() + bias.float()[None]
    y = linear_forward(x, w, bias)
    assert y.shape == (T, N)
    _close(y, ref, rtol=1e-2, atol=3e-2)
    y2 = linear_forward(x, w, bias)  # counters must have been reset by the first call
    assert torch.equal(y, y2)


def test_gemm_grouped_ragged():
    from gcore_b200.ops.gemm import grouped_gemm, grouped_wgrad
    torch.manual_seed(3)
    G, K, N = 5, 256, 384
    real = [100, 0, 257, 128, 31]
    padded = [((r + 127) // 128) * 128 for r in real]
    offs = [0]
    for p in padded:
        offs.append(offs[-1] + p)
    Mtot = offs[-1]
    x = torch.zeros(Mtot, K, device=DEV, dtype=torch.bfloat16)
    for g in range(G):
        x[offs[g]:offs[g] + real[g]] = _rand(real[g], K, scale=0.5)
    w = _rand(G, N, K, scale=0.1)
    offsets = torch.tensor(offs, device=DEV, dtype=torch.int32)
    y = grouped_gemm(x, w, offsets)
    for g in range(G):
        s, e = offs[g], offs[g] + real[g]
        _close(y[s:e], x[s:e].float() @ w[g].float().t(), rtol=1e-2, atol=5e-2)
    # dgrad layout: weights given as [G, K_contract, N_out]
    wt = w.transpose(1, 2).contiguous()  # [G, K, N]: y = x @ wt[g]
    y2 = grouped_gemm(x, wt, offsets, b_mn=True)
    _close(y2, y, rtol=1e-2, atol=5e-2)
    dy = torch.zeros(Mtot, N, device=DEV, dtype=torch.bfloat16)
    for g in range(G):
        dy[offs[g]:offs[g] + real[g]] = _rand(real[g], N, scale=0.5)
    dw = grouped_wgrad(dy, x, offsets, G)
    for g in range(G):
        s, e = offs[g], offs[g + 1]
        _close(dw[g], dy[s:e].float().t() @ x[s:e].float(), rtol=5e-3, atol=5e-2)


def test_linear_autograd_matches_torch():
    from gcore_b200.ops.gemm import linear
    torch.manual_seed(4)
    x = _rand(200, 512, scale=0.5).requires_grad_(True)
    w = _rand(768, 512, scale=0.05).requires_grad_(True)
    b = _rand(768).requires_grad_(True)
    y = linear(x, w, b)
    g = _rand(200, 768)
    y.backward(g)
    xr, wr, br = [t.detach().float().requires_grad_(True) for t in (x, w, b)]
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    _close(y, yr, atol=5e-2)
    _close(x.grad, xr.grad, atol=5e-2)
    _close(w.grad, wr.grad, atol=1e-1)
    _close(b.grad, br.grad, atol=1e-1)


@pytest.mark.parametrize("T,H", [(7, 256), (513, 3584), (64, 8192)])
def test_rmsnorm_fwd_bwd(T, H):
    from gcore_b200.ops.fused import rmsnorm, rmsnorm_ref
    torch.manual_seed(5)
    x, r, w = _rand(T, H), _rand(T, H), (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    for res in (None, r):
        xi = x.clone().requires_grad_(True)
        ri = res.clone().requires_grad_(True) if res is not None else None
        wi = w.clone().requires_grad_(True)
        y, s = rmsnorm(xi, wi, 1e-6, ri)
        gy, gs = _rand(T, H), _rand(T, H)
        (y.float() * gy.float()).sum().add((s.float() * gs.float()).sum()).backward()
        xf = x.float().requires_grad_(True)
        rf = res.float().requires_grad_(True) if res is not None else None
        wf = w.float().requires_grad_(True)
        yr, sr = rmsnorm_ref(xf, wf, 1e-6, rf)
        (yr * gy.float()).sum().add((sr * gs.float()).sum()).backward()
        _close(y, yr)
        _close(s, sr)
        _close(xi.grad, xf.grad, atol=5e-2)
        _close(wi.grad, wf.grad, rtol=2e-2, atol=0.5)
        if res is not None:
            _close(ri.grad, rf.grad, atol=5e-2)


def test_rope_and_swiglu():
    from gcore_b200.ops.fused import rope, rope_ref, swiglu, swiglu_ref
    torch.manual_seed(6)
    T, nh, D = 300, 6, 128
    x = _rand(T, nh, D).requires_grad_(True)
    pos = torch.randint(0, 4000, (T,), device=DEV, dtype=torch.int32)
    y = rope(x, pos, 1e6)
    g = _rand(T, nh, D)
    y.backward(g)
    xf = x.detach().float().requires_grad_(True)
    yr = rope_ref(xf, pos, 1e6)
    yr.backward(g.float())
    _close(y, yr)
    _close(x.grad, xf.grad)
    # partial rotary + packed slice
    buf = _rand(T, 3 * nh * D)
    view = buf.view(T, 3 * nh, D)[:, :nh]
    from gcore_b200.ops.fused import rope_inplace
    ref = rope_ref(view.clone(), pos, 1e4, rot=64)
    rope_inplace(view, pos, 1e4, rot=64)
    _close(view, ref)
    z = _rand(257, 2 * 688).requires_grad_(True)
    o = swiglu(z)
    go = _rand(257, 688)
    o.backward(go)
    zf = z.detach().float().requires_grad_(True)
    orf = swiglu_ref(zf)
    orf.backward(go.float())
    _close(o, orf)
    _close(z.grad, zf.grad)


def test_linear_logprob_entropy_fwd_bwd():
    from gcore_b200.ops import vocab
    torch.manual_seed(7)
    T, H, V = 300, 256, 5000
    old = vocab.CHUNK_TOKENS
    vocab.CHUNK_TOKENS = 128
    try:
        h = _rand(T, H, scale=1.0).requires_grad_(True)
        w = _rand(V, H, scale=0.1).requires_grad_(True)
        tg = torch.randint(0, V, (T,), device=DEV)
        lp, en = vocab.linear_logprob_entropy(h, w, tg, temperature=0.7)
        g1, g2 = torch.randn(T, device=DEV), torch.randn(T, device=DEV)
        (lp * g1 + en * g2).sum().backward()
        hf, wf = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
        lpr, enr = vocab.logprob_entropy_ref(hf @ wf.t(), tg, 0.7)
        (lpr * g1 + enr * g2).sum().backward()
        _close(lp, lpr, atol=5e-2)
        _close(en, enr, atol=5e-2)
        _close(h.grad, hf.grad, atol=5e-2)
        _close(w.grad, wf.grad, atol=5e-2)
    finally:
        vocab.CHUNK_TOKENS = old


@pytest.mark.parametrize("T,H,V,vs", [(300, 256, 5000, 0), (1024, 512, 33000, 0), (130, 192, 777, 1000)])
def test_fused_linear_stats_never_writes_logits(T, H, V, vs):
    """The vocabulary GEMM with the softmax statistics in its epilogue against the fp32 definition, including a
    vocabulary that is not a multiple of the tile, rows that are not a multiple of 128 and targets outside the
    local vocabulary shard."""
    from gcore_b200.ops import _lib, vocab
    torch.manual_seed(17)
    h = _rand(T, H, scale=1.0)
    w = _rand(V, H, scale=0.1)
    tg = torch.randint(vs - 50 if vs else 0, vs + V + (50 if vs else 0), (T,), device=DEV).clamp_min(0)
    part = vocab.fused_linear_stats(h, w, tg, 1.0 / 0.7, vs)
    _lib.check_device_errors()
    assert part.shape[1:] == (T, 4)
    z = (h.float() @ w.float().t()) / 0.7
    lp, en, lse = vocab._combine(part, T)
    lse_ref = torch.logsumexp(z, -1)
    _close(lse, lse_ref, atol=2e-3)
    _close(en, lse_ref - (torch.softmax(z, -1) * z).sum(-1), atol=5e-3)
    local = tg - vs
    mine = (local >= 0) & (local < V)
    zt_ref = z.gather(-1, local.clamp(0, V - 1)[:, None]).squeeze(-1)
    _close(lp[mine], (zt_ref - lse_ref)[mine], atol=5e-3)
    assert (part[:, :, 3].max(0).values[~mine] < -1e30).all()        # no split claims a target it does not own


@pytest.mark.parametrize("E,K,G,TG,sigmoid,norm,scale,use_bias", [
    (128, 8, 1, 1, False, True, 1.0, False), (64, 4, 1, 1, False, False, 1.0, False),
    (256, 8, 8, 4, True, True, 2.5, True), (32, 2, 4, 2, True, False, 1.0, True), (512, 16, 1, 1, True, True, 1.0, False)])
def test_router_kernel_matches_reference(E, K, G, TG, sigmoid, norm, scale, use_bias):
    from gcore_b200.ops.router import route, route_ref
    torch.manual_seed(21)
    T = 777
    logits = torch.randn(T, E, device=DEV, dtype=torch.float32, requires_grad=True)
    bias = torch.randn(E, device=DEV) * 0.3 if use_bias else None
    idx, w = route(logits, bias, None, K, G, TG, sigmoid, norm, scale)
    lr = logits.detach().clone().requires_grad_(True)
    idx_r, w_r = route_ref(lr, bias, None, K, G, TG, sigmoid, norm, scale)
    assert torch.equal(idx.sort(-1).values, idx_r.sort(-1).values)
    # same experts, possibly listed in another order: compare weights per expert
    dense = torch.zeros(T, E, device=DEV).scatter(1, idx, w)
    dense_r = torch.zeros(T, E, device=DEV).scatter(1, idx_r, w_r)
    assert torch.allclose(dense, dense_r, atol=1e-5, rtol=1e-4)
    coef = torch.randn(T, E, device=DEV)
    (dense * coef).sum().backward()
    (dense_r * coef).sum().backward()
    assert torch.allclose(logits.grad, lr.grad, atol=1e-5, rtol=1e-3), (logits.grad - lr.grad).abs().max()
    # forced expert ids (routing replay) give the reference's weights for those ids
    forced = torch.stack([torch.randperm(E, device=DEV)[:K] for _ in range(T)])
    idx_f, w_f = route(logits.detach(), bias, forced, K, G, TG, sigmoid, norm, scale)
    _, w_fr = route_ref(logits.detach(), bias, forced, K, G, TG, sigmoid, norm, scale)
    assert torch.equal(idx_f, forced) and torch.allclose(w_f, w_fr, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("top_k,top_p,min_p", [(50, 1.0, 0.0), (0, 0.9, 0.0), (200, 0.8, 0.0), (0, 1.0, 0.05),
                                                (1000, 0.95, 0.01)])
def test_filtered_sampling_matches_sort_based_definition(top_k, top_p, min_p):
    from gcore_b200.ops.vocab import apply_top_k_top_p, sample_filtered
    torch.manual_seed(23)
    B, V, temp = 48, 50000, 0.8
    logits = (torch.randn(B, V, device=DEV) * 2.5).contiguous()
    seeds = torch.arange(B, device=DEV, dtype=torch.int64)
    steps = torch.full((B,), 3, device=DEV, dtype=torch.int32)
    tok, lp, kept = sample_filtered(logits, temp, top_k, top_p, min_p, seeds, steps, return_kept=True)
    z = apply_top_k_top_p(logits / temp, top_k, top_p, min_p)
    kept_ref = torch.isfinite(z).sum(-1)
    # keys quantise the logits to 2.4e-6: the kept sets may differ by elements that close to the cut
    assert (kept.long() - kept_ref).abs().max() <= 1, (kept, kept_ref)
    assert torch.isfinite(z.gather(-1, tok[:, None])).all()          # every drawn token is inside the reference set
    lp_ref = torch.log_softmax(z, -1).gather(-1, tok[:, None]).squeeze(-1)
    assert torch.allclose(lp, lp_ref, atol=2e-3), (lp - lp_ref).abs().max()
    # the draw is Gumbel-max with the sampler's random stream: same token as the unfiltered sampler run on the
    # masked logits
    from gcore_b200.ops.vocab import sample
    tok_ref, _ = sample(z.contiguous(), 1.0, seeds, steps)
    same = (kept.long() == kept_ref)
    assert torch.equal(tok[same], tok_ref[same])
    tok_g, _ = sample_filtered(logits, temp, top_k, top_p, min_p, seeds, steps, greedy=True)
    assert torch.equal(tok_g, logits.argmax(-1))


def test_sampling_is_independent_of_row_slicing():
    """Large vocabularies are sampled by several CTAs per row; the draw and its log-prob equal the one-CTA result."""
    from gcore_b200.ops import _lib
    from gcore_b200.ops.vocab import sample
    torch.manual_seed(29)
    B, V = 24, 40000
    logits = (torch.randn(B, V, device=DEV) * 3).contiguous()
    seeds = torch.arange(B, device=DEV, dtype=torch.int64) + 5
    steps = torch.full((B,), 11, device=DEV, dtype=torch.int32)
    tok, lp = sample(logits, 0.9, seeds, steps)
    tok1 = torch.empty(B, dtype=torch.int64, device=DEV)
    lp1 = torch.empty(B, dtype=torch.float32, device=DEV)
    _lib.check(_lib.kernels().gk_sample(_lib.ptr(logits), 1, V, V, 0, 1.0 / 0.9, 0, _lib.ptr(seeds), _lib.ptr(steps),
                                        _lib.ptr(tok1), _lib.ptr(lp1), None, B, 1, _lib.stream_ptr()), "sample")
    assert torch.equal(tok, tok1)
    assert torch.allclose(lp, lp1, atol=1e-4)
    ref = torch.log_softmax(logits / 0.9, -1).gather(-1, tok[:, None]).squeeze(-1)
    assert torch.allclose(lp, ref, atol=1e-3)


def test_sampling_distribution_and_logprob():
    from gcore_b200.ops.vocab import sample
    torch.manual_seed(8)
    V = 50
    logits = torch.randn(1, V, device=DEV).repeat(4096, 1).contiguous()
    seeds = torch.arange(4096, device=DEV, dtype=torch.int64)
    steps = torch.zeros(4096, device=DEV, dtype=torch.int32)
    tok, lp = sample(logits, 1.0, seeds, steps)
    ref_lp = torch.log_softmax(logits[0], -1)
    assert torch.allclose(lp, ref_lp[tok], atol=1e-4)
    freq = torch.bincount(tok, minlength=V).float() / 4096
    assert (freq - ref_lp.exp()).abs().max().item() < 0.03
    tok2, _ = sample(logits, 1.0, seeds, steps)
    assert torch.equal(tok, tok2)
    tokg, _ = sample(logits, 1.0, seeds, steps, greedy=True)
    assert (tokg == logits[0].argmax()).all()


def test_grpo_loss_and_gae():
    from gcore_b200.ops.rl import gae, grpo_loss, grpo_token_loss_ref
    torch.manual_seed(9)
    n = 5000
    logp = (-torch.rand(n, device=DEV) * 3).requires_grad_(True)
    old = logp.detach() + 0.3 * torch.randn(n, device=DEV)
    ref = logp.detach() + 0.2 * torch.randn(n, device=DEV)
    adv = torch.randn(n, device=DEV)
    w = (torch.rand(n, device=DEV) > 0.3).float() / n
    kw = dict(clip_low=0.2, clip_high=0.28, dual_clip_c=3.0, kl_beta=0.01, ratio_clamp=10.0, kl_clamp=5.0)
    loss, stats = grpo_loss(logp, old, ref, adv, w, **kw)
    loss.backward()
    lr = logp.detach().clone().requires_grad_(True)
    tl, kl, ratio, clipped = grpo_token_loss_ref(lr, old, ref, adv, **kw)
    (w * tl).sum().backward()
    assert abs(loss.item() - (w * tl).sum().item()) < 1e-4
    assert torch.allclose(logp.grad, lr.grad, atol=1e-6)
    assert abs(stats[3].item() - (w * clipped.float()).sum().item()) < 1e-5
    B, S = 37, 129
    r, v = torch.randn(B, S, device=DEV), torch.randn(B, S, device=DEV)
    mk = (torch.rand(B, S, device=DEV) > 0.2).float()
    a1, r1 = gae(r, v, mk, 0.99, 0.95)
    a2, r2 = gae(r.cpu(), v.cpu(), mk.cpu(), 0.99, 0.95)
    assert torch.allclose(a1.cpu(), a2, atol=1e-4) and torch.allclose(r1.cpu(), r2, atol=1e-4)


def test_adam_and_sumsq():
    from gcore_b200.ops.optim import adam_step, sumsq
    torch.manual_seed(10)
    n = 100003
    master = torch.randn(n, device=DEV)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    g = torch.randn(n, device=DEV).bfloat16()
    p = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    mc, mm, vv = master.cpu().clone(), m.cpu().clone(), v.cpu().clone()
    scale = torch.tensor([0.5], device=DEV)
    for step in (1, 2):
        adam_step(master, m, v, g, p, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                  grad_scale=scale)
        adam_step(mc, mm, vv, g.cpu(), None, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                  grad_scale=scale.cpu())
    assert torch.allclose(master.cpu(), mc, atol=1e-5)
    assert torch.allclose(p.float().cpu(), mc.bfloat16().float(), atol=1e-2)
    s = sumsq(g)
    assert abs(s.item() - g.float().pow(2).sum().item()) / s.item() < 1e-3


@pytest.mark.parametrize("bwd", ["native", "flash", "recompute"])
def test_flash_attention_wide_keys_forward_and_backward(bwd, monkeypatch):
    """192-wide queries / keys with 128-wide values (latent attention expanded to per-head keys): the forward kernel
    and each gradient path behind it (the backward kernels' 192 / 128 instance, the library's flash backward on the
    saved output, per-sequence recompute) against the fp32 reference under autograd."""
    from gcore_b200.ops import _lib
    from gcore_b200.ops.attention import attn_varlen_ref, flash_attn_varlen
    monkeypatch.setenv("GCORE_WIDE_KEY_BWD", bwd)
    torch.manual_seed(3)
    lens = [5, 300, 129, 64, 1000]
    T, H = sum(lens), 6
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=DEV, dtype=torch.int32)
    q = _rand(T, H, 192, scale=0.5).requires_grad_(True)
    k = _rand(T, H, 192, scale=0.5).requires_grad_(True)
    v = _rand(T, H, 128, scale=0.5).requires_grad_(True)
    scale = 1.0 / math.sqrt(192)
    with torch.no_grad():
        out_ng = flash_attn_varlen(q, k, v, cu, cu, max(lens), max(lens), causal=True, scale=scale)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = attn_varlen_ref(qr, kr, vr, cu, cu, True, 0, None, scale)
    assert out_ng.shape == (T, H, 128)
    _close(out_ng, ref.detach())
    out = flash_attn_varlen(q, k, v, cu, cu, max(lens), max(lens), causal=True, scale=scale)
    do = _rand(T, H, 128, scale=0.5)
    out.backward(do)
    ref.backward(do.float())
    _close(q.grad, qr.grad, atol=1e-2)
    _close(k.grad, kr.grad, atol=1e-2)
    _close(v.grad, vr.grad, atol=1e-2)
    _lib.check_device_errors()


@pytest.mark.parametrize("H,C,dr,lens,head_major", [
    (20, 128, 32, [0, 5, 700, 33], False),      # ragged head group (20 = 16 + 4), an empty request, partial tiles
    (128, 512, 64, [2048, 130], True),          # the 512 + 64 geometry, several KV splits, strided operands
    (16, 256, 64, [1, 257, 64, 31, 1000], False),
])
def test_mla_paged_decode(H, C, dr, lens, head_major):
    """Latent attention decode on the paged cache vs fp32 PyTorch: as one KV split per request and with the splits
    the launch plan picks."""
    from gcore_b200.ops import _lib
    from gcore_b200.ops.attention import mla_paged_decode, mla_paged_decode_ref
    torch.manual_seed(5)
    B, bs = len(lens), 16
    max_blocks = (max(lens) + bs - 1) // bs + 1
    nblocks = B * max_blocks + 3
    cache = _rand(nblocks, bs, C + dr, scale=0.5)
    table = torch.randperm(nblocks, device=DEV)[:B * max_blocks].view(B, max_blocks).to(torch.int32)
    ctx = torch.tensor(lens, device=DEV, dtype=torch.int32)
    if head_major:   # [H, B, *] storage seen as [B, H, *]: what the head-batched projections around the kernel produce
        q_lat = _rand(H, B, C, scale=0.3).transpose(0, 1)
        q_rope = _rand(H, B, dr, scale=0.3).transpose(0, 1)
        out = torch.empty(H, B, C, device=DEV, dtype=torch.bfloat16).transpose(0, 1)
    else:
        q_lat, q_rope, out = _rand(B, H, C, scale=0.3), _rand(B, H, dr, scale=0.3), None
    scale = 1.0 / math.sqrt(C // 4 + dr)
    ref = mla_paged_decode_ref(q_lat, q_rope, cache, table, ctx, scale)
    try:
        for target in (1, 296):
            _lib.kernels().gk_mla_set_target_ctas(target)
            got = mla_paged_decode(q_lat, q_rope, cache, table, ctx, max(lens), scale, out=out)
            _close(got, ref, atol=1e-2)
            assert got[ctx == 0].abs().max().item() == 0 if (ctx == 0).any() else True
    finally:
        _lib.kernels().gk_mla_set_target_ctas(296)


@pytest.mark.parametrize("rot,window,use_sinks", [(128, 0, False), (64, 96, True)])
def test_paged_decode_with_fused_rotation_and_append(rot, window, use_sinks):
    """Rotary embedding + cache append + decode attention in one launch against the two kernels in sequence: same
    attention output, same cache rows, for one KV split per request and for several (the newest position is handled
    by the split that ends at the context length); full and partial rotary width."""
    from gcore_b200.ops import _lib
    from gcore_b200.ops.attention import kv_append_rope, paged_decode, paged_decode_append, paged_decode_append_supported
    torch.manual_seed(12)
    B, Hq, Hk, D, bs = 6, 28, 4, 128, 16
    lens = [1, 17, 300, 513, 64, 0]                    # context including the new token; the last request is inactive
    max_blocks, nblocks = 40, 320
    kc = _rand(nblocks, bs, Hk, D, scale=0.5)
    vc = _rand(nblocks, bs, Hk, D, scale=0.5)
    table = torch.randperm(nblocks, device=DEV)[:B * max_blocks].view(B, max_blocks).to(torch.int32)
    ctx = torch.tensor(lens, device=DEV, dtype=torch.int32)
    pos = (ctx - 1).clamp_min(0)
    slots = torch.where(ctx > 0, table.gather(1, (pos // bs).long()[:, None]).squeeze(1) * bs + pos % bs,
                        torch.full_like(pos, -1)).to(torch.int32)
    qkv = _rand(B, (Hq + 2 * Hk) * D, scale=0.5)
    sinks = torch.randn(Hq, device=DEV) if use_sinks else None
    assert paged_decode_append_supported(qkv, Hq, Hk, D, rot)
    # reference: the two kernels on copies
    qkv_r, kc_r, vc_r = qkv.clone(), kc.clone(), vc.clone()
    kv_append_rope(qkv_r, pos, slots, kc_r, vc_r, Hq, Hk, D, 1e6, rot)
    want = paged_decode(qkv_r.view(B, Hq + 2 * Hk, D)[:, :Hq], kc_r, vc_r, table, ctx, max(lens), window=window,
                        sinks=sinks)
    try:
        for target in (1, 444, 4000):
            _lib.kernels().gk_paged_set_target_ctas(target)
            kc_f, vc_f, qkv_f = kc.clone(), vc.clone(), qkv.clone()
            got = paged_decode_append(qkv_f, pos, slots, kc_f, vc_f, table, ctx, max(lens), Hq, Hk, D, 1e6, rot,
                                      window=window, sinks=sinks)
            _close(got[:5], want[:5], atol=2e-2)
            assert torch.equal(vc_f, vc_r)                                  # same rows appended, nothing else touched
            assert (kc_f != kc).any(-1).any(-1).flatten().sum() == 5         # one key row per active request
            _close(kc_f, kc_r, atol=1e-2)                                    # rotated keys: equal up to fp contraction
            assert torch.equal(qkv_f, qkv)                                   # the packed rows stay unrotated
    finally:
        _lib.kernels().gk_paged_set_target_ctas(444)
    _lib.check_device_errors()


@pytest.mark.parametrize("window,use_sinks", [(0, False), (96, True)])
def test_paged_decode_and_kv_append(window, use_sinks):
    from gcore_b200.ops.attention import kv_append_rope, paged_decode
    torch.manual_seed(11)
    B, Hq, Hk, D, bs = 5, 28, 4, 128, 16
    lens = [1, 17, 300, 513, 64]
    max_blocks = 40
    nblocks = 256
    kc = torch.zeros(nblocks, bs, Hk, D, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    perm = torch.randperm(nblocks, device=DEV)[:B * max_blocks].view(B, max_blocks).to(torch.int32)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    # fill the caches through the append kernel, token by token batches
    T = sum(lens)
    qkv = _rand(T, (Hq + 2 * Hk) * D, scale=0.5)
    pos = torch.cat([torch.arange(l) for l in lens]).to(DEV).to(torch.int32)
    bidx = torch.cat([torch.full((l,), i) for i, l in enumerate(lens)]).to(DEV)
    slots = (perm[bidx, (pos // bs).long()] * bs + pos % bs).to(torch.int32)
    qkv_ref = qkv.clone().cpu()
    kv_append_rope(qkv, pos, slots, kc, vc, Hq, Hk, D, 1e6)
    kv_append_rope(qkv_ref, pos.cpu(), slots.cpu(), kc_ref := kc_ref.cpu(), vc_ref := vc_ref.cpu(), Hq, Hk, D, 1e6)
    _close(qkv, qkv_ref.to(DEV))
    _close(kc, kc_ref.to(DEV))
    _close(vc, vc_ref.to(DEV))
    last = torch.tensor([sum(lens[:i + 1]) - 1 for i in range(B)], device=DEV)
    q = qkv.view(T, Hq + 2 * Hk, D)[last][:, :Hq].contiguous()
    ctx = torch.tensor(lens, device=DEV, dtype=torch.int32)
    sinks = torch.randn(Hq, device=DEV) if use_sinks else None
    out = paged_decode(q, kc, vc, perm, ctx, max(lens), window=window, sinks=sinks)
    ref = paged_decode(q.cpu(), kc.cpu(), vc.cpu(), perm.cpu(), ctx.cpu(), max(lens), window=window,
                       sinks=sinks.cpu() if use_sinks else None)
    _close(out, ref.to(DEV), atol=2e-2)
    # the split size follows the number of CTAs the launch aims for: one CTA per (request, kv head) walking the whole
    # context tile by tile (what large batches get), and two splits of several tiles each
    from gcore_b200.ops import _lib
    try:
        for target in (1, 40):
            _lib.kernels().gk_paged_set_target_ctas(target)
            out_t = paged_decode(q, kc, vc, perm, ctx, max(lens), window=window, sinks=sinks)
            _close(out_t, ref.to(DEV), atol=2e-2)
    finally:
        _lib.kernels().gk_paged_set_target_ctas(444)
    _lib.check_device_errors()


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("causal,window,use_sinks", [(True, 0, False), (True, 128, True), (False, 0, False),
                                                     (True, 256, False)])
def test_flash_attn_fwd_varlen(D, causal, window, use_sinks):
    from gcore_b200.ops.attention import attn_varlen_ref, flash_attn_varlen
    torch.manual_seed(12)
    Hq, Hk = 8, 2
    lens = [33, 1023, 3, 128, 129, 255]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=DEV, dtype=torch.int32)
    T = sum(lens)
    q, k, v = _rand(T, Hq, D), _rand(T, Hk, D), _rand(T, Hk, D)
    sinks = torch.randn(Hq, device=DEV) if use_sinks else None
    with torch.no_grad():
        out = flash_attn_varlen(q, k, v, cu, cu, max(lens), max(lens), causal=causal, window=window, sinks=sinks)
        ref = attn_varlen_ref(q, k, v, cu, cu, causal, window, sinks)
    _close(out, ref, atol=3e-2)


def test_flash_attn_prefix_k_and_packed_qkv():
    from gcore_b200.ops.attention import attn_varlen_ref, flash_attn_varlen
    torch.manual_seed(13)
    Hq, Hk, D = 4, 4, 128
    lq, lk = [5, 130], [200, 641]
    cu_q = torch.tensor([0, 5, 135], device=DEV, dtype=torch.int32)
    cu_k = torch.tensor([0, 200, 841], device=DEV, dtype=torch.int32)
    q = _rand(sum(lq), Hq, D)
    kv = _rand(sum(lk), 2 * Hk * D)
    k = kv.view(-1, 2 * Hk, D)[:, :Hk]
    v = kv.view(-1, 2 * Hk, D)[:, Hk:]
    with torch.no_grad():
        out = flash_attn_varlen(q, k, v, cu_q, cu_k, max(lq), max(lk), causal=True)
        ref = attn_varlen_ref(q, k, v, cu_q, cu_k, True)
    _close(out, ref, atol=3e-2)


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("causal,window,use_sinks", [(True, 0, False), (True, 128, True), (False, 0, False)])
def test_flash_attn_bwd_varlen(D, causal, window, use_sinks):
    from gcore_b200.ops.attention import attn_varlen_ref, flash_attn_varlen
    torch.manual_seed(14)
    Hq, Hk = 8, 2
    lens = [33, 700, 3, 128, 129, 255]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=DEV, dtype=torch.int32)
    T = sum(lens)
    q, k, v = [_rand(T, h, D).requires_grad_(True) for h in (Hq, Hk, Hk)]
    sinks = torch.randn(Hq, device=DEV).requires_grad_(True) if use_sinks else None
    out = flash_attn_varlen(q, k, v, cu, cu, max(lens), max(lens), causal=causal, window=window, sinks=sinks)
    go = _rand(T, Hq, D)
    out.backward(go)
    qf, kf, vf = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    sf = sinks.detach().clone().requires_grad_(True) if use_sinks else None
    ref = attn_varlen_ref(qf, kf, vf, cu, cu, causal, window, sf)
    ref.backward(go.float())
    _close(q.grad, qf.grad, rtol=3e-2, atol=3e-2)
    _close(k.grad, kf.grad, rtol=3e-2, atol=3e-2)
    _close(v.grad, vf.grad, rtol=3e-2, atol=3e-2)
    if use_sinks:
        _close(sinks.grad, sf.grad, rtol=3e-2, atol=3e-2)


def test_flash_attn_packed_qkv_bwd_matches_unpacked():
    from gcore_b200.ops.attention import attn_varlen_ref, flash_attn_qkvpacked
    torch.manual_seed(15)
    hq, hk, D = 4, 2, 128
    lens = [200, 56]
    cu = torch.tensor([0, 200, 256], device=DEV, dtype=torch.int32)
    qkv = _rand(256, hq + 2 * hk, D).requires_grad_(True)
    out = flash_attn_qkvpacked(qkv, hq, hk, cu, 200)
    go = _rand(256, hq, D)
    out.backward(go)
    x = qkv.detach().float().requires_grad_(True)
    ref = attn_varlen_ref(x[:, :hq], x[:, hq:hq + hk], x[:, hq + hk:], cu, cu, True)
    ref.backward(go.float())
    _close(qkv.grad, x.grad, rtol=3e-2, atol=3e-2)


def test_quantisers_match_eager_definitions():
    from gcore_b200.ops import quant
    torch.manual_seed(16)
    x = _rand(257, 512, scale=3.0)
    for pow2 in (False, True):
        q, s = quant.quant_act_1x128(x, pow2)
        qr, sr = quant.act_quant_1x128_ref(x, pow2)
        assert torch.allclose(s, sr, rtol=1e-6)
        assert (q.float() - qr.float()).abs().max() <= 32  # at most one e4m3 code step at the largest magnitude
        assert (quant.dequant_1x128(q, s) - x.float()).abs().max() / x.float().abs().max() < 0.07
    w = _rand(300, 640, scale=0.1)
    q, s = quant.quant_weight_128x128(w)
    qr, sr = quant.weight_quant_128x128_ref(w)
    assert torch.allclose(s, sr, rtol=1e-6) and q.shape == (300, 640)
    assert (quant.dequant_128x128(q, s) - w.float()).abs().max() / w.float().abs().max() < 0.07
    y = x.clone()
    quant.qat_fp8_(y, "1x128", pow2=True)
    qr, sr = quant.act_quant_1x128_ref(x, True)
    _close(y, quant.dequant_1x128(qr, sr), rtol=2e-2, atol=2e-2)
    packed, e8, s32 = quant.quant_fp4_1x32(x)
    codes, sr, dq = quant.fp4_quant_1x32_ref(x)
    assert torch.equal(s32, sr)
    assert torch.equal(packed, (codes[0::2] | (codes[1::2] << 4)))


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 520, 1024), (1024, 2048, 7168)])
def test_gemm_fp8_blockscaled(M, N, K):
    from gcore_b200.ops import quant
    torch.manual_seed(17)
    a, b = _rand(M, K, scale=1.0), _rand(N, K, scale=0.05)
    aq, as_ = quant.quant_act_1x128(a)
    bq, bs = quant.quant_weight_128x128(b)
    ref = quant.dequant_1x128(aq, as_) @ quant.dequant_128x128(bq, bs).t()
    out = quant.gemm_fp8_blockscaled(aq, as_, bq, bs)
    _close(out, ref, rtol=1e-2, atol=1e-2)
    full = a.float() @ b.float().t()
    assert (out.float() - full).abs().max() / full.abs().max() < 0.1


@pytest.mark.parametrize("G,N,K,rows", [(4, 256, 512, [128, 0, 384, 256]), (8, 4096, 7168, [256, 128, 0, 0, 512, 128, 128, 384]),
                                        (3, 7168, 2048, [128, 128, 128])])
def test_gemm_fp8_grouped_matches_dequantised_reference(G, N, K, rows):
    """Ragged-M grouped block-fp8 GEMM (experts): every segment against its own expert's dequantised weight; an
    empty expert, spare capacity behind the last segment."""
    from gcore_b200.ops import _lib, quant
    torch.manual_seed(31)
    offs = [0]
    for r in rows:
        offs.append(offs[-1] + r)
    cap = offs[-1] + 256                                     # spare rows beyond the last group stay zero
    a = _rand(cap, K, scale=1.0)
    a[offs[-1]:] = 0
    w = _rand(G, N, K, scale=0.05)
    aq, as_ = quant.quant_act_1x128(a)
    bq, bs = quant.quant_weight_128x128(w.reshape(G * N, K).contiguous())
    offsets = torch.tensor(offs, dtype=torch.int32, device=DEV)
    out = quant.gemm_fp8_grouped(aq, as_, bq, bs, offsets, G)
    _lib.check_device_errors()
    a_dq = quant.dequant_1x128(aq, as_).float()
    w_dq = quant.dequant_128x128(bq, bs)[:G * N, :K].float().view(G, N, K)
    for g in range(G):
        if rows[g]:
            ref = a_dq[offs[g]:offs[g + 1]] @ w_dq[g].t()
            _close(out[offs[g]:offs[g + 1]], ref, rtol=1e-2, atol=1e-2)
    assert not out[offs[-1]:].any()


def test_grouped_fp8_expert_projection_forward_backward():
    from gcore_b200.models.moe import grouped_linear
    torch.manual_seed(32)
    G, N, K = 4, 256, 384
    offs = torch.tensor([0, 128, 128, 384, 512], dtype=torch.int32, device=DEV)
    x = _rand(512, K, scale=1.0).requires_grad_(True)
    w = _rand(G, N, K, scale=0.05).requires_grad_(True)
    y = grouped_linear(x, w, offs, "fp8", {})
    x2, w2 = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    y2 = grouped_linear(x2, w2, offs)
    assert (y.float() - y2.float()).abs().max() / y2.float().abs().max() < 0.08
    g = torch.randn_like(y)
    y.backward(g)
    y2.backward(g)
    assert (x.grad.float() - x2.grad.float()).abs().max() / x2.grad.float().abs().max() < 0.08
    _close(w.grad, w2.grad, rtol=2e-2, atol=2e-2)            # wgrad runs in bf16 on the same operands


def test_fp8_data_and_weight_gradient_products():
    """dX = dY W and dW = dY^T X on the block-fp8 GEMM against the products of the same quantised operands in fp32
    (dense and grouped data gradient), and against the unquantised gradients to fp8 accuracy."""
    from gcore_b200.ops import _lib, quant
    torch.manual_seed(33)
    M, N, K = 300, 384, 512
    dy, x, w = _rand(M, N, scale=1.0), _rand(M, K, scale=1.0), _rand(N, K, scale=0.05)
    q, s = quant.quant_weight_128x128(w)
    cache = {"ver": 1, "q": q, "s": s}
    dx = quant.fp8_dgrad(dy, cache, torch.bfloat16)
    gq, gs = quant.quant_act_1x128(dy)
    ref = quant.dequant_1x128(gq, gs).float() @ quant.dequant_128x128(q, s)[:N, :K].float()
    _close(dx, ref, rtol=1e-2, atol=1e-2)
    assert (dx.float() - dy.float() @ w.float()).abs().max() / (dy.float() @ w.float()).abs().max() < 0.08
    dw = quant.fp8_wgrad(dy, x)
    full = dy.float().t() @ x.float()
    assert dw.dtype == torch.float32 and dw.shape == (N, K)
    assert (dw - full).abs().max() / full.abs().max() < 0.08
    # grouped: experts 0 and 2 have rows, expert 1 none
    G, offs = 3, torch.tensor([0, 128, 128, 384], dtype=torch.int32, device=DEV)
    wg = _rand(G, 256, K, scale=0.05)
    qg, sg = quant.quant_weight_128x128(wg.reshape(G * 256, K).contiguous())
    dyg = _rand(384, 256, scale=1.0)
    dxg = quant.fp8_dgrad(dyg, {"ver": 1, "q": qg, "s": sg}, torch.bfloat16, offsets=offs, groups=G)
    gq, gs = quant.quant_act_1x128(dyg)
    wdq = quant.dequant_128x128(qg, sg)[:G * 256, :K].float().view(G, 256, K)
    a = quant.dequant_1x128(gq, gs).float()
    _close(dxg[:128], a[:128] @ wdq[0], rtol=1e-2, atol=1e-2)
    _close(dxg[128:384], a[128:384] @ wdq[2], rtol=1e-2, atol=1e-2)
    _lib.check_device_errors()


@pytest.mark.parametrize("T,N,K,bias,fp32", [(1, 512, 256, False, False), (8, 4608, 3584, True, False),
                                              (64, 3584, 18944, False, False), (100, 1000, 1792, True, True),
                                              (128, 2304, 3584, True, False), (128, 3584, 9472, False, True),
                                              (17, 256, 128, False, False)])
def test_skinny_cluster_splitk_gemm(T, N, K, bias, fp32):
    from gcore_b200.ops import gemm as G
    torch.manual_seed(18)
    x, w = _rand(T, K, scale=0.5), _rand(N, K, scale=0.05)
    b = _rand(N) if bias else None
    assert G._SKINNY[0]
    # call the cluster kernel directly: linear_forward only routes some shapes to it
    tiles, kb = (N + 127) // 128, (K + 63) // 64
    ks, tpad = G._skinny_plan(T, tiles, kb, K)
    y = torch.empty(T, N, dtype=torch.float32 if fp32 else torch.bfloat16, device="cuda")
    from gcore_b200.ops import _lib
    rc = _lib.kernels().gk_gemm_skinny(_lib.ptr(w), w.stride(0), _lib.ptr(x), x.stride(0), _lib.ptr(y), y.stride(0),
                                       int(fp32), _lib.ptr(b), 0, T, tpad, N, K, ks,
                                       _lib.ptr(_lib.err_flag(x.device)), _lib.stream_ptr())
    assert rc == 0
    _lib.check_device_errors()
    ref = x.float() @ w.float().t() + (b.float() if bias else 0.0)
    _close(y, ref, rtol=1e-2, atol=1e-2 if not fp32 else 2e-3)
    # same numbers as the general kernel's split-K path
    G._SKINNY[0] = False
    try:
        y2 = G.linear_forward(x, w, b, out_dtype=torch.float32 if fp32 else None)
    finally:
        G._SKINNY[0] = True
    _close(y, y2.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("bn,a_mn,b_mn", [(224, False, False), (224, True, False), (192, False, False),
                                           (192, False, True), (192, True, True)])
def test_gemm_intermediate_tile_widths(bn, a_mn, b_mn):
    from gcore_b200.ops.gemm import gemm
    torch.manual_seed(19)
    M, N, K = 384, 1000, 512
    a = _rand(K, M) if a_mn else _rand(M, K)
    b = _rand(K, N, scale=0.05) if b_mn else _rand(N, K, scale=0.05)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    _close(out, ref, rtol=1e-2, atol=1e-2)
    acc = torch.ones(M, N, dtype=torch.float32, device="cuda")
    gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn, out=acc, accumulate=True)
    _close(acc, ref + 1.0, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(1024, 768, 512), (1300, 1000, 320), (2048, 512, 4096)])
def test_gemm_wide_tiles(M, N, K, a_mn, b_mn):
    from gcore_b200.ops import _lib
    from gcore_b200.ops import gemm as G
    torch.manual_seed(20)
    Np = (N + 7) // 8 * 8
    a = _rand(K, (M + 7) // 8 * 8)[:, :M] if a_mn else _rand(M, K)
    b = _rand(K, Np, scale=0.05)[:, :N] if b_mn else _rand(N, K, scale=0.05)
    bias = _rand(N)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    lib = _lib.kernels()

    ws, cnt = G._scratch(a.device, 16 << 20, 4096)

    def run(out, accumulate, bias_t, alpha):
        rc = lib.gk_gemm_wide(_lib.ptr(a), a.stride(0), a.shape[0], int(a_mn), _lib.ptr(b), b.stride(0), b.shape[0],
                              int(b_mn), _lib.ptr(out), out.stride(0), int(out.dtype == torch.float32), int(accumulate),
                              _lib.ptr(bias_t), 0, alpha, M, N, K, _lib.ptr(ws), ws.numel(), _lib.ptr(cnt), cnt.numel(),
                              _lib.ptr(_lib.err_flag(a.device)), _lib.stream_ptr())
        assert rc == 0
        _lib.check_device_errors()

    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    run(out, False, bias, 1.0)
    _close(out, ref + bias.float(), rtol=1e-2, atol=1e-2 * max(1.0, K / 512) ** 0.5)
    acc = torch.full((M, N), 2.0, dtype=torch.float32, device="cuda")
    run(acc, True, None, 0.5)
    _close(acc, 0.5 * ref + 2.0, rtol=1e-2, atol=1e-2 * max(1.0, K / 512) ** 0.5)
    # the dispatcher sends large well-quantised problems here and keeps the rest on the 128-row kernel
    assert G._use_wide(8192, 37888, 3584) and not G._use_wide(512, 4096, 4096)


@pytest.mark.parametrize("M,N,K", [(2048, 2304, 512), (4096, 1024, 1088), (2000, 2100, 520), (8192, 4608, 3584)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_cta_pair_kernel(M, N, K, a_mn, b_mn):
    """256 x 256 tiles on CTA pairs (tcgen05.mma.cta_group::2): forward / dgrad / wgrad layouts, ragged edges, bias,
    fp32 accumulation into an existing buffer; bitwise repeatable."""
    from gcore_b200.ops import gemm as G
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a 16-byte aligned leading dimension")
    was = G.TWO_CTA["enabled"]
    G.TWO_CTA["enabled"] = True                 # opt-in kernel: switched on for this test
    try:
        _check_cta_pair(G, M, N, K, a_mn, b_mn)
    finally:
        G.TWO_CTA["enabled"] = was


def _check_cta_pair(G, M, N, K, a_mn, b_mn):
    assert G._use_two_cta(M, N, K)
    torch.manual_seed(3)
    A, B = _rand(M, K, scale=0.5), _rand(N, K, scale=0.5)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    ref = A.float() @ B.float().t()
    before = G.LAUNCHES["gemm"]
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    assert G.LAUNCHES["gemm"] == before + 1
    _close(out, ref, rtol=1e-2, atol=1e-2 * math.sqrt(K))
    assert torch.equal(out, G.gemm(a, b, a_mn=a_mn, b_mn=b_mn))
    bias = _rand(N)
    C0 = torch.randn(M, N, device=DEV, dtype=torch.float32)
    acc = C0.clone()
    G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=acc, bias=bias, alpha=0.5, accumulate=True)
    _close(acc, C0 + 0.5 * ref + bias.float()[None], rtol=2e-3, atol=2e-3 * math.sqrt(K))
    # the one-CTA kernels agree (same products, different tiling)
    G.TWO_CTA["enabled"] = False
    try:
        one = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    finally:
        G.TWO_CTA["enabled"] = True
    two = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    _close(two, one, rtol=1e-4, atol=1e-3)


def test_dsv4_sparse_mqa_and_indexer_kernels():
    """Gather attention (shared key / value rows, sinks, -1 entries, rows without any entry), its backward, the
    indexer scores with per-row bounds and the gradient through selected entries."""
    from gcore_b200.ops import dsv4 as K4
    torch.manual_seed(5)
    S, T, H, D, K = 200, 333, 6, 128, 40
    q = _rand(S, H, D, scale=0.5).requires_grad_(True)
    kv = _rand(T, D, scale=0.5).requires_grad_(True)
    sinks = torch.randn(H, device=DEV).requires_grad_(True)
    idx = torch.randint(0, T, (S, K), device=DEV, dtype=torch.int32)
    idx[torch.rand(S, K, device=DEV) < 0.3] = -1
    idx[7] = -1
    out = K4.sparse_mqa(q, kv, sinks, idx, D ** -0.5)
    do = _rand(S, H, D)
    out.backward(do)
    qr, kr, sr = (t.detach().float().requires_grad_(True) for t in (q, kv, sinks))
    ref, _ = K4.sparse_mqa_ref(qr, kr, sr, idx, D ** -0.5)
    ref.backward(do.float())
    _close(out, ref, rtol=2e-2, atol=1e-2)
    _close(q.grad, qr.grad, rtol=3e-2, atol=2e-2)
    _close(kv.grad, kr.grad, rtol=3e-2, atol=3e-2)
    _close(sinks.grad, sr.grad, rtol=3e-2, atol=3e-2)
    assert (out[7] == 0).all()

    Hi, Di = 8, 64
    qi, ki = _rand(S, Hi, Di, scale=0.5), _rand(T, Di, scale=0.5)
    w = torch.rand(S, Hi, device=DEV)
    ks = torch.randint(0, T // 2, (S,), device=DEV, dtype=torch.int32)
    ke = ks + torch.randint(0, T // 2, (S,), device=DEV, dtype=torch.int32)
    sc = K4.indexer_scores(qi, ki, w, ks, ke, Di ** -0.5)
    rf = K4.indexer_scores_ref(qi, ki, w, ks, ke, Di ** -0.5)
    assert torch.equal(torch.isinf(sc), torch.isinf(rf))
    fin = torch.isfinite(rf)
    _close(sc[fin], rf[fin], rtol=1e-2, atol=1e-2)
    sel_idx = torch.randint(-1, T, (S, 12), device=DEV, dtype=torch.int32)
    qg, kg, wg = qi.clone().requires_grad_(True), ki.clone().requires_grad_(True), w.clone().requires_grad_(True)
    sel = K4.indexer_selected_scores(qg, kg, wg, sel_idx, Di ** -0.5)
    gs = torch.randn_like(sel)
    sel.backward(gs)
    q2, k2, w2 = (t.detach().float().requires_grad_(True) for t in (qi, ki, w))
    K4._selected_ref(q2, k2, w2, sel_idx, Di ** -0.5).backward(gs)
    _close(qg.grad, q2.grad, rtol=3e-2, atol=2e-2)
    _close(kg.grad, k2.grad, rtol=3e-2, atol=3e-2)
    _close(wg.grad, w2.grad, rtol=3e-2, atol=2e-2)


@pytest.mark.parametrize("n", [16, 128, 512, 2048])
def test_hadamard_rotation(n):
    from gcore_b200.ops import dsv4 as K4
    torch.manual_seed(6)
    x = _rand(37, 3, n)
    y = K4.rotate_activation(x)
    _close(y, K4.hadamard_ref(x.float()), rtol=1e-2, atol=1e-2)
    _close(K4.rotate_activation(y), x, rtol=2e-2, atol=2e-2)


def test_dsv4_model_step_on_gpu():
    from gcore_b200.models.deepseek_v4 import DSV4Config, DeepseekV4Model, causal_lm_loss
    torch.manual_seed(0)
    cfg = DSV4Config(dtype="bfloat16", head_dim=64, index_head_dim=32)
    m = DeepseekV4Model(cfg, device=DEV)
    data = torch.randint(0, 64, (160,), device=DEV)
    from gcore_b200.ops import dsv4 as K4
    before = K4.LAUNCHES["dsv4"]
    loss = causal_lm_loss(m, data, [0, 64, 160])
    loss.backward()
    assert K4.LAUNCHES["dsv4"] > before and torch.isfinite(loss)
    assert m.layers[1].self_attn.compressor.compress.kv_proj.weight.grad.abs().sum() > 0


def test_rope_table_kernel_matches_reference():
    from gcore_b200.ops import fused
    torch.manual_seed(7)
    T, Hh, D = 300, 5, 128
    x = _rand(T, Hh, D)
    pos3 = torch.randint(0, 500, (T, 3), device=DEV)
    tab = fused.mrope_tables(pos3, 1e6, D, (24, 20, 20), True)
    y = fused.rope_inplace(x.clone(), tab, 1e6, D, False, False)
    _close(y, fused.rope_ref(x.float(), tab, 1e6, D), rtol=1e-2, atol=1e-2)
    back = fused.rope_inplace(y.clone(), tab, 1e6, D, False, True)
    _close(back, x, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("T,K,E,ep", [(64, 8, 128, 8), (1, 2, 8, 2), (500, 6, 256, 4), (1024, 8, 64, 2)])
def test_expert_parallel_local_plan_kernel_matches_sort_and_histogram(T, K, E, ep):
    """The single-kernel routing bookkeeping of small batches: per-expert counts and, for every (token, k) pair, its
    rank among the pairs of the same expert in input order = what a stable sort by expert gives."""
    from gcore_b200.ops import _lib
    torch.manual_seed(40)
    flat = torch.randint(0, E, (T * K,), device=DEV, dtype=torch.int64)
    n, El = T * K, E // ep
    idx32 = torch.empty(n, dtype=torch.int32, device=DEV)
    pos = torch.full((n,), -1, dtype=torch.int32, device=DEV)
    cnt = torch.full((E,), -1, dtype=torch.int32, device=DEV)
    offsets = torch.full((El + 1,), 7, dtype=torch.int32, device=DEV)
    tot = torch.full((El,), 7, dtype=torch.int32, device=DEV)
    _lib.check(_lib.kernels().gk_ep_local_plan(_lib.ptr(flat), n, E, El, _lib.ptr(idx32), _lib.ptr(pos), _lib.ptr(cnt),
                                               _lib.ptr(offsets), _lib.ptr(tot), _lib.stream_ptr()), "local_plan")
    want_cnt = torch.bincount(flat, minlength=E)
    order = torch.argsort(flat, stable=True)
    starts = want_cnt.cumsum(0) - want_cnt
    want_pos = torch.empty_like(flat)
    want_pos[order] = torch.arange(n, device=DEV) - starts[flat[order]]
    assert torch.equal(cnt.long(), want_cnt) and torch.equal(pos.long(), want_pos) and torch.equal(idx32.long(), flat)
    assert not offsets.any() and not tot.any()


def test_swiglu_shapes_and_row_bound():
    """SwiGLU forward / backward on shapes whose row length does not divide the grid stride (the index carries of the
    division-free iteration), and the forward that stops at a device-side row count."""
    from gcore_b200.ops import fused
    torch.manual_seed(41)
    for T, F in ((9216, 1536), (64, 18944), (777, 104), (3, 8)):
        x = _rand(T, 2 * F, scale=1.5).requires_grad_(True)
        y = fused.swiglu(x)
        xr = x.detach().float().requires_grad_(True)
        g, u = xr.chunk(2, -1)
        ref = torch.nn.functional.silu(g) * u
        _close(y, ref.detach())
        dy = _rand(T, F)
        y.backward(dy)
        ref.backward(dy.float())
        _close(x.grad, xr.grad)
    x = _rand(1024, 512, scale=1.5)
    n = torch.tensor([300], dtype=torch.int32, device=DEV)
    with torch.no_grad():
        y = fused.swiglu(x, n_rows=n)
    g, u = x.float().chunk(2, -1)
    _close(y[:300], (torch.nn.functional.silu(g) * u)[:300])


def test_qk_headnorm_in_place():
    """Per-head RMSNorm of the q and k heads of packed rows in one launch = the two norms over reshaped copies; the
    value heads and the row padding stay untouched."""
    from gcore_b200.ops import fused
    torch.manual_seed(42)
    T, Hq, Hk, D = 70, 32, 4, 128
    buf = _rand(T, (Hq + 2 * Hk) * D + 64, scale=2.0)          # rows with a pitch larger than their width
    qkv = buf[:, :(Hq + 2 * Hk) * D]
    wq, wk = _rand(D, scale=1.0) + 1.0, _rand(D, scale=1.0) + 1.0
    want = qkv.clone().float().view(T, Hq + 2 * Hk, D)
    for sl, w in ((slice(0, Hq), wq), (slice(Hq, Hq + Hk), wk)):
        x = want[:, sl]
        want[:, sl] = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * w.float()
    before = buf.clone()
    fused.qk_headnorm_(qkv, wq, wk, Hq, Hk, D, 1e-6)
    _close(qkv.reshape(T, Hq + 2 * Hk, D), want)
    assert torch.equal(qkv.reshape(T, Hq + 2 * Hk, D)[:, Hq + Hk:], before[:, :(Hq + 2 * Hk) * D].view(T, -1, D)[:, Hq + Hk:])
    assert torch.equal(buf[:, (Hq + 2 * Hk) * D:], before[:, (Hq + 2 * Hk) * D:])
