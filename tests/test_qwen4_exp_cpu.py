"""Qwen4-exp-class decoder on CPU: component semantics against independent restatements, packed-sequence isolation,
and a short training run."""
import math

import torch
import torch.nn.functional as F

from gcore_b200.models.qwen4_exp import (FULL, LINEAR, GatedDeltaNet, NGramEmbedding, Qwen4ExpConfig, Qwen4ExpModel,
                                         gated_delta_rule, select_qsa_membership)


def _cfg(**kw):
    return Qwen4ExpConfig(**kw)


def test_gated_delta_rule_matches_closed_form_first_steps():
    torch.manual_seed(0)
    T, H, Dk, Dv = 5, 2, 4, 3
    q, k, v = torch.randn(T, H, Dk), torch.randn(T, H, Dk), torch.randn(T, H, Dv)
    g, beta = -torch.rand(T, H), torch.rand(T, H)
    o = gated_delta_rule(q, k, v, g, beta, [0, T])
    qn, kn = F.normalize(q, dim=-1) * Dk ** -0.5, F.normalize(k, dim=-1)
    # step 0: S = k0 (beta0 v0)^T, o0 = (q0 . k0) beta0 v0
    o0 = (qn[0] * kn[0]).sum(-1, keepdim=True) * beta[0][:, None] * v[0]
    assert torch.allclose(o[0], o0, atol=1e-5)
    # step 1 by hand
    S0 = kn[0][:, :, None] * (beta[0][:, None] * v[0])[:, None, :]
    S = S0 * g[1].exp()[:, None, None]
    delta = (v[1] - torch.einsum("hkv,hk->hv", S, kn[1])) * beta[1][:, None]
    S = S + kn[1][:, :, None] * delta[:, None, :]
    assert torch.allclose(o[1], torch.einsum("hkv,hk->hv", S, qn[1]), atol=1e-5)
    # the state restarts at a sequence start
    o2 = gated_delta_rule(q, k, v, g, beta, [0, 2, T])
    assert torch.allclose(o2[:2], o[:2], atol=1e-6)
    assert torch.allclose(o2[2:], gated_delta_rule(q[2:], k[2:], v[2:], g[2:], beta[2:], [0, 3]), atol=1e-6)


def test_qsa_membership_tail_and_topk():
    torch.manual_seed(1)
    cfg = _cfg()
    n, ratio, topk = 19, 4, 2
    iq, raw = torch.randn(n, 2, 16), torch.randn(n, 16)
    ident = lambda x: x
    m = select_qsa_membership(iq, raw, torch.arange(n), [0, n], ident, cfg.rope_theta, 0, ratio, topk)
    for p in range(n):
        vis = (p + 1) // ratio
        row = m[p]
        assert not row[p + 1:].any()                                   # causal
        assert row[vis * ratio:p + 1].all()                            # incomplete tail always attended
        blocks = row[:vis * ratio].view(vis, ratio)
        assert ((blocks.all(-1)) | (~blocks.any(-1))).all()            # whole blocks only
        assert int(blocks.all(-1).sum()) == min(topk, vis)
        if vis > topk:                                                 # the chosen blocks have the best scores
            pooled = raw[:vis * ratio].view(vis, ratio, -1).mean(1)
            sc = torch.relu(torch.einsum("hd,nd->hn", iq[p], pooled)).sum(0)
            chosen = blocks.all(-1)
            assert sc[chosen].min() >= sc[~chosen].max() - 1e-6
    # packed sequences never see one another
    m2 = select_qsa_membership(iq, raw, torch.arange(n), [0, 7, n], ident, cfg.rope_theta, 0, ratio, topk)
    assert not m2[7:, :7].any() and not m2[:7, 7:].any()
    assert torch.equal(m2[:7, :7], select_qsa_membership(iq[:7], raw[:7], torch.arange(7), [0, 7], ident,
                                                         cfg.rope_theta, 0, ratio, topk))


def test_ngram_embedding_respects_boundaries_and_eos():
    cfg = _cfg()
    emb = NGramEmbedding(cfg, cfg.ple_embed_dim, 0)
    ids = torch.tensor([5, 6, 7, 2, 8, 9, 5, 6, 7])
    cu = [0, 6, 9]
    s1 = emb._shifted(ids, cu, 1)
    s2 = emb._shifted(ids, cu, 2)
    eos = cfg.eos_token_id
    assert s1.tolist() == [eos, 5, 6, 7, eos, 8, eos, 5, 6]           # position 4 follows an eos; 6 starts a sequence
    assert s2.tolist() == [eos, eos, 5, 6, eos, eos, eos, eos, 5]
    out = emb(ids, cu)
    assert out.shape == (9, cfg.ple_embed_dim)
    # the same trigram (5, 6, 7) at the same in-sequence offset hashes to the same rows
    assert torch.equal(out[2], out[8])
    # all multipliers odd, table sizes distinct primes
    assert all(int(m) % 2 == 1 for m in emb.mult)
    assert len(set(emb.sizes.tolist())) == emb.sizes.numel()
    emb2 = NGramEmbedding(cfg, cfg.ple_embed_dim, 1)
    assert not set(emb.sizes.tolist()) & set(emb2.sizes.tolist())


def test_delta_net_layer_is_causal_and_packed():
    torch.manual_seed(2)
    cfg = _cfg()
    net = GatedDeltaNet(cfg)
    x = torch.randn(12, cfg.hidden_size)
    y = net(x, [0, 12])
    x2 = x.clone()
    x2[8:] += 1.0
    assert torch.allclose(net(x2, [0, 12])[:8], y[:8], atol=1e-6)     # later tokens do not reach back
    ya = net(x, [0, 5, 12])
    assert torch.allclose(ya[:5], net(x[:5], [0, 5]), atol=1e-6)
    assert torch.allclose(ya[5:], net(x[5:], [0, 7]), atol=1e-6)


def test_model_packed_equals_separate_and_trains():
    torch.manual_seed(3)
    cfg = _cfg(indexer_budget=8)
    model = Qwen4ExpModel(cfg)
    assert [l.kind for l in model.layers] == [LINEAR, LINEAR, LINEAR, FULL]
    assert model.layers[0].ple is not None and model.layers[1].ple is None and model.layers[2].ple is not None
    ids = torch.randint(3, cfg.vocab_size, (40,))
    cu = [0, 17, 40]
    with torch.no_grad():
        h = model(ids, cu)
        ha = model(ids[:17], [0, 17])
        hb = model(ids[17:], [0, 23])
    assert torch.allclose(h[:17], ha, atol=2e-5) and torch.allclose(h[17:], hb, atol=2e-5)

    # memorise a short stream: next-token loss falls well below the uniform baseline
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    first = None
    for step in range(30):
        h = model(ids, cu)
        logits = model.logits(h).float()
        tgt = torch.roll(ids, -1)
        keep = torch.ones(40, dtype=torch.bool)
        keep[16] = keep[39] = False
        loss = F.cross_entropy(logits[keep], tgt[keep]) + 0.01 * model.load_balancing_loss()
        opt.zero_grad()
        loss.backward()
        if step == 0:
            first = float(loss.detach())
            # the indexer only picks discrete block ids (no auxiliary loss, no straight-through path): it stays frozen
            missing = [n for n, p in model.named_parameters() if (p.grad is None or not torch.isfinite(p.grad).all())
                       and not any(t in n for t in ("index_qk_proj", "iq_norm", "ik_norm"))]
            assert not missing, missing
        opt.step()
    assert first > 0.9 * math.log(cfg.vocab_size)
    assert float(loss) < 0.5 * first
