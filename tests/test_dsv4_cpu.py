"""DeepSeek-V4-class decoder on CPU: op definitions against direct computations, layout helpers, the three attention
variants, hyper-connection invariants, hash / top-k routing, and a short training run."""
import math

import torch

from gcore_b200.models.deepseek_v4 import (CSA, HCA, SLIDING, DSV4Config, DeepseekV4Model, HyperConnection,
                                           _window_layout, causal_lm_loss, sliding_window_index)
from gcore_b200.ops import dsv4 as K4


def test_op_references():
    g = torch.Generator().manual_seed(0)
    S, T, H, D, K = 5, 7, 3, 8, 4
    q, kv = torch.randn(S, H, D, generator=g), torch.randn(T, D, generator=g)
    sinks = torch.randn(H, generator=g)
    idx = torch.tensor([[0, 1, -1, -1], [2, 3, 4, -1], [6, 5, 0, 1], [-1, -1, -1, -1], [3, -1, 2, -1]])
    out, lse = K4.sparse_mqa_ref(q, kv, sinks, idx, 0.3)
    for t in range(S):
        rows = [int(i) for i in idx[t] if i >= 0]
        for h in range(H):
            s = torch.tensor([float(q[t, h] @ kv[r]) * 0.3 for r in rows] + [float(sinks[h])])
            p = s.softmax(0)[:-1]
            want = sum(p[j] * kv[r] for j, r in enumerate(rows)) if rows else torch.zeros(D)
            assert torch.allclose(out[t, h], want, atol=1e-5)
    w = torch.rand(S, H, generator=g)
    ks, ke = torch.tensor([0, 1, 0, 3, 2]), torch.tensor([3, 4, 7, 3, 6])
    sc = K4.indexer_scores_ref(q, kv, w, ks, ke, 0.5)
    assert torch.isinf(sc[3]).all() and torch.isinf(sc[1, 0]) and torch.isfinite(sc[1, 1:4]).all()
    assert abs(float(sc[2, 5]) - 0.5 * sum(float(w[2, h]) * max(float(q[2, h] @ kv[5]), 0.0) for h in range(H))) < 1e-5
    sel = K4.indexer_selected_scores(q, kv, w, torch.tensor([[1, -1]] * S), 0.5)
    assert torch.allclose(sel[:, 0], K4.indexer_scores_ref(q, kv, w, torch.zeros(S).long(), torch.full((S,), T), 0.5)[:, 1])
    assert (sel[:, 1] == 0).all()
    x = torch.randn(3, 16, generator=g)
    y = K4.hadamard_ref(x)
    assert torch.allclose(K4.hadamard_ref(y), x, atol=1e-5)                 # involution
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)        # orthogonal
    assert torch.allclose(y[:, 0], x.sum(-1) / 4, atol=1e-5)


def test_layout_helpers():
    starts, seg, pos, first = _window_layout([0, 10, 13, 21], 4)
    assert starts == [0, 4, 13, 17] and seg == [0, 0, 2, 2] and pos == [0, 4, 0, 4] and first == [0, 2, 2, 4]
    w = sliding_window_index([0, 3, 6], 2, "cpu")
    assert w.tolist() == [[0, -1], [1, 0], [2, 1], [3, -1], [4, 3], [5, 4]]


def test_hyper_connection_mixing_is_doubly_stochastic_and_starts_as_identity_residual():
    cfg = DSV4Config(hc_sinkhorn_iters=8)
    hc = HyperConnection(cfg)
    streams = torch.randn(6, cfg.hc_mult, cfg.hidden_size)
    write, mix, collapsed = hc(streams)
    assert torch.allclose(mix.sum(-1), torch.ones(6, cfg.hc_mult), atol=1e-3)
    assert torch.allclose(mix.sum(-2), torch.ones(6, cfg.hc_mult), atol=1e-3)
    assert torch.allclose(collapsed, streams.mean(1), atol=1e-6) and torch.allclose(write, torch.ones_like(write))
    out = HyperConnection.combine(streams, torch.zeros(6, cfg.hidden_size), write, mix)
    assert (out - streams).abs().max() < 0.1                                  # near-identity residual at init


def _model(**kw):
    torch.manual_seed(0)
    return DeepseekV4Model(DSV4Config(**kw))


def test_sequences_of_a_packed_stream_do_not_see_each_other_and_causality_holds():
    m = _model()
    g = torch.Generator().manual_seed(1)
    a, b = torch.randint(0, 1024, (37,), generator=g), torch.randint(0, 1024, (22,), generator=g)
    both = m(torch.cat([a, b]), [0, 37, 59])
    assert torch.allclose(both[:37], m(a, [0, 37]), atol=1e-5)
    assert torch.allclose(both[37:], m(b, [0, 22]), atol=1e-5)
    a2 = a.clone()
    a2[30] = (a2[30] + 1) % 1024
    h2 = m(a2, [0, 37])
    assert torch.allclose(h2[:30], both[:30], atol=1e-5) and not torch.allclose(h2[30:], both[30:37], atol=1e-4)


def test_compressed_history_reaches_beyond_the_sliding_window():
    """A token far outside the window changes later outputs only through the compressed entries."""
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, 1024, (64,), generator=g)
    alt = toks.clone()
    alt[2] = (alt[2] + 5) % 1024
    for types, reaches in (((SLIDING,), False), ((HCA,), True), ((CSA,), True)):
        m = _model(num_layers=1, layer_types=types, sliding_window=8, hash_layers=(), index_topk=16)
        d = (m(toks, [0, 64]) - m(alt, [0, 64])).abs().amax(-1)
        assert d[2] > 0 and (d[:2] == 0).all()
        assert bool(d[40:].max() > 1e-7) == reaches, (types, float(d[40:].max()))


def test_routing_hash_is_a_function_of_the_token_and_topk_follows_scores():
    m = _model()
    hash_moe, topk_moe = m.layers[0].mlp, m.layers[1].mlp
    assert hash_moe.is_hash and not topk_moe.is_hash
    ids = torch.tensor([5, 9, 5, 700, 9])
    x = torch.randn(5, 256)
    _, w, idx = hash_moe.route(x, ids)
    assert torch.equal(idx[0], idx[2]) and torch.equal(idx[1], idx[4])
    assert all(len(set(r.tolist())) == idx.shape[1] for r in idx)
    assert torch.allclose(w.sum(-1), torch.full((5,), 1.5), atol=1e-5)
    logits, w2, idx2 = topk_moe.route(x, ids)
    assert torch.equal(idx2.sort(-1).values, logits.topk(2, -1).indices.sort(-1).values)
    topk_moe.replay_indices = torch.tensor([[0, 1]] * 5)
    assert torch.equal(topk_moe.route(x, ids)[2], topk_moe.replay_indices)


def test_training_reduces_the_loss_and_reaches_every_parameter_group():
    m = _model()
    g = torch.Generator().manual_seed(3)
    data = torch.randint(0, 64, (96,), generator=g)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    losses = []
    for _ in range(12):
        loss = causal_lm_loss(m, data, [0, 40, 96])
        aux = m.indexer_loss()
        (loss + 0.01 * aux).backward()
        if not losses:
            named = dict(m.named_parameters())
            for key in ("layers.1.self_attn.compressor.compress.kv_proj.weight",
                        "layers.1.self_attn.compressor.indexer.q_b_proj.weight",
                        "layers.2.self_attn.compressor.position_bias", "layers.0.self_attn.sinks",
                        "layers.0.attn_hc.proj", "layers.1.mlp.experts.linear_fc1.weight", "layers.0.self_attn.o_a_weight"):
                assert named[key].grad is not None and named[key].grad.abs().sum() > 0, key
        opt.step()
        opt.zero_grad()
        losses.append(float(loss))
    assert losses[-1] < losses[0] - 1.0, losses
