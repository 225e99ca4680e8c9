"""Numerical definitions of the algorithm core against hand-written formulas: policy losses, KL estimators,
off-policy correction, aggregation weights, value / DPO / Bradley-Terry losses, group-normalised and GAE advantages,
rule rewards and datasets."""
import json
import math
import types

import pytest
import torch

from gcore_b200.core import advantage as A
from gcore_b200.loss import policy_loss as PL


def _cfg(**kw):
    d = dict(clip_low=0.2, clip_high=0.3, ppo_dual_clip_ratio_c=None, ppo_logps_ratio_clamp=None, sapo_tau_pos=1.0,
             sapo_tau_neg=1.05, offpolicy_correction="none", offpolicy_correction_level="token",
             offpolicy_correction_upper=2.0, offpolicy_correction_lower=None, offpolicy_correction_veto=None)
    d.update(kw)
    return types.SimpleNamespace(**d)


def _li(T=12, seqs=3, seed=0, roll=False):
    g = torch.Generator().manual_seed(seed)
    lp = (torch.randn(T, generator=g) * 0.3 - 1).requires_grad_(True)
    old = lp.detach() + torch.randn(T, generator=g) * 0.3
    adv = torch.randn(T, generator=g)
    mask = (torch.rand(T, generator=g) > 0.2).float()
    sid = torch.arange(T) * seqs // T
    rl = old + torch.randn(T, generator=g) * 0.1 if roll else None
    return PL.LossInput(lp, old, None, rl, adv, mask, sid.int(), seqs)


def test_grpo_clip_asymmetric_and_dual_clip():
    li = _li()
    cfg = _cfg()
    out = PL.get_loss("grpo")(cfg, li)
    ratio = torch.exp(li.logp - li.old_logp)
    ref = torch.maximum(-li.advantages * ratio, -li.advantages * ratio.clamp(0.8, 1.3))
    assert torch.allclose(out.token_loss, ref, atol=1e-6)
    # dual clip bounds the loss of negative-advantage tokens by -c * A
    cfg2 = _cfg(ppo_dual_clip_ratio_c=3.0)
    out2 = PL.get_loss("grpo")(cfg2, li)
    neg = li.advantages < 0
    ref2 = torch.where(neg, torch.minimum(ref, -3.0 * li.advantages), ref)
    assert torch.allclose(out2.token_loss, ref2, atol=1e-6)
    # gradient of an unclipped token is -A * ratio
    out.token_loss.sum().backward()
    unclipped = (ratio > 0.8) & (ratio < 1.3)
    assert torch.allclose(li.logp.grad[unclipped], (-li.advantages * ratio).detach()[unclipped], atol=1e-5)


def test_gspo_uses_one_ratio_per_sequence():
    li = _li()
    out = PL.get_loss("gspo")(_cfg(), li)
    d = (li.logp - li.old_logp).detach() * li.mask
    for s in range(3):
        sel = li.seq_ids == s
        expect = math.exp(float(d[sel].sum() / li.mask[sel].sum().clamp_min(1)))
        assert torch.allclose(out.ratios[sel], torch.full_like(out.ratios[sel], expect), rtol=1e-5)


def test_cispo_sapo_reinforce_gradients():
    li = _li()
    cfg = _cfg()
    out = PL.get_loss("cispo")(cfg, li)
    out.token_loss.sum().backward()
    ratio = torch.exp(li.logp - li.old_logp).detach()
    assert torch.allclose(li.logp.grad, -ratio.clamp(0.8, 1.3) * li.advantages, atol=1e-6)  # clipped IS weight, detached
    li2 = _li(seed=1)
    out2 = PL.get_loss("sapo")(cfg, li2)
    r2 = torch.exp(li2.logp - li2.old_logp)
    tau = torch.where(li2.advantages > 0, torch.tensor(1.0), torch.tensor(1.05))
    assert torch.allclose(out2.token_loss, -li2.advantages * (4 / tau) * torch.sigmoid(tau * (r2 - 1)), atol=1e-6)
    li3 = _li(seed=2)
    assert torch.allclose(PL.get_loss("reinforce")(cfg, li3).token_loss, -li3.advantages * li3.logp)
    with pytest.raises(KeyError):
        PL.get_loss("no_such_loss")


def test_vespo_sequence_kernel_is_detached():
    li = _li(roll=True)
    out = PL.get_loss("vespo")(_cfg(vespo_c1_pos=1.0, vespo_c1_neg=2.0, vespo_c2_pos=1.0, vespo_c2_neg=0.5), li)
    out.token_loss.sum().backward()
    # gradient = -phi(seq) * A : constant per sequence up to the advantage
    g = -li.logp.grad / li.advantages
    for s in range(3):
        sel = (li.seq_ids == s)
        assert torch.allclose(g[sel], g[sel][0].expand_as(g[sel]), rtol=1e-4, atol=1e-6)


def test_kl_estimators():
    lp, ref = torch.tensor([-1.0, -2.0, -0.5]), torch.tensor([-1.5, -1.0, -0.5])
    d = ref - lp
    assert torch.allclose(PL.kl_penalty(lp, ref, "k1"), -d)
    assert torch.allclose(PL.kl_penalty(lp, ref, "k2"), 0.5 * d * d)
    k3 = PL.kl_penalty(lp, ref, "k3")
    assert torch.allclose(k3, torch.exp(d) - d - 1) and bool((k3 >= 0).all()) and k3[2] == 0
    assert float(PL.kl_penalty(lp, ref, "k3", clamp=0.1).max()) <= 0.1 + 1e-7


@pytest.mark.parametrize("mode", ["truncate", "clip", "mask", "icepop", "kpop"])
def test_offpolicy_correction_modes(mode):
    li = _li(T=16, seqs=4, roll=True)
    cfg = _cfg(offpolicy_correction=mode, offpolicy_correction_upper=1.1)
    w, m = PL.offpolicy_correction(cfg, li.old_logp, li.rollout_logp, li.mask, li.seq_ids, 4)
    raw = torch.exp(li.old_logp - li.rollout_logp)
    lo, hi = 1 / 1.1, 1.1
    if mode == "truncate":
        assert torch.allclose(w, raw.clamp(max=hi))
    elif mode == "clip":
        assert torch.allclose(w, raw.clamp(lo, hi))
    elif mode == "mask":
        assert torch.equal(w, ((raw >= lo) & (raw <= hi)).float())
    elif mode == "icepop":
        assert torch.allclose(w, torch.where((raw >= lo) & (raw <= hi), raw, torch.zeros_like(raw)))
    else:
        for s in range(4):
            sel = li.seq_ids == s
            assert bool((w[sel] == 0).all()) or bool((w[sel] > 0).all())  # whole sequences are kept or dropped
    assert not w.requires_grad and "tis/weight_mean" in m
    cfg_seq = _cfg(offpolicy_correction="truncate", offpolicy_correction_level="sequence")
    ws, _ = PL.offpolicy_correction(cfg_seq, li.old_logp, li.rollout_logp, li.mask, li.seq_ids, 4)
    for s in range(4):
        sel = li.seq_ids == s
        assert torch.allclose(ws[sel], ws[sel][0].expand_as(ws[sel]))


def test_aggregation_weights_sum_to_share_of_global_loss():
    mask = torch.tensor([1, 1, 0, 1, 1, 1.0])
    sid = torch.tensor([0, 0, 0, 1, 1, 1], dtype=torch.int32)
    w_tok = PL.aggregation_weights(mask, sid, 2, True, 10.0)
    assert torch.allclose(w_tok, mask / 10) and abs(float(w_tok.sum()) - 0.5) < 1e-6
    w_seq = PL.aggregation_weights(mask, sid, 2, False, 4.0)   # 4 alive sequences globally, 2 of them here
    assert torch.allclose(w_seq, torch.tensor([1 / 2, 1 / 2, 0, 1 / 3, 1 / 3, 1 / 3]) / 4)
    assert abs(float(w_seq.sum()) - 0.5) < 1e-6


def test_value_dpo_and_bt_losses():
    v, old, ret = torch.tensor([1.0, 3.0]), torch.tensor([0.0, 0.0]), torch.tensor([0.5, 0.5])
    w = torch.tensor([0.5, 0.5])
    assert abs(float(PL.value_loss(v, old, ret, w, None)) - 0.5 * (0.25 * 0.5 + 6.25 * 0.5)) < 1e-6
    # clipping V to old +- 0.2 can only increase the loss (max of the two branches)
    assert float(PL.value_loss(v, old, ret, w, 0.2)) >= float(PL.value_loss(v, old, ret, w, None))
    pc, pr, rc, rr = torch.tensor([-5.0]), torch.tensor([-7.0]), torch.tensor([-6.0]), torch.tensor([-6.5])
    out = PL.dpo_loss(pc, pr, rc, rr, beta=0.1)
    loss = out[0] if isinstance(out, tuple) else out["loss"]
    assert abs(float(loss) - float(-torch.nn.functional.logsigmoid(torch.tensor(0.1 * ((-5 + 7) - (-6 + 6.5)))))) < 1e-6
    bt = PL.rm_bt_loss(torch.tensor([2.0, 0.0]), torch.tensor([1.0, 1.0]))
    bt_loss = bt[0] if isinstance(bt, tuple) else bt["loss"] if isinstance(bt, dict) else bt
    assert abs(float(bt_loss) - float(-torch.nn.functional.logsigmoid(torch.tensor([1.0, -1.0])).mean())) < 1e-6


def test_group_normalised_advantages():
    r = torch.tensor([1.0, 0.0, 0.0, 1.0, 5.0, 5.0, 5.0, 5.0])
    gid = torch.tensor([0, 0, 0, 0, 1, 1, 1, 1])
    adv = A.group_normalize(r, gid, None, eps=1e-6)
    g0 = r[:4]
    assert torch.allclose(adv[:4], (g0 - g0.mean()) / (g0.std() + 1e-6), atol=1e-5)
    assert torch.allclose(adv[4:], torch.zeros(4), atol=1e-4)       # no spread: no signal
    sm = torch.tensor([1, 1, 1, 0, 1, 1, 1, 1.0])
    adv2 = A.group_normalize(r, gid, sm, eps=1e-6)
    assert adv2[3] == 0 and abs(float(adv2[:3].sum())) < 1e-5        # invalid sample excluded from the statistics
    adv3 = A.group_normalize(r, gid, None, eps=1e-6, norm_by_std=False)
    assert torch.allclose(adv3[:4], g0 - g0.mean())


def test_gae_matches_backward_recursion():
    from gcore_b200.ops.rl import gae
    torch.manual_seed(0)
    B, S, gamma, lam = 3, 9, 0.97, 0.9
    r, v = torch.randn(B, S), torch.randn(B, S)
    m = torch.ones(B, S)
    m[0, 6:] = 0
    m[1, :2] = 0
    adv, ret = gae(r, v, m, gamma, lam)
    for b in range(B):
        last = 0.0
        idx = [t for t in range(S) if m[b, t] > 0]
        exp = {}
        for j in reversed(range(len(idx))):
            t = idx[j]
            nv = float(v[b, idx[j + 1]]) if j + 1 < len(idx) else 0.0
            delta = float(r[b, t]) + gamma * nv - float(v[b, t])
            last = delta + gamma * lam * last
            exp[t] = last
        for t in idx:
            assert abs(float(adv[b, t]) - exp[t]) < 1e-4
            assert abs(float(ret[b, t]) - (exp[t] + float(v[b, t]))) < 1e-4
        assert all(float(adv[b, t]) == 0 for t in range(S) if m[b, t] == 0)


def test_rule_reward_and_datasets(tmp_path):
    from gcore_b200.data.datasets import IndexedJsonlDataset, ResumableDistributedSampler
    from gcore_b200.reward.rewards import boxed_answer
    assert boxed_answer("so the answer is \\boxed{42}.") == "42"
    assert boxed_answer("nested \\boxed{\\frac{1}{2}} done") == "\\frac{1}{2}"
    assert boxed_answer("none here") is None
    p = tmp_path / "d.jsonl"
    with open(p, "w") as f:
        for i in range(10):
            f.write(json.dumps({"id": i, "prompt": [1, 2, i]}) + "\n")
    ds = IndexedJsonlDataset(str(p))
    assert len(ds) == 10 and ds[7]["id"] == 7
    s0 = ResumableDistributedSampler(len(ds), dp_rank=0, dp_size=2, shuffle=True, seed=3)
    s1 = ResumableDistributedSampler(len(ds), dp_rank=1, dp_size=2, shuffle=True, seed=3)
    a, b = list(iter(s0)), list(iter(s1))
    assert sorted(a + b) == list(range(10))
    # resume in the middle of an epoch: the remaining indices are exactly the tail of the same order
    s0.set_start_index(3)
    assert list(iter(s0)) == a[3:]
    sd = s0.state_dict()
    s2 = ResumableDistributedSampler(len(ds), dp_rank=0, dp_size=2, shuffle=True, seed=3)
    s2.load_state_dict(sd)
    assert list(iter(s2)) == a


def test_fipo_future_sum_and_influence_weights():
    from gcore_b200.configs.config import PpoConfig
    from gcore_b200.loss import policy_loss as PL
    torch.manual_seed(0)
    lens = [5, 1, 700, 33]
    seq_ids = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)])
    x = torch.randn(sum(lens)) * 0.05
    gamma = 2.0 ** (-1.0 / 8.0)
    got = PL.discounted_future_sum(x, seq_ids, gamma, chunk=64)
    ref = torch.zeros_like(x)
    o = 0
    for n in lens:
        acc = 0.0
        for t in range(n - 1, -1, -1):
            acc = float(x[o + t]) + gamma * acc
            ref[o + t] = acc
        o += n
    assert torch.allclose(got, ref, atol=1e-5)
    # loss: with logp == old every influence weight is 1 and fipo equals the clipped surrogate of grpo
    cfg = PpoConfig(loss_func="fipo", fipo_decay_rate=8.0, fipo_chunk_size=64)
    T = sum(lens)
    lp = (torch.randn(T) * 0.1 - 2.0).requires_grad_(True)
    adv = torch.randn(T)
    mask = torch.ones(T)
    li = PL.LossInput(lp, lp.detach().clone(), None, None, adv, mask, seq_ids, len(lens))
    a, b = PL.get_loss("fipo")(cfg, li), PL.get_loss("grpo")(cfg, li)
    assert torch.allclose(a.token_loss, b.token_loss, atol=1e-6)
    # a later token whose probability rose lifts the weight of the earlier tokens of its sequence only
    old = lp.detach().clone()
    cur = lp.detach().clone()
    cur[5 + 1 + 10] += 0.1                       # token 10 of the third sequence
    li = PL.LossInput(cur.requires_grad_(True), old, None, None, torch.ones(T), mask, seq_ids, len(lens))
    out = PL.get_loss("fipo")(cfg, li)
    w = -out.token_loss.detach() / torch.exp(cur.detach() - old)     # = influence weight where nothing is clipped
    s3 = 5 + 1
    assert torch.allclose(w[:s3], torch.ones(s3), atol=1e-6) and torch.allclose(w[s3 + 11:], torch.ones(T - s3 - 11), atol=1e-6)
    exp_w = torch.exp(0.1 * gamma ** torch.arange(10, -1, -1.0))
    assert torch.allclose(w[s3:s3 + 11], exp_w.clamp(0.8, 1.2), atol=1e-5)


def test_steer_token_weights():
    from gcore_b200.configs.config import PpoConfig
    from gcore_b200.loss import policy_loss as PL
    torch.manual_seed(1)
    T = 12
    cfg = PpoConfig(loss_func="steer", steer_token_weight_min=0.6)
    lp = (torch.randn(T) * 0.5 - 1.5).requires_grad_(True)
    old = lp.detach() + torch.randn(T) * 0.01
    adv = torch.randn(T)
    ent = torch.rand(T) * 2
    mask = torch.ones(T)
    mask[-2:] = 0
    seq_ids = torch.zeros(T, dtype=torch.long)
    li = PL.LossInput(lp, old, None, None, adv, mask, seq_ids, 1, ent, None)
    out, base = PL.get_loss("steer")(cfg, li), PL.get_loss("grpo")(cfg, li)
    p = lp.detach().exp()
    metric = (adv / old.exp() * p * (1 - p) * (p.log() + ent)).abs()
    k = -torch.log(torch.tensor(0.6)) / torch.clamp(metric[:10].max(), min=0.02)
    w = torch.exp(-k * metric).clamp(0.6, 1.0) * mask
    assert torch.allclose(out.token_loss, base.token_loss * w, atol=1e-6)
    assert abs(float(w[:10].min()) - 0.6) < 1e-5 and float(w[-1]) == 0.0   # the largest metric gets the floor


def test_ce_token_compaction_is_exact_and_skips_prompt_rows(monkeypatch):
    """Only positions inside the loss mask go through the vocabulary projection; losses, gradient norms and the
    masked log-probs are those of the full computation."""
    import sys
    import os
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "workers"))
    import parallel_worker as pw
    from gcore_b200.engine import train_engine as te
    from gcore_b200.models.config import get_preset
    rows = []
    real = te.linear_logprob_entropy

    def spy(hidden, *a, **k):
        rows.append(hidden.shape[0])
        return real(hidden, *a, **k)

    monkeypatch.setattr(te, "linear_logprob_entropy", spy)
    res = {}
    for on in (True, False):
        e = pw.engine(get_preset("tiny_llama", dtype="float32", qkv_bias=True), 1)
        e.policy_cfg.ce_token_compaction = on
        rows.clear()
        samples = pw.samples(8, 7)        # the loss mask covers about two thirds of every sequence
        m = e.finetune_step(samples)
        lp = e.compute_log_probs([{"tokens": s["tokens"], "prompt_length": 10} for s in pw.samples(2, 9)])
        res[on] = (m["lm_loss"], float(e.optimizer.last_grad_norm), lp, list(rows))
    assert abs(res[True][0] - res[False][0]) < 1e-6 and abs(res[True][1] - res[False][1]) < 1e-5
    for a, b in zip(res[True][2], res[False][2]):
        n = a["tokens"].numel()
        assert torch.allclose(a["logprobs"][9:n - 1], b["logprobs"][9:n - 1], atol=1e-6)
        assert float(a["logprobs"][:9].abs().sum()) == 0.0 and float(b["logprobs"][:9].abs().sum()) > 0.0
    assert sum(res[True][3]) < 0.8 * sum(res[False][3])


def test_low_precision_linear_modes_train(tmp_path):
    """policy.fp8 / fp8_qat / fp4_qat switch the decoder projections: fp8 compute stays close to bf16 / fp32 training,
    QAT sees fake-quantised weights with straight-through gradients, a frozen fp8 base trains under LoRA."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "workers"))
    import parallel_worker as pw
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import get_preset
    from gcore_b200.ops import lowp_linear, quant
    mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True, ffn_hidden_size=512)

    def run(steps=4, **flags):
        pc = PolicyConfig(recompute="none", without_ref=True, **flags)
        e = TrainingEngine(pc, OptimizerConfig(lr=1e-3, lr_decay_style="constant", weight_decay=0.0, max_grad_norm=1.0),
                           TrainingConfig(train_mbs=2, train_gbs=8), model_cfg=mcfg)
        e.setup_model_and_get_optimizer(seed=11)
        return e, [e.finetune_step(pw.samples(8, 50 + s))["lm_loss"] for s in range(steps)]

    base_e, base = run()
    assert base_e.lowp_modules == []
    for flags, tol in (({"fp8": True}, 0.02), ({"fp8_qat": True}, 0.02), ({"fp4_qat": True}, 0.08)):
        e, losses = run(**flags)
        assert len(e.lowp_modules) == 4 * mcfg.num_layers            # qkv, proj, fc1, fc2 of every layer
        assert all(abs(a - b) < tol for a, b in zip(base, losses)), (flags, base, losses)
        assert losses != base                                         # the low-precision path really ran
    # the QAT forward equals a plain linear on the fake-quantised weight, its gradient reaches the bf16 weight
    w = torch.randn(256, 256, requires_grad=True)
    x = torch.randn(5, 256)
    y = lowp_linear.qat_linear(x, w, None, None, "fp8_qat")
    q, s = quant.weight_quant_128x128_ref(w.detach(), pow2=True)
    assert torch.allclose(y, x @ quant.dequant_128x128(q, s).t(), atol=1e-4)
    y.sum().backward()
    assert torch.allclose(w.grad, x.sum(0)[None, :].expand(256, 256), atol=1e-5)
    # frozen block-fp8 base under LoRA: only the adapters train, the loss falls
    pc = PolicyConfig(recompute="none", without_ref=True, fp8=True)
    pc.lora.rank, pc.lora.alpha = 8, 16
    e = TrainingEngine(pc, OptimizerConfig(lr=5e-3, lr_decay_style="constant", weight_decay=0.0),
                       TrainingConfig(train_mbs=2, train_gbs=8), model_cfg=mcfg)
    e.setup_model_and_get_optimizer(seed=11)
    w0 = e.model.decoder.layers[0].self_attention.linear_qkv.weight.detach().clone()
    batch = pw.samples(8, 77)
    ls = [e.finetune_step(batch)["lm_loss"] for _ in range(8)]
    assert ls[-1] < ls[0] - 0.05 and torch.equal(w0, e.model.decoder.layers[0].self_attention.linear_qkv.weight)


def test_gdpo_advantage_variants():
    from gcore_b200.configs.config import PpoConfig
    from gcore_b200.core.advantage import get_advantage_fn
    torch.manual_seed(0)

    def batch():
        out = []
        for g in range(3):
            for j in range(4):
                out.append({"group_id": g, "mask": torch.tensor([0.0, 1.0, 1.0]), "rewards": torch.tensor(0.0),
                            "reward_dict": {"acc": float((g + j) % 2), "fmt": float(j % 3 == 0) * 0.5}})
        return out

    cfg = PpoConfig(advantage_type="group_gdpo", gdpo_reward_weights={"acc": 1.0, "fmt": 0.5})
    plain = get_advantage_fn("group_gdpo")(batch(), cfg)
    comb = torch.tensor([float(s["advantages"][1]) for s in plain])
    for g in range(3):       # every head is group-normalised, so the mix has zero mean inside each group
        assert abs(float(comb[g * 4:(g + 1) * 4].mean())) < 1e-5
    bn = get_advantage_fn("group_gdpo_sample_bn")(batch(), cfg)
    a = torch.tensor([float(s["advantages"][1]) for s in bn])
    assert abs(float(a.mean())) < 1e-5 and abs(float(a.std()) - 1.0) < 1e-3      # unbiased std of the batch is 1
    assert torch.allclose(a, (comb - comb.mean()) / (comb.std() + cfg.grpo_advantage_epsilon), atol=1e-5)
    assert bn[0]["advantages"][0] == 0 and abs(bn[0]["pre_bn_advantages"] - float(comb[0])) < 1e-6
    # without a process group the cross-rank form equals the local one; masked samples get no advantage
    b = batch()
    b[5]["sample_mask"] = False
    g1 = get_advantage_fn("gdpo_sample_bn")(b, cfg, dp_group=None)
    assert float(g1[5]["advantages"].abs().sum()) == 0.0 and "gdpo/bn_std" in g1[0]["advantage_stats"]
    PpoConfig(advantage_type="gdpo_sample_bn")      # accepted by the configuration


def test_entropy_regularisation_clip_cov_and_kl_cov():
    """kl-cov adds coef * |log-ratio| on exactly the top share of tokens by covariance; clip-cov removes the gradient
    of a bounded number of tokens inside the covariance window; both reduce to the clipped surrogate elsewhere."""
    from gcore_b200.configs.config import PpoConfig, ConfigError
    T = 200
    g = torch.Generator().manual_seed(3)
    lp = (torch.randn(T, generator=g) * 0.5 - 1.5).requires_grad_(True)
    old = lp.detach() + torch.randn(T, generator=g) * 0.05
    adv = torch.randn(T, generator=g) * 2
    mask = torch.ones(T)
    mask[:20] = 0
    li = PL.LossInput(lp, old, None, None, adv, mask, torch.zeros(T, dtype=torch.int32), 1)
    base = PL.get_loss("grpo")(PpoConfig(), li).token_loss

    cfg = PpoConfig(entropy_regularization_type="kl-cov", kl_cov_ratio=0.05, kl_cov_coef=0.5)
    out = PL.get_loss("kl_cov")(cfg, li)
    a, l = adv[20:], lp.detach()[20:]
    cov = (a - a.mean()) * (l - l.mean())
    top = torch.topk(cov, int(180 * 0.05)).indices + 20
    want = base.clone()
    want[top] = want[top] + 0.5 * (lp - old).abs()[top]
    assert torch.allclose(out.token_loss, want, atol=1e-6)
    assert float(out.metrics["kl_cov_frac"][0]) == 9.0

    cfg = PpoConfig(entropy_regularization_type="clip-cov", clip_cov_ratio=0.02, clip_cov_lb=0.2, clip_cov_ub=50.0)
    torch.manual_seed(0)
    out = PL.get_loss("clip_cov")(cfg, li)
    dropped = torch.nonzero((out.token_loss == 0) & (base != 0)).flatten()
    assert 1 <= dropped.numel() <= int(0.02 * 180)
    full_cov = torch.zeros(T)
    full_cov[20:] = cov
    assert bool(((full_cov[dropped] > 0.2) & (full_cov[dropped] < 50.0)).all()) and bool((dropped >= 20).all())
    kept = torch.ones(T, dtype=torch.bool)
    kept[dropped] = False
    assert torch.allclose(out.token_loss[kept], base[kept], atol=1e-6)
    out.token_loss.sum().backward()
    assert bool((lp.grad[dropped] == 0).all())

    with pytest.raises(ConfigError):
        PpoConfig(entropy_regularization_type="cov")
    with pytest.raises(ConfigError):
        PpoConfig(entropy_regularization_type="kl-cov", loss_func="cispo")
