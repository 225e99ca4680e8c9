"""Rollout decoder on CPU (eager op fallbacks): paged KV + continuous batching must reproduce a naive full-recompute
decode of the trainer model, token for token and log-prob for log-prob."""
import torch

from gcore_b200.models.config import get_preset
from gcore_b200.models.gpt import GPTModel
from gcore_b200.rollout.engine import InferEngine, RolloutWeights, SamplingParams


def naive_greedy(model, prompt, n_new):
    toks = list(prompt)
    lps = []
    for _ in range(n_new):
        t = torch.tensor(toks)
        cu = torch.tensor([0, len(toks)], dtype=torch.int32)
        with torch.no_grad():
            h, _ = model(t, torch.arange(len(toks), dtype=torch.int32), cu, len(toks))
            logits = model.logits(h[-1:]).float()
        lp = torch.log_softmax(logits, -1)[0]
        nxt = int(lp.argmax())
        toks.append(nxt)
        lps.append(float(lp[nxt]))
    return toks[len(prompt):], lps


def build(qk_ln=False):
    cfg = get_preset("tiny_llama", dtype="float32", qk_layernorm=qk_ln)
    torch.manual_seed(0)
    model = GPTModel(cfg, recompute="none")
    model.eval()
    return cfg, model


def test_greedy_matches_naive_decode_with_prefix_sharing():
    cfg, model = build()
    eng = InferEngine(cfg, RolloutWeights.from_model(model), max_running_requests=8, max_model_len=96,
                      kv_block_size=4, sync_interval=3, use_cuda_graph=False)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(3, 1024, (l,), generator=g).tolist() for l in (5, 9, 14)]
    reqs = eng.generate(prompts, SamplingParams(max_new_tokens=7, greedy=True), n=2)
    assert len(reqs) == 6
    for i, p in enumerate(prompts):
        ref_t, ref_lp = naive_greedy(model, p, 7)
        for j in range(2):
            r = reqs[i * 2 + j]
            assert r.finished and r.finish_reason == "length"
            assert r.out_tokens == ref_t, (i, j, r.out_tokens, ref_t)
            assert max(abs(a - b) for a, b in zip(r.out_logprobs, ref_lp)) < 1e-3
    st = eng.get_load()
    assert st["running"] == 0 and st["free_blocks"] == st["num_blocks"]


def test_more_requests_than_slots_and_stop_tokens():
    cfg, model = build(qk_ln=True)
    eng = InferEngine(cfg, RolloutWeights.from_model(model), max_running_requests=4, max_model_len=64,
                      kv_block_size=8, sync_interval=4, use_cuda_graph=False)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(3, 1024, (6 + i,), generator=g).tolist() for i in range(5)]
    ref = [naive_greedy(model, p, 6)[0] for p in prompts]
    stop = ref[0][2]
    reqs = eng.generate(prompts, SamplingParams(max_new_tokens=6, greedy=True, stop_token_ids=(stop,)), n=2)
    for i in range(5):
        want = ref[i]
        if stop in want:
            want = want[:want.index(stop) + 1]
        assert reqs[2 * i].out_tokens == want and reqs[2 * i + 1].out_tokens == want
    assert reqs[0].finish_reason == "stop"


def test_sampling_seeds_are_per_request_and_reproducible():
    cfg, model = build()
    eng = InferEngine(cfg, RolloutWeights.from_model(model), max_running_requests=8, max_model_len=64,
                      kv_block_size=8, sync_interval=2, use_cuda_graph=False)
    p = [[5, 6, 7, 8]]
    a = eng.generate(p, SamplingParams(max_new_tokens=5, seed=11), n=4)
    b = eng.generate(p, SamplingParams(max_new_tokens=5, seed=11), n=4)
    assert [r.out_tokens for r in a] == [r.out_tokens for r in b]
    assert len({tuple(r.out_tokens) for r in a}) > 1  # samples of one prompt differ
    eng.sleep(("kv_cache",))
    assert eng.asleep["kv_cache"]
    c = eng.generate(p, SamplingParams(max_new_tokens=5, seed=11), n=4)
    assert [r.out_tokens for r in a] == [r.out_tokens for r in c]


def test_block_fp8_serving_tracks_bf16_logprobs():
    """The engine can hold its dense projections in e4m3 with 128x128 scales and quantise activations 1x128 on the fly;
    generated log-probs stay close to the full-precision engine's for the same tokens."""
    import torch
    from gcore_b200.models.config import ModelConfig
    from gcore_b200.models.gpt import GPTModel
    from gcore_b200.rollout.engine import InferEngine, RolloutWeights, SamplingParams
    mcfg = ModelConfig(num_layers=2, hidden_size=256, num_attention_heads=4, num_kv_heads=2, ffn_hidden_size=768,
                       vocab_size=512, dtype="float32")
    model = GPTModel(mcfg, tp_size=1)
    model.reset_parameters(4)
    mk = lambda: InferEngine(mcfg, RolloutWeights.from_model(model, clone=True), num_kv_blocks=64, kv_block_size=4,  # noqa: E731
                             max_model_len=48, use_cuda_graph=False)
    ref, q8 = mk(), mk()
    q8.quantize_weights_fp8()
    assert set(q8.w.layers[0].fp8) == {"qkv_w", "o_w", "fc1_w", "fc2_w"}
    assert q8.w.layers[0].fp8["fc1_w"][0].dtype == torch.float8_e4m3fn
    prompts = [[5, 9, 33, 70, 2], [100, 101, 102]]
    # sampling with the same seeds: the Gumbel noise is identical, so tokens differ only where quantisation moves the
    # logits by more than the noise gap; log-probs are compared on the common prefix
    sp = SamplingParams(temperature=1.0, max_new_tokens=8, seed=11)
    for e in (ref, q8):
        e.wake_up(("kv_cache",))
    a = ref.generate(prompts, sp)
    b = q8.generate(prompts, sp)
    compared = 0
    for ra, rb in zip(a, b):
        for t, (x, y) in enumerate(zip(ra.out_tokens, rb.out_tokens)):
            if x != y:
                break
            assert abs(ra.out_logprobs[t] - rb.out_logprobs[t]) < 0.1
            compared += 1
    assert compared >= 8


def test_weight_sync_into_a_separate_rollout_copy_and_verify():
    """Engine with its own weight copy (not sharing storage): ``sync_weights`` moves the trainer's current weights in
    bucketed copies and ``verify`` (per-tensor hashes) finds no difference afterwards."""
    import torch
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import get_preset
    from gcore_b200.rollout.engine import InferEngine, RolloutWeights
    from gcore_b200.rollout.weight_sync import plan_buckets, reshard_tensor, sync_weights, verify
    mcfg = get_preset("tiny_llama", dtype="float32")
    eng = TrainingEngine(PolicyConfig(recompute="none", without_ref=True), OptimizerConfig(lr=1e-2), TrainingConfig(),
                         model_cfg=mcfg)
    eng.setup_model_and_get_optimizer(seed=1, with_ref=False)
    ie = InferEngine(mcfg, RolloutWeights.from_model(eng.model, clone=True), num_kv_blocks=32, kv_block_size=4,
                     max_model_len=32, use_cuda_graph=False)
    assert verify(eng, ie) == []
    with torch.no_grad():
        for p in eng.model.parameters():
            p.add_(0.01)
    stale = verify(eng, ie)
    assert len(stale) > 5                                   # the copy is now out of date ...
    stats = sync_weights(eng, ie, max_bucket_mb=1)
    assert stats["bytes"] > 0 and verify(eng, ie) == []     # ... and in sync again
    # bucket planner: sequential buckets below the byte limit
    b = plan_buckets([("a", 600), ("b", 500), ("c", 300), ("d", 900)], 1000)
    assert b == [["a"], ["b", "c"], ["d"]]
    # re-sharding a fused QKV weight from TP=2 to TP=1 restores the [Q | K | V] layout
    D, hq, hk = mcfg.head_dim, mcfg.num_attention_heads, mcfg.num_kv_heads
    full = torch.arange((hq + 2 * hk) * D, dtype=torch.float32)[:, None].repeat(1, 4)
    name = "decoder.layers.0.self_attention.linear_qkv.weight"
    shards = [reshard_tensor(name, [full], "column", 2, r, mcfg) for r in range(2)]
    assert torch.equal(reshard_tensor(name, shards, "column", 1, 0, mcfg), full)


def test_mla_moe_model_serves_from_latent_cache():
    """DeepSeek-V3-style model (multi-head latent attention, sigmoid group routing with a shared expert, first layer
    dense): the decoder caches only the latent + shared rotated key and attends in the absorbed form; it must equal
    the trainer model's full recompute, with more requests than batch slots and shared prompt prefixes."""
    from gcore_b200.models.config import ModelConfig
    cfg = ModelConfig(arch="deepseek_v3", num_layers=3, hidden_size=64, num_attention_heads=4, num_kv_heads=4,
                      ffn_hidden_size=128, vocab_size=256, use_mla=True, q_lora_rank=32, kv_lora_rank=32,
                      qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, head_dim=24, num_experts=8, moe_top_k=2,
                      moe_ffn_hidden_size=32, moe_shared_expert_ffn=32, moe_router_type="sigmoid_group", moe_n_group=4,
                      moe_topk_group=2, first_k_dense=1, moe_routed_scaling_factor=2.5, moe_router_bias=True,
                      rope_interleaved=True, dtype="float32")
    torch.manual_seed(0)
    model = GPTModel(cfg, recompute="none")
    model.eval()
    # the model trains: gradients reach the latent projections
    t = torch.randint(3, 256, (12,))
    h, _ = model(t, torch.arange(12, dtype=torch.int32), torch.tensor([0, 12], dtype=torch.int32), 12)
    model.logits(h).float().logsumexp(-1).sum().backward()
    a = model.decoder.layers[1].self_attention
    assert a.linear_kv_down_proj.weight.grad.abs().sum() > 0 and a.linear_q_up_proj.weight.grad.abs().sum() > 0
    eng = InferEngine(cfg, RolloutWeights.from_model(model), max_running_requests=4, max_model_len=48,
                      kv_block_size=4, sync_interval=3, use_cuda_graph=False)
    assert eng.k_cache == [] and eng.mla_dim == 40
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(3, 256, (l,), generator=g).tolist() for l in (5, 9, 7)]
    reqs = eng.generate(prompts, SamplingParams(max_new_tokens=6, greedy=True), n=2)
    assert tuple(eng.k_cache[0].shape[2:]) == (1, 40) and eng.v_cache[0].numel() == 0
    for i, p in enumerate(prompts):
        ref_t, ref_lp = naive_greedy(model, p, 6)
        for j in range(2):
            r = reqs[i * 2 + j]
            assert r.out_tokens == ref_t, (i, j, r.out_tokens, ref_t)
            assert max(abs(x - y) for x, y in zip(r.out_logprobs, ref_lp)) < 1e-3


def test_mla_rollout_with_lora_adapters_on_the_latent_projections():
    """LoRA on the q / kv up-projections and the output projection of an MLA model (non-zero B): the decoder's
    absorbed attention folds the adapter of the kv up-projection into its matrices and must still equal the model."""
    from gcore_b200.configs.config import LoRAConfig
    from gcore_b200.models.config import ModelConfig
    from gcore_b200.models.lora import apply_lora
    cfg = ModelConfig(arch="deepseek_v3", num_layers=2, hidden_size=64, num_attention_heads=4, num_kv_heads=4,
                      ffn_hidden_size=128, vocab_size=256, use_mla=True, q_lora_rank=32, kv_lora_rank=32,
                      qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, head_dim=24, rope_interleaved=True,
                      dtype="float32")
    torch.manual_seed(0)
    model = GPTModel(cfg, recompute="none")
    ads = apply_lora(model, LoRAConfig(rank=4, alpha=8, type="lora", lora_B_init_method="normal",
                                       target_modules=["linear_q_up_proj", "linear_kv_up_proj", "linear_proj"]), seed=1)
    assert len(ads) == 6
    with torch.no_grad():
        for a in ads.values():
            for b in a.lora_B:
                b.mul_(20.0)   # make the adapters matter
    model.eval()
    eng = InferEngine(cfg, RolloutWeights.from_model(model), max_running_requests=4, max_model_len=48,
                      kv_block_size=4, sync_interval=3, use_cuda_graph=False)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(3, 256, (l,), generator=g).tolist() for l in (6, 9)]
    reqs = eng.generate(prompts, SamplingParams(max_new_tokens=6, greedy=True))
    for p, r in zip(prompts, reqs):
        ref_t, ref_lp = naive_greedy(model, p, 6)
        assert r.out_tokens == ref_t and max(abs(x - y) for x, y in zip(r.out_logprobs, ref_lp)) < 1e-3
    # and the adapters do change the outputs
    for m in model.modules():
        if getattr(m, "lora", None) is not None:
            m.lora = None
    assert naive_greedy(model, prompts[0], 6)[1] != [round(x, 9) for x in reqs[0].out_logprobs]


def test_block_manager_accounting_fork_and_exhaustion():
    """The C++ scheduler / block manager on its own: admission order, block accounting across reserve / advance /
    finish, copy-on-write fork of a prompt's blocks (shared full blocks, one private copy of the partial block), and
    refusal instead of over-commitment when the cache is exhausted."""
    from gcore_b200.rollout.engine import _Sched
    bs = 4
    s = _Sched(num_blocks=12, block_size=bs, max_running=8, max_prefill_tokens=64)
    assert s.stats()["free_blocks"] == 12
    assert s.add(1, 10, 6) == 0 and s.add(2, 5, 4) == 0          # prompts of 10 and 5 tokens
    pre, dec = s.step(8, 0)
    assert pre == [1, 2] and dec == []
    for rid in pre:
        s.commit(rid, True)
    used = 12 - s.stats()["free_blocks"]
    assert used >= 3 + 2                                            # ceil(10/4) + ceil(5/4) blocks hold the prompts
    tabs, _ = s.tables([1, 2], 8)
    assert len(set(tabs[0, :3].tolist())) == 3 and not set(tabs[0, :3].tolist()) & set(tabs[1, :2].tolist())
    # fork request 1: full blocks are shared, the partial last block (10 % 4 = 2 tokens) is copied
    rc, src, dst = s.fork(1, 3, 6)
    assert rc == 0 and src >= 0 and dst >= 0 and src != dst
    t3, _ = s.tables([3], 8)
    assert t3[0, :2].tolist() == tabs[0, :2].tolist() and int(t3[0, 2]) == dst and int(tabs[0, 2]) == src
    free_after_fork = s.stats()["free_blocks"]
    # decode: reservations take blocks only when a block boundary is crossed
    assert s.reserve(1, 3) == 0
    s.advance(1, 2)
    assert s.reserve(3, 3) == 0
    s.advance(3, 2)
    assert s.stats()["free_blocks"] <= free_after_fork
    # finishing the parent keeps the shared blocks alive for the child; finishing both returns everything
    s.finish(1)
    t3b, _ = s.tables([3], 8)
    assert t3b[0, :3].tolist() == t3[0, :3].tolist()
    s.finish(3)
    s.finish(2)
    st = s.stats()
    assert st["free_blocks"] == st["num_blocks"] == 12 and st["running"] == 0
    # exhaustion: a request that cannot fit is refused at add time, the cache stays consistent
    assert s.add(9, 100, 50) != 0
    assert s.stats()["free_blocks"] == 12 and s.stats()["waiting"] == 0


def test_repetition_penalty_follows_the_definition_across_slot_reuse():
    """Greedy decode with a repetition penalty = a full recompute that divides (positive) / multiplies (negative) the
    logits of every token of the prompt and of the output so far; more requests than slots, so slots are re-used and
    their tables of seen tokens restart."""
    cfg, model = build()
    pen = 1.7
    eng = InferEngine(cfg, RolloutWeights.from_model(model), max_running_requests=2, max_model_len=64,
                      kv_block_size=4, sync_interval=3, use_cuda_graph=False)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, 1024, (l,), generator=g).tolist() for l in (6, 11, 4, 9, 7)]
    reqs = eng.generate(prompts, SamplingParams(max_new_tokens=8, greedy=True, repetition_penalty=pen))
    plain = eng.generate(prompts, SamplingParams(max_new_tokens=8, greedy=True))
    assert any(a.out_tokens != b.out_tokens for a, b in zip(reqs, plain))     # the penalty changes something
    for r, p in zip(reqs, prompts):
        toks = list(p)
        for want, want_lp in zip(r.out_tokens, r.out_logprobs):
            t = torch.tensor(toks)
            with torch.no_grad():
                h, _ = model(t, torch.arange(len(toks), dtype=torch.int32), torch.tensor([0, len(toks)], dtype=torch.int32),
                             len(toks))
                z = model.logits(h[-1:]).float()[0]
            seen = torch.zeros_like(z, dtype=torch.bool)
            seen[t] = True
            z = torch.where(seen, torch.where(z > 0, z / pen, z * pen), z)
            lp = torch.log_softmax(z, -1)
            assert int(lp.argmax()) == want
            assert abs(float(lp[want]) - want_lp) < 1e-3
            toks.append(want)


def test_prompt_ids_outside_the_vocabulary_are_refused_on_the_host():
    import pytest
    cfg, model = build()
    eng = InferEngine(cfg, RolloutWeights.from_model(model), max_running_requests=2, max_model_len=32,
                      kv_block_size=4, use_cuda_graph=False)
    with pytest.raises(ValueError, match="outside"):
        eng.generate([[5, 6, cfg.vocab_size]], SamplingParams(max_new_tokens=2, greedy=True))
    with pytest.raises(ValueError, match="outside"):
        eng.generate([[5, -1]], SamplingParams(max_new_tokens=2, greedy=True))
    assert len(eng.generate([[5, 6, cfg.vocab_size - 1]], SamplingParams(max_new_tokens=2, greedy=True))) == 1


def test_separate_rollout_copy_owns_its_moe_and_latent_attention_weights():
    """``share_rollout_weights=false`` with an MoE + latent-attention model: the engine's copy is really separate
    (trainer updates do not show through), ``verify`` sees the stale expert / router / latent tensors, ``sync_weights``
    brings them over and the engine then reproduces the trainer's log-probs."""
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import ModelConfig
    from gcore_b200.rollout.weight_sync import sync_weights, verify
    mcfg = ModelConfig(arch="deepseek_v3", num_layers=2, hidden_size=64, num_attention_heads=4, num_kv_heads=4,
                       ffn_hidden_size=128, vocab_size=256, use_mla=True, q_lora_rank=32, kv_lora_rank=32,
                       qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, head_dim=24, num_experts=8, moe_top_k=2,
                       moe_ffn_hidden_size=32, moe_shared_expert_ffn=32, moe_router_type="sigmoid_group", moe_n_group=4,
                       moe_topk_group=2, first_k_dense=1, moe_router_bias=True, dtype="float32")
    eng = TrainingEngine(PolicyConfig(recompute="none", without_ref=True), OptimizerConfig(lr=1e-2), TrainingConfig(),
                         model_cfg=mcfg)
    eng.setup_model_and_get_optimizer(seed=1, with_ref=False)
    ie = InferEngine(mcfg, RolloutWeights.from_model(eng.model, clone=True), num_kv_blocks=64, kv_block_size=4,
                     max_model_len=48, use_cuda_graph=False)
    moe = eng.model.decoder.layers[1].mlp
    assert ie.w.layers[1].moe is not moe
    assert ie.w.layers[1].moe.experts.linear_fc1.weight.data_ptr() != moe.experts.linear_fc1.weight.data_ptr()
    assert ie.w.layers[0].mla is not eng.model.decoder.layers[0].self_attention
    assert verify(eng, ie) == []
    prompt = [5, 9, 200, 31, 7]
    before = ie.generate([prompt], SamplingParams(max_new_tokens=6, greedy=True))[0]
    with torch.no_grad():
        for p in eng.model.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    stale = verify(eng, ie)
    assert any("experts.linear_fc1" in n for n in stale) and any("router" in n for n in stale)
    assert any("linear_kv_up_proj" in n for n in stale)
    again = ie.generate([prompt], SamplingParams(max_new_tokens=6, greedy=True))[0]
    assert again.out_tokens == before.out_tokens            # the trainer's update does not show through
    sync_weights(eng, ie, max_bucket_mb=1)
    assert verify(eng, ie) == []
    ref_t, ref_lp = naive_greedy(eng.model.eval(), prompt, 6)
    after = ie.generate([prompt], SamplingParams(max_new_tokens=6, greedy=True))[0]
    assert after.out_tokens == ref_t and max(abs(a - b) for a, b in zip(after.out_logprobs, ref_lp)) < 1e-3
