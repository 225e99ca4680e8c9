"""End-to-end GRPO step on CPU with a tiny model: rollout (paged decoder) -> reward -> log-probs -> advantages ->
clipped policy update with KL -> shared-storage weight hand-over."""
import torch

from gcore_b200.configs.base import from_dict
from gcore_b200.configs.config import RlConfig
from gcore_b200.models.config import get_preset
from gcore_b200.trainer.grpo_trainer import GrpoTrainer


def make_cfg(critic=None, **ppo):
    extra = {"critic": critic} if critic is not None else {}
    return from_dict(RlConfig, {**extra,
        "training": {"rollout_gbs": 4, "sampling_repeat_n": 4, "train_gbs": 16, "train_mbs": 4, "seed": 3},
        "policy": {"recompute": "none"},
        "optimizer": {"lr": 3e-3, "lr_decay_style": "constant", "weight_decay": 0.0},
        "sampler": {"infer_engine_configs": [{"generate_max_tokens": 12, "max_model_len": 40, "kv_block_size": 4,
                                               "disable_cuda_graph": True}]},
        "data": {"max_prompt_length": 16},
        "ppo": ppo,
    })


def reward_has_small_token(samples, **_):
    # reward responses that contain a token id below 300: learnable signal for a random-init model
    return torch.tensor([float((s["tokens"][s["prompt_length"]:] < 300).float().mean()) for s in samples])


def test_grpo_steps_improve_reward_and_keep_engine_in_sync():
    torch.manual_seed(0)
    cfg = make_cfg()
    tr = GrpoTrainer(cfg, model_cfg=get_preset("tiny_llama", dtype="float32"), reward_fn=reward_has_small_token).setup()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 1024, (8,), generator=g).tolist() for _ in range(4)]
    rewards = []
    for _ in range(16):
        m = tr.step(prompts)
        rewards.append(m["rollout-rewards/mean"])
        assert m["policy/grad_norm"] > 0
        assert abs(m["ppo-metrics/ratio"] - 1.0) < 1e-3  # first epoch after on-policy rollout: ratio == 1
    assert sum(rewards[-3:]) / 3 > sum(rewards[:3]) / 3 + 0.1, rewards
    # the rollout engine reads the trainer's parameter storage
    w = tr.engine.w.layers[0].qkv_w
    p = tr.policy.model.decoder.layers[0].self_attention.linear_qkv.weight
    assert w.data_ptr() == p.data_ptr()
    # trainer log-probs agree with the log-probs the decoder reported for the tokens it sampled
    s = tr.last_samples[0]
    P, S = s["prompt_length"], s["sequence_length"]
    assert torch.allclose(s["logprobs"][P - 1:S - 1], s["rollout_log_probs"][P - 1:S - 1], atol=2e-3)


def test_alternative_losses_run():
    for loss, extra in (("gspo", {"per_token_loss": False}), ("cispo", {}), ("sapo", {}), ("steer", {}),
                        ("steer", {"steer_policy_method": "cispo", "steer_token_weight_min": 0.5}),
                        ("fipo", {"ppo_dual_clip_ratio_c": 3.0}),
                        ("grpo", {"entropy_regularization_type": "kl-cov", "kl_cov_ratio": 0.1}),
                        ("grpo", {"entropy_regularization_type": "clip-cov", "clip_cov_lb": 0.0})):
        cfg = make_cfg(loss_func=loss, **extra)
        tr = GrpoTrainer(cfg, model_cfg=get_preset("tiny_llama", dtype="float32"),
                         reward_fn=reward_has_small_token).setup()
        m = tr.step([[5, 6, 7, 8, 9], [10, 11, 12], [13, 14, 15, 16], [20, 21]])
        assert m["policy/grad_norm"] >= 0 and "ppo-metrics/pg_loss" in m
        if extra.get("entropy_regularization_type") == "kl-cov":
            assert m["ppo-metrics/kl_cov_frac"] > 0


def test_grpo_step_with_moe_policy_and_ppo_critic_value_path():
    """MoE decoder through the whole loop (the rollout engine runs the router + grouped experts of the shared
    module), and the trainer's log-probs still agree with the decoder's."""
    from gcore_b200.models.config import ModelConfig
    torch.manual_seed(1)
    mcfg = ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=128, num_attention_heads=4, num_kv_heads=2,
                       ffn_hidden_size=256, vocab_size=512, num_experts=8, moe_top_k=2, moe_ffn_hidden_size=64,
                       moe_aux_loss_coef=1e-3, dtype="float32", qk_layernorm=True)
    tr = GrpoTrainer(make_cfg(), model_cfg=mcfg, reward_fn=reward_has_small_token).setup()
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(3, 512, (6,), generator=g).tolist() for _ in range(4)]
    for _ in range(2):
        m = tr.step(prompts)
    assert m["policy/grad_norm"] > 0
    s = tr.last_samples[0]
    P, S = s["prompt_length"], s["sequence_length"]
    assert torch.allclose(s["logprobs"][P - 1:S - 1], s["rollout_log_probs"][P - 1:S - 1], atol=5e-3)


def test_ppo_with_critic_runs_gae_and_value_update():
    """advantage_type=ppo: a value-head critic supplies values, GAE builds advantages / returns, both models step."""
    torch.manual_seed(2)
    cfg = make_cfg(critic={"recompute": "none", "optimizer": {"lr": 1e-3, "lr_decay_style": "constant"}},
                   advantage_type="ppo", ppo_gae_lambda=0.95, ppo_discount_factor=1.0)
    tr = GrpoTrainer(cfg, model_cfg=get_preset("tiny_llama", dtype="float32"), reward_fn=reward_has_small_token).setup()
    assert tr.critic is not None
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(3, 1024, (8,), generator=g).tolist() for _ in range(4)]
    m = tr.step(prompts)
    assert "value/loss" in m and m["policy/grad_norm"] >= 0
    s = tr.last_samples[0]
    assert "values" in s and "returns" in s and s["advantages"].numel() == s["tokens"].numel()


def test_lora_grpo_resyncs_only_the_adapted_projections():
    """LoRA on q/kv/o: the base stays frozen and shared with the rollout engine, the adapted projections get a private
    rollout copy that is rebuilt from base + delta at every hand-over; the decoder's log-probs follow the adapters."""
    torch.manual_seed(3)
    cfg = make_cfg()
    cfg.policy.lora.rank = 4      # rank > 0 switches LoRA on
    cfg.policy.lora.alpha = 8
    cfg.policy.lora.target_modules = ["linear_qkv", "linear_proj"]
    tr = GrpoTrainer(cfg, model_cfg=get_preset("tiny_llama", dtype="float32"), reward_fn=reward_has_small_token).setup()
    layer = tr.policy.model.decoder.layers[0]
    lw = tr.engine.w.layers[0]
    assert lw.qkv_w.data_ptr() != layer.self_attention.linear_qkv.weight.data_ptr()   # private (adapted)
    assert lw.fc1_w.data_ptr() == layer.mlp.linear_fc1.weight.data_ptr()              # shared (not adapted)
    base_before = layer.self_attention.linear_qkv.weight.detach().clone()
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(3, 1024, (8,), generator=g).tolist() for _ in range(4)]
    for _ in range(3):
        m = tr.step(prompts)
    assert m["policy/grad_norm"] > 0
    assert torch.equal(layer.self_attention.linear_qkv.weight.detach(), base_before)  # frozen base
    merged = base_before + layer.self_attention.linear_qkv.lora.delta_weight()
    assert torch.allclose(lw.qkv_w, merged, atol=1e-6) and not torch.allclose(lw.qkv_w, base_before, atol=1e-6)
    s = tr.last_samples[0]
    P, S = s["prompt_length"], s["sequence_length"]
    assert torch.allclose(s["logprobs"][P - 1:S - 1], s["rollout_log_probs"][P - 1:S - 1], atol=5e-3)


def test_generative_and_bt_reward_models_drive_a_grpo_step():
    """Generative-reward RL: a second decoder judges every response (votes parsed from its sampled tokens), a
    Bradley-Terry reward model (value-head engine) scores the same responses, and a rule reward is mixed in."""
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.gpt import GPTModel
    from gcore_b200.reward.rewards import BtRmReward, GenRmReward, MixReward, RuleReward
    from gcore_b200.rollout.engine import InferEngine, RolloutWeights, SamplingParams
    torch.manual_seed(4)
    mcfg = get_preset("tiny_llama", dtype="float32")
    judge_model = GPTModel(mcfg, tp_size=1)
    judge_model.reset_parameters(21)
    judge = InferEngine(mcfg, RolloutWeights.from_model(judge_model), num_kv_blocks=256, kv_block_size=4,
                        max_model_len=64, use_cuda_graph=False)
    judge.wake_up(("kv_cache",))
    gen_rm = GenRmReward(judge, build_prompt=lambda s: s["tokens"][-12:].tolist() + [7],
                         parse=lambda toks: 1.0 if toks[0] % 2 == 0 else -1.0,
                         sampling=SamplingParams(temperature=1.0, max_new_tokens=2, seed=3), repeat_n=3)
    rm = TrainingEngine(PolicyConfig(recompute="none", without_ref=True), OptimizerConfig(), TrainingConfig(),
                        model_cfg=mcfg, value_head=True)
    rm.setup_model_and_get_optimizer(seed=22, with_ref=False)
    reward = MixReward([("rule", RuleReward(reward_has_small_token), 1.0), ("gen_rm", gen_rm, 0.5),
                        ("bt_rm", BtRmReward(rm), 0.25)])
    tr = GrpoTrainer(make_cfg(), model_cfg=mcfg, reward_fn=reward).setup()
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(3, 1024, (8,), generator=g).tolist() for _ in range(4)]
    m = tr.step(prompts)
    assert m["policy/grad_norm"] > 0
    s = tr.last_samples[0]
    assert set(s["reward_dict"]) == {"rule", "gen_rm", "bt_rm"}
    assert -1.0 <= s["reward_dict"]["gen_rm"] <= 1.0
    total = s["reward_dict"]["rule"] + 0.5 * s["reward_dict"]["gen_rm"] + 0.25 * s["reward_dict"]["bt_rm"]
    assert abs(float(s["rewards"]) - total) < 1e-5


def test_grpo_with_fp8_base_lora_and_mla_moe_policy():
    """The shape of the fp8 + LoRA recipe in miniature: DeepSeek-V3-style model (MLA, sigmoid-group MoE, dense first
    layer), frozen block-fp8 projections, adapters on the MLA projections; the rollout engine serves the latent cache
    with the fp8 products of the trainer, so its log-probs stay close to the trainer's."""
    from gcore_b200.models.config import ModelConfig
    mcfg = ModelConfig(arch="deepseek_v3", num_layers=3, hidden_size=128, num_attention_heads=4, num_kv_heads=4,
                       ffn_hidden_size=256, vocab_size=512, use_mla=True, q_lora_rank=128, kv_lora_rank=128,
                       qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, head_dim=48, num_experts=8, moe_top_k=2,
                       moe_ffn_hidden_size=64, moe_shared_expert_ffn=128, moe_router_type="sigmoid_group",
                       moe_n_group=4, moe_topk_group=2, first_k_dense=1, moe_routed_scaling_factor=2.5,
                       moe_router_bias=True, rope_interleaved=True, dtype="float32")
    cfg = make_cfg()
    cfg.policy.fp8 = True
    cfg.policy.lora.rank, cfg.policy.lora.alpha, cfg.policy.lora.type = 8, 16, "lora"
    cfg.policy.lora.target_modules = ["linear_q_down_proj", "linear_q_up_proj", "linear_kv_down_proj",
                                      "linear_kv_up_proj", "linear_proj"]
    torch.manual_seed(0)
    tr = GrpoTrainer(cfg, model_cfg=mcfg, reward_fn=reward_has_small_token).setup()
    assert tr.serve_fp8 and len(tr.policy.adapters) == 15 and len(tr.policy.lowp_modules) > 15
    base = tr.policy.model.decoder.layers[1].self_attention.linear_kv_up_proj.weight.detach().clone()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 512, (8,), generator=g).tolist() for _ in range(4)]
    m = tr.step(prompts)
    s = tr.last_samples[0]
    P, S = s["prompt_length"], s["sequence_length"]
    assert float((s["logprobs"][P - 1:S - 1] - s["rollout_log_probs"][P - 1:S - 1]).abs().max()) < 0.03
    assert m["policy/grad_norm"] > 0 and abs(m["ppo-metrics/ratio"] - 1.0) < 1e-3
    tr.step(prompts)
    assert torch.equal(base, tr.policy.model.decoder.layers[1].self_attention.linear_kv_up_proj.weight)  # frozen base


def test_lora_on_the_router_trains_and_reaches_the_rollout_engine():
    """"router" in lora.target_modules: the routing matrix gets an adapter (replicated), it trains with the base frozen,
    and the rollout engine (which runs the shared MoE module) routes with it."""
    from gcore_b200.models.config import ModelConfig
    mcfg = ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=128, num_attention_heads=4, num_kv_heads=2,
                       ffn_hidden_size=256, vocab_size=512, num_experts=8, moe_top_k=2, moe_ffn_hidden_size=64,
                       moe_aux_loss_coef=1e-3, dtype="float32", qk_layernorm=True)
    cfg = make_cfg()
    cfg.policy.lora.rank, cfg.policy.lora.alpha = 4, 8
    cfg.policy.lora.target_modules = ["linear_qkv", "router"]
    torch.manual_seed(1)
    tr = GrpoTrainer(cfg, model_cfg=mcfg, reward_fn=reward_has_small_token).setup()
    routers = [n for n in tr.policy.adapters if n.endswith("router")]
    assert len(routers) == 2
    r0 = tr.policy.model.decoder.layers[0].mlp.router
    base = r0.weight.detach().clone()
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(3, 512, (8,), generator=g).tolist() for _ in range(4)]
    for _ in range(3):
        m = tr.step(prompts)
    assert torch.equal(base, r0.weight) and float(r0.lora.lora_B[0].detach().abs().sum()) > 0   # only the adapter moved
    s = tr.last_samples[0]
    P, S = s["prompt_length"], s["sequence_length"]
    assert torch.allclose(s["logprobs"][P - 1:S - 1], s["rollout_log_probs"][P - 1:S - 1], atol=2e-3)


def test_lora_on_grouped_experts_shared_and_per_expert():
    """`linear_fc1` / `linear_fc2` among the LoRA targets also adapt the grouped expert projections: one adapter per
    layer or one per expert; the adapted forward equals the forward with the deltas merged into the expert weights."""
    from gcore_b200.configs.config import LoRAConfig
    from gcore_b200.models.config import ModelConfig
    from gcore_b200.models.gpt import GPTModel
    from gcore_b200.models.lora import ExpertLoRA, apply_lora, merge_lora_
    mcfg = ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=64, num_attention_heads=2, num_kv_heads=2,
                       ffn_hidden_size=128, vocab_size=128, num_experts=4, moe_top_k=2, moe_ffn_hidden_size=32,
                       dtype="float32")
    t = torch.randint(3, 128, (14,))
    pos, cu = torch.arange(14, dtype=torch.int32), torch.tensor([0, 14], dtype=torch.int32)
    for shared in (True, False):
        torch.manual_seed(0)
        model = GPTModel(mcfg, recompute="none")
        ads = apply_lora(model, LoRAConfig(rank=4, alpha=8, target_modules=["linear_fc1", "linear_fc2"],
                                           share_expert_adapters=shared), seed=3)
        ex = [a for a in ads.values() if isinstance(a, ExpertLoRA)]
        assert len(ex) == 4 and ex[0].lora_A.shape[0] == (1 if shared else 4)
        assert not model.decoder.layers[0].mlp.experts.linear_fc1.weight.requires_grad and ex[0].lora_A.requires_grad
        # gradients reach the adapters through the whole model
        with torch.no_grad():
            for a in ex:
                a.lora_B.normal_(0, 0.3)
        h, _ = model(t, pos, cu, 14)
        h.float().pow(2).sum().backward()
        assert all(a.lora_A.grad is not None and a.lora_B.grad.abs().sum() > 0 for a in ex)
        # adapted experts == experts with the deltas merged (fixed routing: the expert module is called directly)
        experts = model.decoder.layers[0].mlp.experts
        offsets = torch.tensor([0, 5, 5, 12, 16], dtype=torch.int32)
        x_perm = torch.randn(16, 64)
        with torch.no_grad():
            ref = experts(x_perm, offsets)
            saved = [(a, a.lora_B.detach().clone()) for a in ex]
            for a in ex:
                a.lora_B.zero_()
            plain = experts(x_perm, offsets)
            for a, b in saved:
                a.lora_B.copy_(b)
            merge_lora_(model)
            for a in ex:
                a.lora_B.zero_()
            merged = experts(x_perm, offsets)
        # expert GEMM outputs are rounded to bf16, so "equal" is to bf16 resolution - far below what the adapters change
        err, effect = float((ref - merged).abs().max()), float((ref - plain).abs().max())
        assert err < 0.03 * max(1.0, float(ref.abs().max())) and effect > 5 * err, (err, effect)


def test_user_post_advantage_hook_edits_samples_and_reports_metrics(tmp_path):
    """``ppo.post_advantage_py_path``: a user function sees the samples once the advantages exist, may change them and
    returns metrics that land in the step's metrics."""
    hook = tmp_path / "post_adv.py"
    hook.write_text(
        "def halve(samples, ppo_cfg, dp_group):\n"
        "    tot = 0.0\n"
        "    for s in samples:\n"
        "        tot += float(s['advantages'].abs().sum())\n"
        "        s['advantages'] = s['advantages'] * 0.0\n"
        "    return samples, {'post-adv/abs_sum': tot}\n")
    cfg = make_cfg(post_advantage_py_path=str(hook), post_advantage_fn_name="halve", grpo_kl_loss_beta=0.0)
    tr = GrpoTrainer(cfg, model_cfg=get_preset("tiny_llama", dtype="float32"), reward_fn=reward_has_small_token).setup()
    m = tr.step([[5, 6, 7, 8, 9], [10, 11, 12], [13, 14, 15, 16], [20, 21]])
    assert m["post-adv/abs_sum"] > 0
    assert m["policy/grad_norm"] < 1e-7     # zeroed advantages and no KL term: nothing to learn from
    assert all(float(s["advantages"].abs().sum()) == 0.0 for s in tr.last_samples)


def test_separate_rollout_copy_is_freed_after_rollout_and_rebuilt_at_resync():
    """``share_rollout_weights=false`` with ``release_rollout_weights``: the engine owns a copy only while it serves;
    every resync rebuilds it through the staging bucket from the trained weights (the library baseline's hand-over)."""
    torch.manual_seed(0)
    cfg = make_cfg()
    cfg.policy.share_rollout_weights = False
    cfg.policy.release_rollout_weights = True
    tr = GrpoTrainer(cfg, model_cfg=get_preset("tiny_llama", dtype="float32"), reward_fn=reward_has_small_token).setup()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 1024, (8,), generator=g).tolist() for _ in range(4)]
    p = tr.policy.model.decoder.layers[0].self_attention.linear_qkv.weight
    for _ in range(2):
        m = tr.step(prompts)
        assert m["policy/grad_norm"] > 0
        w = tr.engine.w.layers[0].qkv_w           # rebuilt by the resync at the end of the step
        assert w.data_ptr() != p.data_ptr() and torch.equal(w, p.detach())
    tr.rollout(prompts)
    assert tr.engine.w is None                    # dropped with the KV cache when the rollout ends
    tr.update_weights()
    s = tr.rollout(prompts)[0]
    assert len(s["tokens"]) > s["prompt_length"]


def test_reference_and_policy_weights_swap_to_host_and_back():
    """``policy.offload_ref_model``: the reference policy holds no device storage outside its forward pass and the
    step's numbers do not change; ``offload_model`` / ``onload_model`` round-trip the trainable weights."""
    prompts = [torch.randint(3, 1024, (8,), generator=torch.Generator().manual_seed(5)).tolist() for _ in range(4)]
    out = []
    for swap in (False, True):
        torch.manual_seed(0)
        cfg = make_cfg(grpo_kl_loss_beta=0.05)
        cfg.policy.offload_ref_model = swap
        tr = GrpoTrainer(cfg, model_cfg=get_preset("tiny_llama", dtype="float32"),
                         reward_fn=reward_has_small_token).setup()
        ms = [tr.step(prompts) for _ in range(2)]
        out.append([(m["policy/grad_norm"], m["ppo-metrics/kl_to_ref"]) for m in ms])
        if swap:
            assert all(p.numel() == 0 for p in tr.policy.ref_model.parameters())
            before = [p.detach().clone() for p in tr.policy.model.parameters()]
            tr.offload_model()
            assert all(p.numel() == 0 for p in tr.policy.model.parameters()) and tr.engine.w is None
            tr.onload_model()
            assert tr.engine.w.layers[0].qkv_w.data_ptr() == \
                tr.policy.model.decoder.layers[0].self_attention.linear_qkv.weight.data_ptr()
            for a, p in zip(before, tr.policy.model.parameters()):
                assert torch.equal(a, p)
            assert tr.step(prompts)["policy/grad_norm"] > 0
    assert out[0] == out[1] and out[0][1][1] > 0
