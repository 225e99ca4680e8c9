"""Tensor / expert parallel parity on CPU (gloo, world 2) against the single-process model, checkpoint resharding
(saved at TP=2, loaded at TP=1), independent read-back of the torch_dist files by torch.distributed.checkpoint, and the
HF safetensors export."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "workers"))


def _spawn(mode, out, extra=(), port="29541", world=2):
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT=port, OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "workers", "parallel_worker.py"), mode,
                               str(out), *extra], env=dict(env, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r)))
             for r in range(world)]
    for p in procs:
        assert p.wait(timeout=900) == 0


def test_tp2_sp_matches_single_process_and_checkpoint_reshards(tmp_path):
    import parallel_worker as pw
    from gcore_b200.models.config import get_preset
    out = tmp_path / "tp.json"
    _spawn("tp", out, [str(tmp_path)])
    got = json.load(open(out))
    mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
    e = pw.engine(mcfg, 1)
    ref = [e.finetune_step(pw.samples(8, 50 + s))["lm_loss"] for s in range(4)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 5e-4, (ref, got)
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 5e-3
    # the TP=2 checkpoint loads into a TP=1 engine and reproduces the trained weights and optimizer state
    from gcore_b200.checkpoint.torch_dist import CheckpointReader, load_checkpoint
    e2 = pw.engine(mcfg, 1)
    assert load_checkpoint(e2, str(tmp_path / "ckpt")) == 4
    for (n, p), (_, q) in zip(e.model.named_parameters(), e2.model.named_parameters()):
        assert torch.allclose(p, q, atol=2e-4), n
    for a, b in zip(e.optimizer.shards, e2.optimizer.shards):
        assert torch.allclose(a["m"], b["m"], atol=1e-5) and torch.allclose(a["v"], b["v"], atol=1e-6)
    assert e2.optimizer.step_count == 4
    # Megatron-style keys: stacked layer axis, interleaved QKV, fc1 = [gate; up]
    rd = CheckpointReader(str(tmp_path / "ckpt" / "iter_0000004"))
    keys = set(rd.keys())
    assert "decoder.layers.self_attention.linear_qkv.weight" in keys
    assert "decoder.layers.self_attention.linear_qkv.layer_norm_weight" in keys
    assert "optimizer.state.exp_avg.decoder.layers.mlp.linear_fc1.weight" in keys
    qkv = rd.full_tensor("decoder.layers.self_attention.linear_qkv.weight")
    assert tuple(qkv.shape) == (2, (4 + 2 * 2) * 64, 256)
    for f in ("common.pt", "metadata.json", ".metadata"):
        assert os.path.exists(tmp_path / "ckpt" / "iter_0000004" / f)
    # independent reader: torch.distributed.checkpoint itself
    import torch.distributed.checkpoint as dcp
    sd = {"decoder.layers.self_attention.linear_qkv.weight": torch.zeros_like(qkv)}
    dcp.load(sd, checkpoint_id=str(tmp_path / "ckpt" / "iter_0000004"), no_dist=True)
    assert torch.equal(sd["decoder.layers.self_attention.linear_qkv.weight"], qkv)
    # HF export gathered over TP equals the single-process weights under HF names
    from gcore_b200.checkpoint.hf import read_hf_dir
    from gcore_b200.checkpoint.layout import export_full_weights
    hf = read_hf_dir(str(tmp_path / "hf"))
    mine = dict(export_full_weights(e))
    assert set(hf) == set(mine)
    for k in mine:
        assert torch.allclose(hf[k].float(), mine[k].float(), atol=2e-4), k
    assert hf["model.layers.0.self_attn.k_proj.weight"].shape == (2 * 64, 256)
    assert hf["model.layers.1.mlp.gate_proj.weight"].shape == (688, 256)


def test_ep2_matches_single_process(tmp_path):
    import parallel_worker as pw
    from gcore_b200.models.config import ModelConfig
    out = tmp_path / "ep.json"
    _spawn("ep", out, port="29543")
    got = json.load(open(out))
    mcfg = ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=128, num_attention_heads=4, num_kv_heads=2,
                       ffn_hidden_size=256, vocab_size=512, num_experts=8, moe_top_k=2, moe_ffn_hidden_size=64,
                       moe_aux_loss_coef=1e-2, dtype="float32", qk_layernorm=True)
    e = pw.engine(mcfg, 1)
    ref = [e.finetune_step(pw.samples(8, 70 + s, vocab=512))["lm_loss"] for s in range(3)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 2e-3, (ref, got)
    # the gradient norm pins the scale of the expert gradients (a factor of the expert-parallel size on them moves it
    # by 3 % here, while Adam hides such a factor from the losses)
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 5e-3, (float(e.optimizer.last_grad_norm), got)


@pytest.mark.parametrize("mode,port", [("tp_lora", "29569"), ("tp_lora_moe", "29571")])
def test_tp2_lora_matches_single_process(tmp_path, mode, port):
    """LoRA under tensor + sequence parallelism (dense model; MoE model with adapters on the router and a shared
    adapter on the experts): losses, gradient norm, and the replicated adapter halves stay identical on both ranks."""
    import dataclasses
    import parallel_worker as pw
    from gcore_b200.models.config import get_preset
    out = tmp_path / f"{mode}.json"
    _spawn(mode, out, port=port)
    got = json.load(open(out))
    if mode == "tp_lora":
        e, vocab = pw.lora_engine(get_preset("tiny_llama", dtype="float32", qkv_bias=True), 1), 1024
    else:
        e = pw.lora_engine(dataclasses.replace(pw.MOE_CFG, moe_aux_loss_coef=0.0), 1,
                           ["linear_qkv", "linear_proj", "linear_fc1", "linear_fc2", "router"])
        vocab = 512
    ref = [e.finetune_step(pw.samples(8, 50 + s, vocab=vocab))["lm_loss"] for s in range(3)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 5e-4, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 2e-3, (float(e.optimizer.last_grad_norm), got)
    assert got["replicated_halves_equal"]


@pytest.mark.parametrize("mode,port", [("tp_mla", "29573"), ("tp_mla_lora", "29575")])
def test_tp2_latent_attention_matches_single_process(tmp_path, mode, port):
    """Latent attention under tensor parallelism, plain and with adapters on all five projections: the replicated
    down-projections (and their adapters) collect their gradient from both ranks' heads."""
    import parallel_worker as pw
    out = tmp_path / f"{mode}.json"
    _spawn(mode, out, port=port)
    got = json.load(open(out))
    if mode == "tp_mla":
        e = pw.engine(pw.MLA_CFG, 1)
    else:
        e = pw.lora_engine(pw.MLA_CFG, 1, ["linear_q_down_proj", "linear_q_up_proj", "linear_kv_down_proj",
                                           "linear_kv_up_proj", "linear_proj"])
    ref = [e.finetune_step(pw.samples(8, 50 + s, vocab=512))["lm_loss"] for s in range(3)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 5e-4, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 2e-3, (float(e.optimizer.last_grad_norm), got)


def test_pp2_with_moe_layers_on_both_stages_matches_single_process(tmp_path):
    """The load-balance loss of MoE layers on a stage that does not evaluate the loss enters the backward with the
    weight the last stage gives its own (1 / (micro-batches x data-parallel size))."""
    import dataclasses
    import parallel_worker as pw
    out = tmp_path / "ppmoe.json"
    _spawn("pp_moe", out, port="29579")
    got = json.load(open(out))
    e = pw.engine(dataclasses.replace(pw.MOE_CFG, num_layers=4), 1)
    ref = [e.finetune_step(pw.samples(8, 130 + s, vocab=512))["lm_loss"] for s in range(3)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 3e-4, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 3e-4, (float(e.optimizer.last_grad_norm), got)


def test_cp2_latent_attention_matches_single_process(tmp_path):
    import parallel_worker as pw
    out = tmp_path / "cpmla.json"
    _spawn("cp_mla", out, port="29581")
    got = json.load(open(out))
    e = pw.engine(pw.MLA_CFG, 1)
    ref = [e.finetune_step(pw.samples(8, 170 + s, vocab=512))["lm_loss"] for s in range(3)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 3e-4, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 3e-4, (float(e.optimizer.last_grad_norm), got)


def test_cp2_multi_token_prediction_matches_single_process(tmp_path):
    import parallel_worker as pw
    out = tmp_path / "cpmtp.json"
    _spawn("cp_mtp", out, port="29582")
    got = json.load(open(out))
    e = pw.engine(pw.NOSP_CFG, 1)
    ref = [e.finetune_step(pw.samples(8, 180 + s))["lm_loss"] for s in range(3)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 3e-4, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 3e-4, (float(e.optimizer.last_grad_norm), got)


@pytest.mark.parametrize("mode", ["dpo_cp", "dpo_dp", "dpo_tp"])
def test_two_rank_dpo_matches_single_process(tmp_path, mode):
    import parallel_worker as pw
    from gcore_b200.models.config import get_preset
    from gcore_b200.trainer.preference_trainers import dpo_step
    out = tmp_path / f"{mode}.json"
    _spawn(mode, out, port="29583")
    got = json.load(open(out))
    e = pw.engine(get_preset("tiny_llama", dtype="float32", qkv_bias=True), 1)
    ref = [dpo_step(e, pw.samples(4, 200 + s), pw.samples(4, 300 + s), beta=0.5, reference_free=True, sft_coef=0.1)
           for s in range(2)]
    for r, a, b in zip(ref, got["losses"], got["grad_norms"]):
        assert abs(r["dpo/loss"] - a) < 1e-3 * abs(r["dpo/loss"]), (ref, got)
        assert abs(r["grad_norm"] - b) < 1e-3 * r["grad_norm"], (ref, got)


def test_cp2_reward_model_and_embedding_steps_match_single_process(tmp_path):
    import parallel_worker as pw
    out = tmp_path / "rmcp.json"
    _spawn("rm_cp", out, port="29584")
    got = json.load(open(out))["runs"]
    ref = pw.preference_run()["runs"]
    for (l0, g0), (l1, g1) in zip(ref, got):
        assert abs(l0 - l1) < 1e-3 * max(abs(l0), 1e-2), (ref, got)
        assert abs(g0 - g1) < 1e-3 * max(g0, 1e-2), (ref, got)


def test_pp2_critic_trains_and_scores_like_a_single_process(tmp_path):
    import parallel_worker as pw
    out = tmp_path / "ppvalue.json"
    _spawn("pp_value", out, port="29585")
    got = json.load(open(out))
    ref = pw.value_run()
    for k in ref:
        assert abs(ref[k] - got[k]) < 1e-3 * max(abs(ref[k]), 1e-1), (k, ref, got)


def test_tp2_without_sequence_parallel_matches_single_process(tmp_path):
    """Every TP rank holds all tokens: the hidden state in front of the vocabulary-parallel head sums the ranks'
    gradient parts, the per-head q/k gains sum theirs, and the replicated multi-token-prediction branch hands the
    trunk its gradient once."""
    import parallel_worker as pw
    out = tmp_path / "nosp.json"
    _spawn("tp_nosp", out, port="29580")
    got = json.load(open(out))
    e = pw.engine(pw.NOSP_CFG, 1)
    ref = [e.finetune_step(pw.samples(8, 150 + s))["lm_loss"] for s in range(3)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 3e-4, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 3e-4, (float(e.optimizer.last_grad_norm), got)


def test_moe_under_tensor_parallelism_demands_sequence_parallel():
    from gcore_b200.models.gpt import GPTModel
    import parallel_worker as pw
    with pytest.raises(ValueError, match="sequence_parallel"):
        GPTModel(pw.MOE_CFG, tp_size=2, sequence_parallel=False, device="meta")


def test_tp2_critic_matches_single_process(tmp_path):
    """Value head under tensor parallelism: same loss and gradient norm as one process (the replicated head's
    gradient into the gathered hidden states is not added up over the TP ranks)."""
    import parallel_worker as pw
    out = tmp_path / "tpvalue.json"
    _spawn("tp_value", out, port="29577")
    got = json.load(open(out))
    ref = pw.value_engine(1).rl_train_value(pw.value_samples())
    assert abs(ref["value/loss"] - got["value/loss"]) < 1e-5
    assert abs(ref["value/grad_norm"] - got["value/grad_norm"]) < 2e-3, (ref, got)


def test_tp2_multi_token_prediction_matches_single_process(tmp_path):
    import dataclasses
    import parallel_worker as pw
    from gcore_b200.models.config import get_preset
    out = tmp_path / "tpmtp.json"
    _spawn("tp_mtp", out, port="29567")
    got = json.load(open(out))
    mcfg = dataclasses.replace(get_preset("tiny_llama", dtype="float32", qkv_bias=True), mtp_num_layers=2,
                               mtp_loss_scaling_factor=0.3)
    e = pw.engine(mcfg, 1)
    ref = [e.finetune_step(pw.samples(8, 50 + s)) for s in range(3)]
    for r, a, b in zip(ref, got["losses"], got["mtp"]):
        assert abs(r["lm_loss"] - a) < 5e-4 and abs(r["mtp_loss"] - b) < 5e-4, (ref, got)
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 5e-3


def test_tp2_with_unsplit_experts_matches_single_process(tmp_path):
    """MoE under tensor parallelism without expert parallelism: the TP ranks hold whole experts and see different
    tokens, so their expert gradients are reduced over a group that contains both (losses, gradient norm and the
    updated expert weights equal the single-process run; the two ranks' expert weights stay identical)."""
    import parallel_worker as pw
    out = tmp_path / "tpmoe.json"
    _spawn("tp_moe", out, port="29561")
    got = json.load(open(out))
    e = pw.engine(pw.MOE_CFG, 1)
    ref = [e.finetune_step(pw.samples(8, 70 + s, vocab=512))["lm_loss"] for s in range(4)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 2e-3, (ref, got["losses"])
    assert got["expert_weights_equal"]
    # the gradient norm pins the scale of the expert gradients (summed over the two ranks, not averaged)
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 5e-3


@pytest.mark.parametrize("mode,port", [("tp2ep2", "29563"), ("ep2dp4", "29565")])
def test_four_rank_expert_layouts_match_single_process(tmp_path, mode, port):
    """Experts split over two ranks and replicated over two more, under tensor parallelism 2 x data parallelism 2 and
    under data parallelism 4: losses and the global gradient norm of the single-process run (the norm pins the scale
    of the expert gradients across the expert-data-parallel replicas)."""
    import parallel_worker as pw
    out = tmp_path / f"{mode}.json"
    _spawn(mode, out, port=port, world=4)
    got = json.load(open(out))
    assert got["edp"] == 2
    e = pw.engine(pw.MOE_CFG, 1)
    ref = [e.finetune_step(pw.samples(8, 70 + s, vocab=512))["lm_loss"] for s in range(2)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 2e-3, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 5e-3, (float(e.optimizer.last_grad_norm), got)


def test_cp2_matches_single_process(tmp_path):
    """Context parallel over the packed token stream (full + sliding-window-with-sink layers): same losses, gradient
    norm and per-token log-probs as one process."""
    import parallel_worker as pw
    from gcore_b200.models.config import get_preset
    out = tmp_path / "cp.json"
    _spawn("cp", out, port="29545")
    got = json.load(open(out))
    mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True, sliding_window=16, sliding_window_pattern=[0, 1],
                      attention_sinks=True)
    e = pw.engine(mcfg, 1)
    ref = [e.finetune_step(pw.samples(8, 90 + s))["lm_loss"] for s in range(4)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 5e-4, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 5e-3
    lp = e.compute_log_probs(pw.samples(3, 99))
    for a, b in zip(lp, got["logprobs"]):
        assert torch.allclose(a["logprobs"], torch.tensor(b), atol=2e-4)


def test_cp_plan_covers_every_key_row_once():
    from gcore_b200.parallel.cp import plan_cp
    cu = [0, 37, 120, 121, 300, 512]
    cp, s = 4, 128
    for window in (0, 16):
        plans = [plan_cp(cu, s, cp, r, window) for r in range(cp)]
        for r, p in enumerate(plans):
            assert p.cu_q[-1] == s and p.cu_k[-1] == p.rows
            assert sum(n for *_, n in p.pulls) == p.rows
            # every returned range lands inside the owner's chunk and matches what the source gathered
            for src, src_row, dst_row, n in p.returns:
                assert 0 <= dst_row and dst_row + n <= s
                assert plans[src].k0 + src_row == r * s + dst_row
        if window:
            assert all(p.k0 >= r * s - (window - 1) for r, p in enumerate(plans))


def test_pp2_1f1b_matches_single_process(tmp_path):
    """Two pipeline stages (1F1B over gloo p2p, 4 micro-batches): same losses, gradient norm and log-probs."""
    import parallel_worker as pw
    from gcore_b200.models.config import get_preset
    out = tmp_path / "pp.json"
    _spawn("pp", out, [str(tmp_path)], port="29547")
    got = json.load(open(out))
    mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True, num_layers=4)
    e = pw.engine(mcfg, 1)
    ref = [e.finetune_step(pw.samples(8, 130 + s))["lm_loss"] for s in range(4)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 5e-4, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 5e-3
    lp = e.compute_log_probs(pw.samples(3, 199))
    for a, b in zip(lp, got["logprobs"]):
        assert torch.allclose(a["logprobs"], torch.tensor(b), atol=2e-4)
    # the two-stage checkpoint resumes on two stages ...
    assert abs(got["next_loss"][0] - got["next_loss"][1]) < 1e-5, got["next_loss"]
    # ... and loads into the unpartitioned model: layers are stored under their global index
    from gcore_b200.checkpoint.torch_dist import CheckpointReader, load_checkpoint
    rd = CheckpointReader(str(tmp_path / "ckpt" / "iter_0000004"))
    assert tuple(rd.full_tensor("decoder.layers.mlp.linear_fc2.weight").shape)[0] == 4
    e2 = pw.engine(mcfg, 1)
    e2.setup_model_and_get_optimizer(seed=5)
    assert load_checkpoint(e2, str(tmp_path / "ckpt")) == 4
    for (n, p), (_, q) in zip(e.model.named_parameters(), e2.model.named_parameters()):
        # Adam's first steps move an element by ~lr whatever the size of its gradient, so an element whose gradient
        # is at rounding level may differ by a few lr between the pipelined and the single-process run
        assert float((p - q).abs().mean()) < 2e-5 and float((p - q).abs().max()) < 5e-3, n
    for a, b in zip(e.optimizer.shards, e2.optimizer.shards):
        assert torch.allclose(a["m"], b["m"], atol=1e-5) and torch.allclose(a["v"], b["v"], atol=1e-6)
    nxt = [x.finetune_step(pw.samples(8, 140))["lm_loss"] for x in (e, e2)]
    assert abs(nxt[0] - nxt[1]) < 5e-4 and abs(nxt[0] - got["next_loss"][0]) < 5e-4


def test_pp2_interleaved_virtual_stages_match_single_process(tmp_path):
    """Two stages x two model chunks each (interleaved 1F1B over gloo p2p): same losses, gradient norm and log-probs
    as one process; its checkpoint loads into the unpartitioned model."""
    import parallel_worker as pw
    from gcore_b200.checkpoint.torch_dist import load_checkpoint
    from gcore_b200.models.config import get_preset
    out = tmp_path / "vpp.json"
    _spawn("vpp", out, [str(tmp_path)], port="29549")
    got = json.load(open(out))
    mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True, num_layers=4)
    e = pw.engine(mcfg, 1)
    ref = [e.finetune_step(pw.samples(8, 130 + s))["lm_loss"] for s in range(4)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 5e-4, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 5e-3
    lp = e.compute_log_probs(pw.samples(3, 199))
    for a, b in zip(lp, got["logprobs"]):
        assert torch.allclose(a["logprobs"], torch.tensor(b), atol=2e-4)
    assert abs(got["next_loss"][0] - got["next_loss"][1]) < 1e-5, got["next_loss"]
    e2 = pw.engine(mcfg, 1)
    e2.setup_model_and_get_optimizer(seed=5)
    assert load_checkpoint(e2, str(tmp_path / "ckpt")) == 4
    for (n, p), (_, q) in zip(e.model.named_parameters(), e2.model.named_parameters()):
        assert float((p - q).abs().mean()) < 2e-5 and float((p - q).abs().max()) < 5e-3, n


def test_expert_parallel_rollout_engines_stay_in_lockstep(tmp_path):
    """Two rollout engines share their experts (EP = 2) and get unequal work; the one that finishes early keeps
    stepping with an inactive batch.  Both must reproduce the full-recompute greedy decode of the EP = 1 model."""
    from test_rollout_cpu import naive_greedy
    from gcore_b200.models.config import ModelConfig
    from gcore_b200.models.gpt import GPTModel
    out = tmp_path / "ep_rollout.json"
    _spawn("ep_rollout", out, port="29551")
    mcfg = ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=128, num_attention_heads=4, num_kv_heads=2,
                       ffn_hidden_size=256, vocab_size=512, num_experts=8, moe_top_k=2, moe_ffn_hidden_size=64,
                       dtype="float32", qk_layernorm=True)
    torch.manual_seed(0)
    model = GPTModel(mcfg, recompute="none")
    model.reset_parameters(21)
    model.eval()
    for rank, n_new in ((0, 9), (1, 3)):
        got = json.load(open(f"{out}.{rank}"))
        assert len(got["prompts"]) == (3 if rank == 0 else 1)
        for p, toks, lps in zip(got["prompts"], got["tokens"], got["logprobs"]):
            ref_t, ref_lp = naive_greedy(model, p, n_new)
            assert toks == ref_t, (rank, toks, ref_t)
            assert max(abs(a - b) for a, b in zip(lps, ref_lp)) < 1e-3


def test_grpo_steps_with_expert_parallel_trainer_and_rollout(tmp_path):
    """GRPO on two ranks that split the experts (trainer and colocated rollout engine), different prompts and stop
    tokens per rank: steps complete, the first-epoch ratio is 1 and rollout log-probs agree with the trainer's."""
    out = tmp_path / "ep_grpo.json"
    _spawn("ep_grpo", out, port="29553")
    got = json.load(open(out))["ranks"]
    assert len(got) == 2
    for r in got:
        assert all(g > 0 for g in r["grad_norm"]) and all(abs(x - 1.0) < 1e-3 for x in r["ratio"]), got
        assert r["logprob_gap"] < 2e-3, got


def test_stage_layer_ranges():
    from gcore_b200.parallel.pp import stage_layer_range
    assert [stage_layer_range(12, 4, s) for s in range(4)] == [(0, 3), (3, 6), (6, 9), (9, 12)]
    assert [stage_layer_range(10, 4, s, 2, 2) for s in range(4)] == [(0, 2), (2, 5), (5, 8), (8, 10)]


def test_fsdp2_engine_matches_single_process_and_resumes(tmp_path):
    """ZeRO-3 engine on 2 gloo ranks: parameters are really sharded, losses and gradient norm match the ZeRO-1 engine
    in one process, and a DCP checkpoint restores a differently initialised engine to the same next step."""
    import parallel_worker as pw
    from gcore_b200.models.config import get_preset
    out = tmp_path / "fsdp.json"
    _spawn("fsdp", out, [str(tmp_path / "ck")], port="29549")
    got = json.load(open(out))
    assert got["local_frac"] < 0.6
    mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
    e = pw.engine(mcfg, 1)
    ref = [e.finetune_step(pw.samples(8, 150 + s))["lm_loss"] for s in range(4)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 1e-3, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 1e-2
    assert abs(got["next_loss"][0] - got["next_loss"][1]) < 1e-5


def test_interleaved_schedule_is_deadlock_free_and_exact():
    """The interleaved 1F1B schedule driven by threads over in-memory FIFOs (one per channel and direction, blocking
    receives with a timeout): every (stages, chunks, micro-batches) case must finish and give the gradients of the
    sequential model; messages must arrive in the order the receiver expects them."""
    import queue
    import threading
    from gcore_b200.parallel.pp import forward_backward_interleaved

    class FakeComm:
        def __init__(self, rank, size, chans):
            self.rank, self.size, self.chans = rank, size, chans

        def send_forward(self, t):
            self.chans[("f", self.rank, (self.rank + 1) % self.size)].put(t.clone())

        def send_backward(self, t):
            self.chans[("b", self.rank, (self.rank - 1) % self.size)].put(t.clone())

        def recv_forward(self, shape, dtype, device):
            return self.chans[("f", (self.rank - 1) % self.size, self.rank)].get(timeout=20)

        def recv_backward(self, shape, dtype, device):
            return self.chans[("b", (self.rank + 1) % self.size, self.rank)].get(timeout=20)

        def drain(self):
            pass

    for P, V, M in ((2, 2, 4), (2, 2, 2), (2, 3, 6), (4, 2, 8), (4, 2, 4), (3, 2, 5), (4, 3, 12), (2, 1, 3)):
        torch.manual_seed(P * 100 + V * 10 + M)
        w = [[torch.randn(3, requires_grad=True) for _ in range(V)] for _ in range(P)]  # w[stage][chunk]
        xs = [torch.randn(3) for _ in range(M)]
        # sequential reference: virtual stage order is chunk-major
        ref_loss = 0.0
        for i in range(M):
            h = xs[i]
            for v in range(V):
                for s in range(P):
                    h = torch.tanh(h * w[s][v] + 0.1 * (i + 1))
            ref_loss = ref_loss + h.sum()
        ref = torch.autograd.grad(ref_loss, [t for row in w for t in row])
        for row in w:
            for t in row:
                t.grad = None
        chans = {(c, a, b): queue.Queue() for c in "fb" for a in range(P) for b in range(P)}
        errors, losses = [], []

        def run(s):
            try:
                def forward_step(i, v, x):
                    h = xs[i] if x is None else x
                    return torch.tanh(h * w[s][v] + 0.1 * (i + 1)), None

                def loss_step(i, out, aux):
                    losses.append(float(out.detach().sum()))
                    return out.sum()

                forward_backward_interleaved(FakeComm(s, P, chans), M, V, forward_step, loss_step,
                                             lambda i: ((3,), torch.float32, "cpu"))
            except Exception as e:  # noqa: BLE001
                errors.append((s, repr(e)))

        th = [threading.Thread(target=run, args=(s,)) for s in range(P)]
        for t in th:
            t.start()
        for t in th:
            t.join(60)
        assert not errors and not any(t.is_alive() for t in th), (P, V, M, errors)
        assert all(q.empty() for q in chans.values())
        got = [t.grad for row in w for t in row]
        for a, b in zip(ref, got):
            assert torch.allclose(a, b, atol=1e-5), (P, V, M)
        assert abs(sum(losses) - float(ref_loss)) < 1e-4
