"""Multi-token prediction blocks: shifted labels and masks inside packed sequences, SFT training of trunk + blocks,
online training of the blocks during an RL update without touching the trunk's gradient."""
import dataclasses

import torch

from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, PpoConfig, TrainingConfig
from gcore_b200.engine.train_engine import TrainingEngine
from gcore_b200.models.config import get_preset


def _engine(mtp=2, online=False, ppo=False, lr=1e-3):
    mc = dataclasses.replace(get_preset("tiny_llama", dtype="float32"), mtp_num_layers=mtp, mtp_loss_scaling_factor=0.3)
    pc = PolicyConfig(recompute="none", without_ref=True)
    oc = OptimizerConfig(lr=lr, lr_decay_style="constant", weight_decay=0.0, max_grad_norm=0.0)
    tc = TrainingConfig(train_mbs=4, train_gbs=4, online_mtp_sft=online)
    eng = TrainingEngine(pc, oc, tc, ppo_cfg=PpoConfig() if ppo else None, model_cfg=mc)
    eng.setup_model_and_get_optimizer(seed=7)
    return eng


def _samples(n=4, L=48, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for i in range(n):
        t = torch.randint(3, 1024, (L - 4 * i,), generator=g)
        m = torch.zeros(L - 4 * i)
        m[10:L - 4 * i - 1] = 1.0
        out.append({"tokens": t, "loss_mask": m, "mask": m.clone(), "prompt_length": 11,
                    "sequence_length": L - 4 * i})
    return out


def test_shifted_targets_and_masks_follow_the_definition():
    eng = _engine(mtp=2)
    samples = _samples()
    mb = eng._pack(samples, [0, 1, 2, 3], ())
    model = eng.model
    with torch.no_grad():
        hidden, _ = eng._hidden(model, mb)
        outs, _ = model.mtp_hidden(hidden, mb.tokens, mb.position_ids, mb.cu_seqlens, mb.max_seqlen, mb.seq_ids.long())
    assert len(outs) == 2
    cu = mb.cu_seqlens.tolist()
    for k, (h, valid) in enumerate(outs, start=1):
        assert h.shape == hidden.shape
        want = torch.zeros_like(valid)
        for a, b in zip(cu[:-1], cu[1:]):
            want[a:max(a, b - k)] = True          # the last k positions of a sequence look beyond it
        assert torch.equal(valid[:cu[-1]], want[:cu[-1]])
    # depth-1 hidden at t depends on token t + 1 (its embedding input) but not on token t + 2
    toks2 = mb.tokens.clone()
    toks2[7] = (toks2[7] + 1) % 1024
    with torch.no_grad():
        outs2, _ = model.mtp_hidden(hidden, toks2, mb.position_ids, mb.cu_seqlens, mb.max_seqlen, mb.seq_ids.long())
    d = (outs2[0][0] - outs[0][0]).abs().sum(-1)
    assert d[6] > 0 and d[:6].max() == 0          # causal: position 6 reads token 7, earlier positions do not


def test_sft_trains_trunk_and_prediction_blocks():
    torch.manual_seed(0)
    eng = _engine(mtp=2)
    names = [n for n, _ in eng.model.named_parameters()]
    assert any(n.startswith("mtp.layers.1.eh_proj") for n in names)
    before = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    hist = [eng.finetune_step(_samples()) for _ in range(10)]
    assert hist[0]["mtp_loss"] > 6.5 and hist[-1]["mtp_loss"] < hist[0]["mtp_loss"] - 0.5
    assert hist[-1]["lm_loss"] < hist[0]["lm_loss"] - 0.5
    moved = {n for n, p in eng.model.named_parameters() if not torch.equal(p, before[n])}
    assert "mtp.layers.0.eh_proj.weight" in moved and "mtp.layers.1.transformer_layer.mlp.linear_fc1.weight" in moved
    assert "decoder.layers.0.self_attention.linear_qkv.weight" in moved


def test_online_training_during_rl_leaves_the_trunk_gradient_alone():
    def rl_samples():
        out = _samples()
        g = torch.Generator().manual_seed(9)
        for s in out:
            n = s["tokens"].numel()
            s["advantages"] = torch.randn(n, generator=g) * s["mask"]
            s["logprobs"] = -torch.rand(n, generator=g) * 3
        return out

    grads = {}
    for online in (False, True):
        torch.manual_seed(0)
        eng = _engine(mtp=1, online=online, ppo=True, lr=0.0)
        eng.ppo_cfg.skip_prev_logps = False
        eng.ppo_cfg.grpo_kl_loss_beta = 0.0
        m = eng.rl_train_actor(rl_samples())
        grads[online] = {n: p.main_grad.detach().clone() for n, p in eng.model.named_parameters()
                         if getattr(p, "main_grad", None) is not None}
        if online:
            assert m["ppo-metrics/mtp_loss"] > 6.0
        else:
            assert "ppo-metrics/mtp_loss" not in m
    trunk = "decoder.layers.1.mlp.linear_fc2.weight"
    assert torch.allclose(grads[True][trunk], grads[False][trunk], atol=1e-7)
    assert grads[False]["mtp.layers.0.eh_proj.weight"].abs().max() == 0
    assert grads[True]["mtp.layers.0.eh_proj.weight"].abs().max() > 0
    # the shared embedding and output matrices do receive the blocks' gradient
    assert not torch.allclose(grads[True]["embedding.word_embeddings.weight"],
                              grads[False]["embedding.word_embeddings.weight"])


def test_checkpoints_carry_the_prediction_blocks(tmp_path):
    """torch_dist save / load and the Hugging Face export / import keep the blocks (stored as layers behind the last
    decoder layer, the DeepSeek-V3 convention)."""
    import os
    from safetensors.torch import load_file
    from gcore_b200.checkpoint import hf
    from gcore_b200.checkpoint.torch_dist import load_checkpoint, save_checkpoint
    torch.manual_seed(0)
    eng = _engine(mtp=1)
    eng.finetune_step(_samples())
    want = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    save_checkpoint(eng, str(tmp_path / "ck"), 1)
    hf.save_hf(eng, str(tmp_path / "hf"))
    sd = {}
    for f in os.listdir(tmp_path / "hf"):
        if f.endswith(".safetensors"):
            sd.update(load_file(str(tmp_path / "hf" / f)))
    L = eng.model_cfg.num_layers
    for k in (f"model.layers.{L}.eh_proj.weight", f"model.layers.{L}.enorm.weight", f"model.layers.{L}.hnorm.weight",
              f"model.layers.{L}.shared_head.norm.weight", f"model.layers.{L}.self_attn.q_proj.weight",
              f"model.layers.{L}.mlp.down_proj.weight"):
        assert k in sd, k
    for loader in ("dist", "hf"):
        other = _engine(mtp=1)
        other.model.reset_parameters(seed=99)
        assert not torch.equal(dict(other.model.named_parameters())["mtp.layers.0.eh_proj.weight"],
                               want["mtp.layers.0.eh_proj.weight"])
        if loader == "dist":
            load_checkpoint(other, str(tmp_path / "ck"), 1)
        else:
            hf.load_hf(other, str(tmp_path / "hf"))
        for n, p in other.model.named_parameters():
            assert torch.equal(p, want[n]), (loader, n)
