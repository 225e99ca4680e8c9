"""Vision-language model on CPU: the tower's output replaces the image placeholder embeddings, gradients reach both
towers, and a few optimisation steps fit a synthetic image -> label task."""
import torch

from gcore_b200.models.config import get_preset
from gcore_b200.models.vlm import VisionConfig, VLModel


def _batch(model, n_img, seed):
    g = torch.Generator().manual_seed(seed)
    vc = model.vc
    toks, pos, cu, patches, grids, targets = [], [], [0], [], [], []
    for i in range(n_img):
        h, w = (4, 4) if i % 2 == 0 else (2, 6)
        label = int(torch.randint(10, 20, (1,), generator=g))
        img = torch.randn(h * w, vc.patch_dim, generator=g) * 0.1 + (label - 15) * 0.2   # brightness encodes the label
        n_vis = h * w // 4
        seq = [3] + [model.image_token_id] * n_vis + [4, label]
        toks += seq
        pos += list(range(len(seq)))
        cu.append(cu[-1] + len(seq))
        patches.append(img)
        grids.append((h, w))
        targets.append((cu[-1] - 2, label))          # position that predicts the label token
    return (torch.tensor(toks), torch.tensor(pos, dtype=torch.int32), torch.tensor(cu, dtype=torch.int32),
            max(cu[i + 1] - cu[i] for i in range(n_img)), torch.cat(patches), grids, targets)


def test_vlm_forward_backward_and_learning():
    torch.manual_seed(0)
    cfg = get_preset("tiny_llama", dtype="float32")
    vc = VisionConfig(patch_size=2, hidden_size=64, num_layers=2, num_heads=2, ffn_hidden_size=128, max_grid=8)
    model = VLModel(cfg, vc, image_token_id=5)
    model.reset_parameters(1)
    assert model.num_image_tokens([(4, 4), (2, 6)]) == [4, 3]
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    losses = []
    for step in range(30):
        toks, pos, cu, mx, patches, grids, targets = _batch(model, 8, 100 + step % 4)
        hidden, _ = model(toks, pos, cu, mx, vision=(patches, grids))
        logits = hidden @ model.output_weight().t()
        idx = torch.tensor([t[0] for t in targets])
        lab = torch.tensor([t[1] for t in targets])
        loss = torch.nn.functional.cross_entropy(logits[idx].float(), lab)
        opt.zero_grad()
        loss.backward()
        if step == 0:
            assert model.vision.patch_embed.weight.grad.abs().sum() > 0          # gradients reach the vision tower
            assert model.language_model.decoder.layers[0].mlp.linear_fc1.weight.grad.abs().sum() > 0
        opt.step()
        losses.append(float(loss.detach()))
    assert sum(losses[-4:]) / 4 < 0.6 * sum(losses[:4]) / 4, losses
    # without images the wrapper is exactly the text decoder
    toks = torch.tensor([3, 9, 8, 7])
    pos = torch.arange(4, dtype=torch.int32)
    cu = torch.tensor([0, 4], dtype=torch.int32)
    a, _ = model(toks, pos, cu, 4)
    b, _ = model.language_model(toks, pos, cu, 4)
    assert torch.allclose(a, b, atol=1e-6)


def test_vlm_sft_through_the_training_engine():
    """The ZeRO-1 engine trains the vision-language model: samples carry ``pixel_patches`` + ``image_grid`` next to their
    tokens, packing concatenates the images of a micro-batch, and the masked next-token loss falls."""
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    vc = VisionConfig(patch_size=2, hidden_size=64, num_layers=2, num_heads=2, ffn_hidden_size=128, max_grid=8)
    eng = TrainingEngine(PolicyConfig(recompute="none", without_ref=True),
                         OptimizerConfig(lr=3e-3, lr_decay_style="constant", weight_decay=0.0), TrainingConfig(train_mbs=4),
                         model_cfg=get_preset("tiny_llama", dtype="float32"), vision_cfg=vc, image_token_id=5)
    eng.setup_model_and_get_optimizer(seed=2, with_ref=False)

    def samples(seed):
        g = torch.Generator().manual_seed(seed)
        out = []
        for i in range(8):
            label = int(torch.randint(10, 20, (1,), generator=g))
            img = torch.randn(16, vc.patch_dim, generator=g) * 0.1 + (label - 15) * 0.2
            toks = torch.tensor([3] + [5] * 4 + [4, label])
            m = torch.zeros(7)
            m[5] = 1.0            # position 5 (token 4) predicts the label
            out.append({"tokens": toks, "loss_mask": m, "pixel_patches": img, "image_grid": (4, 4)})
        return out

    losses = [eng.finetune_step(samples(200 + s % 4))["lm_loss"] for s in range(30)]
    assert sum(losses[-4:]) / 4 < 0.6 * sum(losses[:4]) / 4, losses
    assert any(n.startswith("vision.") for n, _ in eng.model.named_parameters())


def test_vlm_grpo_step_rolls_out_with_images():
    """GRPO with image prompts: the rollout engine's prefill takes the vision tower's rows at the placeholder tokens
    (its log-probs agree with the trainer's, which re-runs the tower), and the update reaches the vision tower."""
    from test_grpo_cpu import make_cfg, reward_has_small_token
    from gcore_b200.trainer.grpo_trainer import GrpoTrainer
    torch.manual_seed(0)
    vc = VisionConfig(patch_size=2, hidden_size=64, num_layers=2, num_heads=2, ffn_hidden_size=128, max_grid=8)
    tr = GrpoTrainer(make_cfg(), model_cfg=get_preset("tiny_llama", dtype="float32"), reward_fn=reward_has_small_token,
                     vision_cfg=vc, image_token_id=5).setup()
    g = torch.Generator().manual_seed(3)
    prompts = []
    for i in range(4):
        h, w = (4, 4) if i % 2 == 0 else (2, 6)
        n_vis = h * w // 4
        prompts.append({"tokens": [3] + [5] * n_vis + [4, 30 + i],
                        "pixel_patches": torch.randn(h * w, vc.patch_dim, generator=g), "image_grid": (h, w)})
    prompts[3] = [3, 40, 41, 42]  # a text-only prompt in the same batch
    before = tr.policy.model.vision.patch_embed.weight.detach().clone()
    m = tr.step(prompts)
    assert m["policy/grad_norm"] > 0
    assert not torch.equal(before, tr.policy.model.vision.patch_embed.weight)
    s = tr.last_samples[0]
    assert "pixel_patches" in s and "pixel_patches" not in tr.last_samples[-1]
    P, S = s["prompt_length"], s["sequence_length"]
    assert torch.allclose(s["logprobs"][P - 1:S - 1], s["rollout_log_probs"][P - 1:S - 1], atol=2e-3)
    # the images matter: the same tokens without the pixels give other log-probs
    blind = [dict(tokens=s["tokens"], prompt_length=P, sequence_length=S, mask=s["mask"])]
    tr.policy.compute_log_probs(blind, use_ref=False)
    assert not torch.allclose(blind[0]["logprobs"][P - 1:S - 1], s["logprobs"][P - 1:S - 1], atol=1e-3)


def test_vision_policy_from_config():
    from gcore_b200.configs.base import from_dict
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    pc = from_dict(PolicyConfig, {"recompute": "none", "without_ref": True, "image_token_id": 5,
                                  "vision_config": {"patch_size": 2, "hidden_size": 64, "num_layers": 1, "num_heads": 2,
                                                    "ffn_hidden_size": 128, "max_grid": 8}})
    e = TrainingEngine(pc, OptimizerConfig(lr=1e-3), TrainingConfig(train_mbs=2, train_gbs=2),
                       model_cfg=get_preset("tiny_llama", dtype="float32"))
    e.setup_model_and_get_optimizer(seed=1)
    assert isinstance(e.model, VLModel) and e.model.image_token_id == 5 and e.model.vc.num_layers == 1


def test_freeze_flags_select_tower_projector_decoder_router_and_shared_experts():
    """``training.freeze_*``: each flag takes exactly its parameter group out of training."""
    from gcore_b200.configs.base import from_dict
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import ModelConfig
    mc = ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=64, num_attention_heads=2, num_kv_heads=2,
                     ffn_hidden_size=128, vocab_size=128, num_experts=4, moe_top_k=2, moe_ffn_hidden_size=32,
                     moe_shared_expert_ffn=32, dtype="float32")

    def frozen(**flags):
        pc = from_dict(PolicyConfig, {"recompute": "none", "without_ref": True, "image_token_id": 5,
                                      "vision_config": {"patch_size": 2, "hidden_size": 64, "num_layers": 1,
                                                        "num_heads": 2, "ffn_hidden_size": 128, "max_grid": 8}})
        e = TrainingEngine(pc, OptimizerConfig(lr=1e-3), TrainingConfig(train_mbs=2, train_gbs=2, **flags), model_cfg=mc)
        e.setup_model_and_get_optimizer(seed=1)
        names = [n for n, _ in e.model.named_parameters()]
        return names, {n for n, p in e.model.named_parameters() if not p.requires_grad}

    names, f = frozen()
    assert not f
    names, f = frozen(freeze_vit=True)
    assert f == {n for n in names if n.startswith("vision.") and "merge_fc" not in n} and f
    names, f = frozen(freeze_projector=True)
    assert f == {n for n in names if n.startswith("vision.merge_fc")} and len(f) >= 2
    names, f = frozen(freeze_llm=True)
    assert f == {n for n in names if not n.startswith("vision.")}
    names, f = frozen(freeze_moe_router=True, freeze_moe_shared_experts=True)
    assert f == {n for n in names if ".router." in n or ".shared_experts." in n} and \
        any(".router." in n for n in f) and any(".shared_experts." in n for n in f)
