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


def test_qwen3_vl_rope_index_video_frames_and_deepstack():
    """Multi-axis position ids (text / image / video blocks), interleaved frequency assignment, per-frame attention
    over video patch volumes and intermediate vision features joining the first decoder layers."""
    from gcore_b200.models.config import ModelConfig
    from gcore_b200.models.qwen3_vl import Qwen3VLModel, get_rope_index
    from gcore_b200.models.vlm import VisionConfig
    from gcore_b200.ops.fused import mrope_tables, rope_ref
    IMG, VID = 500, 501
    # text(2) image 4x4 -> 4 tokens, text(1), video (t=2, 4x2) -> 2 * 2 * 1 = 4 tokens, text(2)
    toks = [5, 6] + [IMG] * 4 + [7] + [VID] * 4 + [8, 9]
    pos, delta = get_rope_index(toks, [(1, 4, 4)], IMG, VID, 2, [(2, 4, 2)])
    assert pos[:2].tolist() == [[0, 0, 0], [1, 1, 1]]
    assert pos[2:6].tolist() == [[2, 2, 2], [2, 2, 3], [2, 3, 2], [2, 3, 3]]          # one frame, 2 x 2 merged grid
    assert pos[6].tolist() == [4, 4, 4]                                                # text resumes after max + 1
    assert pos[7:11].tolist() == [[5, 5, 5], [5, 6, 5], [6, 5, 5], [6, 6, 5]]          # two frames, 2 x 1 grid each
    assert pos[11].tolist() == [7, 7, 7] and delta == 9 - len(toks)
    # text-only streams rotate exactly like plain 1-D rotary embedding
    p1 = torch.arange(6)
    x = torch.randn(6, 2, 16)
    tab = mrope_tables(p1[:, None].expand(6, 3), 10000.0, 16, (4, 2, 2), True)
    assert torch.allclose(rope_ref(x, tab, 10000.0, 16), rope_ref(x, p1, 10000.0, 16), atol=1e-6)
    # interleaved vs chunked assignment differ once the axes differ
    p3 = torch.tensor([[3, 1, 2]])
    ci, _ = mrope_tables(p3, 10000.0, 16, (4, 2, 2), True)
    cc, _ = mrope_tables(p3, 10000.0, 16, (4, 2, 2), False)
    inv = 10000.0 ** (-torch.arange(8) * 2.0 / 16)
    assert torch.allclose(ci[0], torch.cos(torch.tensor([3., 1., 2., 3., 1., 2., 3., 3.]) * inv), atol=1e-6)
    assert torch.allclose(cc[0], torch.cos(torch.tensor([3., 3., 3., 3., 1., 1., 2., 2.]) * inv), atol=1e-6)

    mcfg = ModelConfig(arch="qwen3", num_layers=2, hidden_size=64, num_attention_heads=4, num_kv_heads=2, head_dim=16,
                       ffn_hidden_size=128, vocab_size=512, dtype="float32", qk_layernorm=True, mrope_sections=(4, 2, 2))
    vc = VisionConfig(patch_size=2, hidden_size=32, num_layers=2, num_heads=2, ffn_hidden_size=64, max_grid=8)
    torch.manual_seed(0)
    m = Qwen3VLModel(mcfg, vc, IMG, VID, deepstack_layers=(0,), temporal_patch=2, recompute="none")
    m.reset_parameters(3)
    ids = torch.tensor(toks + [11, 12, 13])          # a second, text-only sequence in the same packed batch
    cu = torch.tensor([0, len(toks), len(toks) + 3], dtype=torch.int32)
    vision = {"image_patches": torch.randn(16, vc.patch_dim), "image_grid": [(4, 4)],
              "video_patches": torch.randn(16, vc.patch_dim * 2), "video_grid": [(2, 4, 2)]}
    h, _ = m(ids, None, cu, len(toks), vision=vision)
    assert h.shape == (ids.numel(), 64) and torch.isfinite(h).all()
    h.sum().backward()
    assert m.vision.deep_fc2[0].weight.grad.abs().sum() > 0 and m.vision.video_embed.weight.grad.abs().sum() > 0
    # the text-only sequence is unaffected by the visual sequence in front of it
    h2, _ = m(ids[len(toks):], None, torch.tensor([0, 3], dtype=torch.int32), 3)
    assert torch.allclose(h[len(toks):], h2, atol=1e-5)


def test_qwen3_vl_trains_through_the_engine_with_images_and_videos():
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import ModelConfig
    from gcore_b200.models.qwen3_vl import Qwen3VLModel
    IMG, VID = 500, 501
    mcfg = ModelConfig(arch="qwen3", num_layers=2, hidden_size=64, num_attention_heads=4, num_kv_heads=2, head_dim=16,
                       ffn_hidden_size=128, vocab_size=512, dtype="float32", qk_layernorm=True, mrope_sections=(4, 2, 2))
    pc = PolicyConfig(recompute="none", without_ref=True, image_token_id=IMG,
                      vision_config=dict(patch_size=2, hidden_size=32, num_layers=2, num_heads=2, ffn_hidden_size=64,
                                         max_grid=8),
                      vision_options={"video_token_id": VID, "deepstack_layers": [0, 1]})
    e = TrainingEngine(pc, OptimizerConfig(lr=2e-3, lr_decay_style="constant", weight_decay=0.0),
                       TrainingConfig(train_mbs=2, train_gbs=4), model_cfg=mcfg)
    e.setup_model_and_get_optimizer(seed=5)
    assert isinstance(e.model, Qwen3VLModel)
    g = torch.Generator().manual_seed(1)

    def sample(kind):
        if kind == "image":
            toks = [3, 4] + [IMG] * 4 + [9, 10, 11, 12]
            extra = {"pixel_patches": torch.randn(16, 12, generator=g), "image_grid": (4, 4)}
        elif kind == "video":
            toks = [3] + [VID] * 4 + [9, 10, 11]
            extra = {"video_patches": torch.randn(16, 24, generator=g), "video_grid": (2, 4, 2)}
        else:
            toks, extra = [3, 4, 5, 6, 7, 8], {}
        m = torch.zeros(len(toks))
        m[-4:-1] = 1
        return dict(tokens=torch.tensor(toks), loss_mask=m, **extra)

    batch = [sample("image"), sample("video"), sample("text"), sample("image")]
    losses = [e.finetune_step(batch)["lm_loss"] for _ in range(6)]
    assert losses[-1] < losses[0] - 0.2, losses
    lp = e.compute_log_probs(batch)
    assert all(torch.isfinite(s["logprobs"]).all() for s in lp)
