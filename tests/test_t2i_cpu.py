"""Image-generation family on CPU with tiny models: sampler mathematics, the GRPO / DPO / edit / unified trainers and
their entry points."""
import math

import pytest
import torch
import yaml

from gcore_b200.configs.base import from_dict
from gcore_b200.configs.config import T2iConfig

TINY = {"model": {"transformer": {"hidden_size": 64, "num_heads": 2, "depth_double": 1, "depth_single": 1,
                                  "text_dim": 32, "pooled_dim": 16, "axes_dims_rope": [8, 12, 12]},
                  "text_max_length": 16, "latent_channels": 4, "vae_base_channels": 4, "lm_hidden_size": 64},
        "training": {"height": 32, "width": 32, "sampling_steps": 5, "rollout_gbs": 2, "sampling_repeat_n": 4,
                     "train_gbs_wo_timestep": 4, "train_mbs": 2, "total_ppo_step": 2, "total_training_step": 3,
                     "use_bf16": False, "eta": 0.4},
        "optimizer": {"lr": 2e-3, "lr_decay_style": "constant", "weight_decay": 0.0},
        "ppo": {"ppo_ratio_eps": 0.2}}


def _cfg(**over):
    import copy
    d = copy.deepcopy(TINY)
    for k, v in over.items():
        d.setdefault(k, {}).update(v)
    return from_dict(T2iConfig, d)


def test_sde_step_is_a_gaussian_transition_and_replays_its_log_prob():
    from gcore_b200.pipelines.scheduling import sde_step, sigma_schedule, sd3_time_shift
    sig, ts = sigma_schedule(3.0, 6)
    assert float(sig[0]) == 1.0 and float(sig[-1]) == 0.0 and torch.all(sig[:-1] > sig[1:])
    assert torch.allclose(sd3_time_shift(1.0, sig), sig)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 10, 8, generator=g)
    v = torch.randn(3, 10, 8, generator=g)
    nxt, x0, lp, noise = sde_step(v, x, sig, 2, eta=0.3, generator=g)
    # replay: the same transition under the same model output has the same log-probability
    _, _, lp2, _ = sde_step(v, x, sig, 2, eta=0.3, prev_sample=nxt)
    assert torch.allclose(lp, lp2)
    # closed form: mean log density of a standard normal draw scaled by std
    std = 0.3 * math.sqrt(float(sig[2] - sig[3]))
    want = (-(noise ** 2) / 2 - math.log(std) - 0.5 * math.log(2 * math.pi)).mean((1, 2))
    assert torch.allclose(lp, want, atol=1e-4)
    # eta -> 0 approaches the deterministic Euler step
    det = x + float(sig[3] - sig[2]) * v
    near, _, _, _ = sde_step(v, x, sig, 2, eta=1e-4, noise=torch.zeros_like(x))
    assert torch.allclose(near, det, atol=1e-5)
    assert torch.allclose(x0, x - float(sig[2]) * v)


def test_flux_pipeline_rollout_batch_and_on_policy_ratio():
    from gcore_b200.pipelines import FluxPipeline
    cfg = _cfg(training={"train_gas_wo_timestep": 2})   # one optimizer step after both micro-batches
    pipe = FluxPipeline(cfg)
    pipe.setup_pipeline()
    prompts = ["a red square"] * 4
    rb, req = pipe(prompt=prompts, generator=torch.Generator().manual_seed(1))
    steps = cfg.training.sampling_steps - 1
    assert len(rb["latents"]) == 4 and rb["latents"][0].shape == (steps, 4, 16) and rb["log_probs"][0].shape == (steps,)
    assert req["images"][0].shape == (3, 32, 32) and torch.equal(rb["latents"][0][1], rb["next_latents"][0][0])
    rb["advantages"] = [torch.tensor(a) for a in (1.0, -1.0, 0.5, -0.5)]
    rb = pipe.permute_timesteps(rb, torch.Generator().manual_seed(2))
    samples = [{k: rb[k][i] for k in rb if k != "images"} for i in range(4)]
    w0 = [p.detach().clone() for p in pipe.model.parameters()]
    m = pipe.ppo_train_step(samples)
    assert abs(m["policy/ppo_ratio"] - 1.0) < 1e-3, m      # the first pass after an on-policy rollout
    assert m["policy/grad_norm"] > 0
    assert any(not torch.equal(a, b) for a, b in zip(w0, pipe.model.parameters()))


def test_t2i_grpo_raises_the_colour_reward():
    from gcore_b200.trainer.t2i_trainers import T2iGrpoTrainer
    cfg = _cfg(training={"total_ppo_step": 6, "timestep_fraction": 1.0}, optimizer={"lr": 5e-3})
    tr = T2iGrpoTrainer(cfg).setup()
    hist = tr.run()
    assert len(hist) == 6 and all(h["policy/grad_norm"] > 0 for h in hist)
    adv = tr.calculate_advantage({"a": torch.tensor([1.0, 2.0, 3.0, 4.0]), "b": torch.tensor([0.0, 0.0, 1.0, 1.0])}, 4)
    assert abs(float(adv.sum())) < 1e-5 and adv[3] > adv[0]


def test_diffusion_dpo_prefers_the_chosen_image_and_sft_mode_trains():
    from gcore_b200.trainer.t2i_trainers import T2iDpoTrainer
    cfg = _cfg(training={"total_training_step": 16, "train_mbs": 4}, dpo={"beta_dpo": 5000.0}, optimizer={"lr": 3e-3})
    hist = T2iDpoTrainer(cfg).setup().run()
    assert abs(hist[0]["train_loss"] - math.log(2)) < 1e-3    # policy == reference at the start
    tail = hist[-6:]
    assert sum(h["train_loss"] for h in tail) / 6 < math.log(2) - 0.02, [h["train_loss"] for h in hist]
    assert sum(h["implicit_acc"] for h in tail) / 6 > 0.6
    cfg2 = _cfg(training={"total_training_step": 4, "train_method": "sft"})
    h2 = T2iDpoTrainer(cfg2).setup().run()
    assert all(h["grad_norm"] > 0 for h in h2)


def test_edit_pipeline_conditions_on_the_source_image():
    from gcore_b200.pipelines import QwenImageEditPipeline
    from gcore_b200.trainer.t2i_trainers import T2iEditSftTrainer
    cfg = _cfg(model={"pipeline": "qwen_image_edit"}, training={"total_training_step": 3})
    hist = T2iEditSftTrainer(cfg).setup().run()
    assert len(hist) == 3 and hist[0]["grad_norm"] > 0
    pipe = QwenImageEditPipeline(cfg)
    pipe.setup_pipeline()
    torch.manual_seed(0)
    for p in pipe.model.parameters():   # zero-initialised gates / output layer would hide the conditioning
        if p.dim() == 2 and not p.any():
            torch.nn.init.normal_(p, std=0.1)
    src_a, src_b = torch.zeros(1, 3, 32, 32), torch.ones(1, 3, 32, 32)
    ra, _ = pipe(prompt=["make it red"], image=src_a, generator=torch.Generator().manual_seed(3))
    rb_, _ = pipe(prompt=["make it red"], image=src_b, generator=torch.Generator().manual_seed(3))
    assert "cond_latents" in ra and not torch.allclose(ra["next_latents"][0], rb_["next_latents"][0])


def test_bagel_unified_training_and_grpo(tmp_path):
    from gcore_b200.trainer.t2i_trainers import BagelTrainer, T2iGrpoTrainer
    cfg = _cfg(model={"pipeline": "bagel"}, training={"total_training_step": 6, "eval_interval": 3, "guidance_scale": 1.0,
                                                     "save_interval": 3},
               checkpoint={"save_ckpt_path": str(tmp_path / "ck")}, optimizer={"lr": 3e-3})
    tr = BagelTrainer(cfg).setup()
    hist = tr.run()
    assert hist[-1]["ce"] < hist[0]["ce"] and "valid/mse" in hist[2] and hist[0]["mse"] > 0
    # resume picks the step and the weights up
    tr2 = BagelTrainer(cfg).setup()
    assert tr2.step == 6
    for a, b in zip(tr.pipe.model.parameters(), tr2.pipe.model.parameters()):
        assert torch.equal(a, b)
    # reinforcement learning starts from the supervised checkpoint (a zero-initialised velocity head has no
    # guidance direction to renormalise)
    cfg_g = _cfg(model={"pipeline": "bagel"}, training={"total_ppo_step": 8, "guidance_scale": 2.0},
                 checkpoint={"load_ckpt_path": str(tmp_path / "ck")})
    trg = T2iGrpoTrainer(cfg_g).setup()
    assert trg.step == 6
    h = trg.run()
    assert len(h) == 2 and all(x["policy/grad_norm"] > 0 for x in h)
    v = tr.pipe.merge_uncond_predict(torch.zeros(4, 8), torch.ones(4, 8), 3.0)
    assert torch.allclose(v, torch.ones(4, 8), atol=1e-5)   # renormalised back to the conditional prediction's norm


def test_t2i_entry_points(tmp_path):
    from gcore_b200.entry import (train_bagel, train_bagel_t2i_grpo, train_t2i_dpo, train_t2i_edit_sft,
                                  train_t2i_grpo)
    p = tmp_path / "t2i.yaml"
    p.write_text(yaml.safe_dump(TINY))
    small = ["training.total_ppo_step=1", "training.total_training_step=1", f"report.log_dir={tmp_path / 'log'}"]
    for mod in (train_t2i_grpo, train_t2i_dpo, train_t2i_edit_sft, train_bagel, train_bagel_t2i_grpo):
        hist = mod.main(["--config", str(p)] + small)
        assert len(hist) == 1, mod.__name__


def test_generation_validation_runs_inside_the_training_loop(tmp_path):
    """Validation cases are generated with the live weights every ``eval_interval`` steps; images, ``metrics.json``
    and the aggregated similarities land below ``val_results/step_*``; module modes are restored afterwards."""
    import json
    import os
    from gcore_b200.trainer.t2i_trainers import T2iGrpoTrainer
    from gcore_b200.validation import EmbeddingMetrics, restore_modes, snapshot_modes
    cases = tmp_path / "val.jsonl"
    with open(cases, "w") as f:
        for p in ("a red square", "a blue square", "a green square"):
            f.write(json.dumps({"prompt": p, "task_type": "t2i"}) + "\n")
    cfg = _cfg(training={"total_ppo_step": 2, "eval_interval": 2}, data={"eval_data_path": str(cases)},
               report={"log_dir": str(tmp_path)})
    tr = T2iGrpoTrainer(cfg).setup()
    tr.pipe.model.train()
    hist = tr.run()
    assert tr.pipe.model.training
    assert "val/train/t2i/text_image" not in hist[0]
    m = hist[1]
    assert m["val/train/t2i/cases"] == 3 and -1.0 <= m["val/train/t2i/text_image"] <= 1.0
    root = os.path.join(str(tmp_path), "val_results", "step_0000002")
    assert json.load(open(os.path.join(root, "metrics.json")))["val/train/t2i/cases"] == 3
    assert len([n for n in os.listdir(os.path.join(root, "train")) if n.endswith(".pt")]) == 3
    # the scorer: an image is most similar to itself; mode snapshot / restore is exact
    em = EmbeddingMetrics()
    a, b = torch.rand(3, 16, 16), torch.rand(3, 16, 16)
    assert em.image_image_score(a, a) > 0.999 > em.image_image_score(a, b)
    mod = torch.nn.Sequential(torch.nn.Linear(2, 2), torch.nn.Dropout())
    mod[1].eval()
    snap = snapshot_modes(mod)
    mod.eval()
    restore_modes(mod, snap)
    assert mod.training and mod[0].training and not mod[1].training
