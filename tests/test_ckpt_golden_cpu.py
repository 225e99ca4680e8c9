"""A torch_dist tree written WITHOUT this package's writer - torch.distributed.checkpoint plus the sidecars, laid out
from Megatron-Core's format description - must load into the engine:

* keys are parameter paths with an empty prefix (``decoder.layers.<rest>`` with the layer index as a prepended axis,
  ``embedding.word_embeddings.weight``, ``output_layer.weight``), input norms live under the following linear
  (``linear_qkv.layer_norm_weight`` / ``linear_fc1.layer_norm_weight``), ``linear_qkv.weight`` rows are interleaved per
  KV group ``[q .. q, k, v]``, ``linear_fc1.weight`` is ``cat[gate; up]``
  (gpatch_v4/training_backend/megatron_backend/checkpoint.py:1007-1065, tools/px_ckpt_conv/mlm_to_hf.py:61-163);
* optimizer state per parameter under ``optimizer.state.{exp_avg,exp_avg_sq,fp32_param}.<parameter key>``;
* ``rng_state`` is a sharded object of shape (pp, tp) holding a list of dicts with Megatron's field names
  (checkpoint.py:753-797); ``common.pt`` carries the non-tensor state (iteration, optimizer param groups, scheduler);
  ``metadata.json`` names the backend.
"""
import io
import json
import os
import random

import numpy as np
import torch
import torch.distributed.checkpoint as dcp

from gcore_b200.checkpoint.torch_dist import load_checkpoint
from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
from gcore_b200.engine.train_engine import TrainingEngine
from gcore_b200.models.config import get_preset

L, H, HQ, HK, D, F, V = 2, 256, 4, 2, 64, 688, 1024


def _golden_tensors():
    g = torch.Generator().manual_seed(123)

    def r(*shape):
        return torch.randn(*shape, generator=g) * 0.05

    # what the model must hold after loading, in plain per-layer form
    want = {"embed": r(V, H), "out": r(V, H), "final_ln": 1 + r(H),
            "ln1": 1 + r(L, H), "ln2": 1 + r(L, H), "q": r(L, HQ * D, H), "k": r(L, HK * D, H), "v": r(L, HK * D, H),
            "o": r(L, H, HQ * D), "gate": r(L, F, H), "up": r(L, F, H), "down": r(L, H, F)}
    rep = HQ // HK
    qkv = []
    for li in range(L):
        rows = []
        for grp in range(HK):   # Megatron: [q heads of the group, k of the group, v of the group], group after group
            rows += [want["q"][li, (grp * rep) * D:(grp * rep + rep) * D], want["k"][li, grp * D:(grp + 1) * D],
                     want["v"][li, grp * D:(grp + 1) * D]]
        qkv.append(torch.cat(rows, 0))
    tree = {
        "embedding.word_embeddings.weight": want["embed"],
        "output_layer.weight": want["out"],
        "decoder.final_layernorm.weight": want["final_ln"],
        "decoder.layers.self_attention.linear_qkv.layer_norm_weight": want["ln1"],
        "decoder.layers.self_attention.linear_qkv.weight": torch.stack(qkv),
        "decoder.layers.self_attention.linear_proj.weight": want["o"],
        "decoder.layers.mlp.linear_fc1.layer_norm_weight": want["ln2"],
        "decoder.layers.mlp.linear_fc1.weight": torch.cat([want["gate"], want["up"]], 1),
        "decoder.layers.mlp.linear_fc2.weight": want["down"],
    }
    return want, tree


def _write_golden(path, step):
    want, tree = _golden_tensors()
    d = os.path.join(path, f"iter_{step:07d}")
    os.makedirs(d)
    sd = {k: v.clone() for k, v in tree.items()}
    for k, v in tree.items():
        sd[f"optimizer.state.exp_avg.{k}"] = v.float() * 0.5
        sd[f"optimizer.state.exp_avg_sq.{k}"] = v.float() ** 2
        sd[f"optimizer.state.fp32_param.{k}"] = v.float()
    rng = [{"random_rng_state": random.Random(5).getstate(), "np_rng_state": np.random.RandomState(6).get_state(),
            "torch_rng_state": torch.Generator().manual_seed(7).get_state(),
            "rng_tracker_states": {"model-parallel-rng": torch.Generator().manual_seed(8).get_state()}}]
    buf = io.BytesIO()
    torch.save(rng, buf)
    buf.seek(0)
    sd["rng_state/shard_0_0_1_1"] = buf
    dcp.save(sd, checkpoint_id=d, no_dist=True)
    torch.save({"iteration": step, "checkpoint_version": 3.0,
                "optimizer": {"optimizer": {"param_groups": [{"lr": 1e-4, "betas": (0.9, 0.999), "eps": 1e-8,
                                                              "weight_decay": 0.01, "step": step}]},
                              "param_state_sharding_type": "fully_sharded_model_space"},
                "lr_scheduler": {"max_lr": 1e-4, "lr_warmup_steps": 0, "num_steps": step, "lr_decay_style": "constant",
                                 "lr_decay_steps": 100, "min_lr": 0.0, "start_wd": 0.01, "end_wd": 0.01,
                                 "wd_incr_style": "constant", "wd_incr_steps": 100}},
               os.path.join(d, "common.pt"))
    json.dump({"sharded_backend": "torch_dist", "sharded_backend_version": 1, "common_backend": "torch",
               "common_backend_version": 1}, open(os.path.join(d, "metadata.json"), "w"))
    open(os.path.join(path, "latest_checkpointed_iteration.txt"), "w").write(str(step))
    return want, rng


def test_engine_loads_a_tree_written_from_the_megatron_format_description(tmp_path):
    want, rng = _write_golden(str(tmp_path), 7)
    mcfg = get_preset("tiny_llama", dtype="float32")
    assert (mcfg.num_layers, mcfg.hidden_size, mcfg.ffn_hidden_size, mcfg.vocab_size) == (L, H, F, V)
    e = TrainingEngine(PolicyConfig(recompute="none", without_ref=True),
                       OptimizerConfig(lr=1e-4, lr_decay_style="constant"), TrainingConfig(), model_cfg=mcfg)
    e.setup_model_and_get_optimizer(seed=1)
    assert load_checkpoint(e, str(tmp_path)) == 7
    m = e.model
    assert torch.equal(m.embedding.word_embeddings.weight, want["embed"])
    assert torch.equal(m.output_weight(), want["out"])
    assert torch.equal(m.decoder.final_layernorm.weight, want["final_ln"])
    for li, layer in enumerate(m.decoder.layers):
        a = layer.self_attention
        assert torch.equal(layer.input_layernorm.weight, want["ln1"][li])
        assert torch.equal(layer.pre_mlp_layernorm.weight, want["ln2"][li])
        # the engine keeps [Q | K | V] and [gate | up] blocks (kernel-friendly); the tree interleaves per KV group
        assert torch.equal(a.linear_qkv.weight, torch.cat([want["q"][li], want["k"][li], want["v"][li]], 0))
        assert torch.equal(a.linear_proj.weight, want["o"][li])
        assert torch.equal(layer.mlp.linear_fc1.weight, torch.cat([want["gate"][li], want["up"][li]], 0))
        assert torch.equal(layer.mlp.linear_fc2.weight, want["down"][li])
    # optimizer state follows its parameter through the same re-layout
    opt = e.optimizer
    assert opt.step_count == 7 and e.step == 7
    names = {id(p): n for n, p in m.named_parameters()}
    for sh in opt.shards:
        buf = sh["buf"]
        for p in sh["bucket"].params:
            o = buf.offsets[id(p)] - sh["s"]
            w = p.detach().float().reshape(-1)
            assert torch.allclose(sh["master"][o:o + p.numel()], w), names[id(p)]
            assert torch.allclose(sh["m"][o:o + p.numel()], 0.5 * w), names[id(p)]
            assert torch.allclose(sh["v"][o:o + p.numel()], w * w), names[id(p)]
    # the RNG object was applied
    assert torch.equal(torch.get_rng_state(), rng[0]["torch_rng_state"])
    assert random.getstate() == rng[0]["random_rng_state"]
    # and the engine trains on from there
    g = torch.Generator().manual_seed(0)
    batch = [{"tokens": torch.randint(3, V, (24,), generator=g), "loss_mask": torch.ones(24)} for _ in range(4)]
    out = e.finetune_step(batch)
    assert out["lm_loss"] == out["lm_loss"] and out["grad_norm"] > 0


def test_trees_of_this_package_use_the_same_names(tmp_path):
    from gcore_b200.checkpoint.torch_dist import CheckpointReader, save_checkpoint
    mcfg = get_preset("tiny_llama", dtype="float32")
    e = TrainingEngine(PolicyConfig(recompute="none", without_ref=True), OptimizerConfig(), TrainingConfig(),
                       model_cfg=mcfg)
    e.setup_model_and_get_optimizer(seed=1)
    save_checkpoint(e, str(tmp_path), 3)
    rd = CheckpointReader(str(tmp_path / "iter_0000003"))
    keys = set(rd.keys())
    _, tree = _golden_tensors()
    for k, v in tree.items():
        assert k in keys and tuple(rd.md.state_dict_metadata[k].size) == tuple(v.shape), k
        for st in ("exp_avg", "exp_avg_sq", "fp32_param"):
            assert f"optimizer.state.{st}.{k}" in keys
    assert "rng_state/shard_0_0_1_1" in keys
    obj = rd.read_object("rng_state/shard_0_0_1_1")
    assert isinstance(obj, list) and {"random_rng_state", "np_rng_state", "torch_rng_state",
                                      "rng_tracker_states"} <= set(obj[0])
    common = torch.load(tmp_path / "iter_0000003" / "common.pt", weights_only=False)
    assert common["iteration"] == 3 and "param_groups" in common["optimizer"]["optimizer"]
    assert common["lr_scheduler"]["num_steps"] == e.optimizer.step_count
