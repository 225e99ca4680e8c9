"""Checkpoint conversion between Hugging Face safetensors and the Megatron torch_dist layout
(the reference's ``tools/px_ckpt_conv`` HF <-> MLM converters and ``convert_mcore_to_hf``,
gpatch_v4/trainer/helper.py:11-122).

    python -m gcore_b200.tools.ckpt_convert hf2mcore --model qwen2.5-7b --src /path/hf --dst /path/ckpt [--step 0]
    python -m gcore_b200.tools.ckpt_convert mcore2hf --model qwen2.5-7b --src /path/ckpt --dst /path/hf [--step N]

    python -m gcore_b200.tools.ckpt_convert policy2critic --model qwen2.5-7b --src /path/policy --dst /path/critic
    python -m gcore_b200.tools.ckpt_convert strip --model qwen2.5-7b --src /path/rl_ckpt --dst /path/policy_only

``policy2critic`` (also the start of reward-model training): the decoder weights of a policy checkpoint initialise a
model with a scalar value head (new head: small random values; the vocabulary projection is left out);
``strip`` keeps the model weights of a training checkpoint and drops optimizer state, RNG and trainer extras - the
hand-over between stages (SFT -> RL policy / reference, RL -> evaluation; the reference's RM / critic / DPO stage
converters under ``tools/px_ckpt_conv``).

Runs on CPU in one process (TP = PP = 1); the torch_dist format is resharded on load, so the result can be read by
any parallel layout.
"""
from __future__ import annotations

import argparse
import json
import os


def build_engine(model: str, overrides=None, dtype: str = "bfloat16", value_head: bool = False):
    import torch
    from ..configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from ..engine.train_engine import TrainingEngine
    from ..models.config import ModelConfig, get_preset
    if os.path.isfile(model):
        mcfg = ModelConfig(**json.load(open(model)))
    else:
        mcfg = get_preset(model, dtype=dtype, **(overrides or {}))
    eng = TrainingEngine(PolicyConfig(recompute="none", without_ref=True), OptimizerConfig(), TrainingConfig(),
                         model_cfg=mcfg, value_head=value_head, role="critic" if value_head else "policy")
    eng.device = torch.device("cpu")
    eng.setup_model_and_get_optimizer(seed=0, with_ref=False)
    return eng


def hf_to_mcore(model: str, src: str, dst: str, step: int = 0, dtype: str = "bfloat16"):
    from ..checkpoint.hf import load_hf
    from ..checkpoint.torch_dist import save_checkpoint
    eng = build_engine(model, dtype=dtype)
    load_hf(eng, src)
    eng.optimizer.reload_master_from_params()
    save_checkpoint(eng, dst, step, save_optim=False)
    return dst


def mcore_to_hf(model: str, src: str, dst: str, step=None, dtype: str = "bfloat16"):
    from ..checkpoint.hf import save_hf
    from ..checkpoint.torch_dist import load_checkpoint
    eng = build_engine(model, dtype=dtype)
    got = load_checkpoint(eng, src, step, load_optim=False, load_rng=False)
    save_hf(eng, dst)
    return got


def policy_to_critic(model: str, src: str, dst: str, step=None, dtype: str = "bfloat16", out_step: int = 0):
    """Decoder weights from the policy checkpoint, value head freshly initialised; missing keys (the head) are
    expected, everything else must be found."""
    from ..checkpoint.torch_dist import load_checkpoint, save_checkpoint
    eng = build_engine(model, dtype=dtype, value_head=True)
    head = {n for n, _ in eng.model.named_parameters() if n.startswith("output_layer")}
    load_checkpoint(eng, src, step, load_optim=False, load_rng=False, strict=False)
    from ..checkpoint.torch_dist import CheckpointReader, iter_dir, read_latest_step
    rd = CheckpointReader(iter_dir(src, step if step is not None else read_latest_step(src)))
    have = set(rd.keys())
    rd.close()
    assert any(k.startswith(("decoder.layers", "model.decoder.layers")) for k in have), f"{src} holds no decoder weights"
    assert head, "the critic model has no value head"
    eng.optimizer.reload_master_from_params()
    save_checkpoint(eng, dst, out_step, save_optim=False)
    return dst


def strip_checkpoint(model: str, src: str, dst: str, step=None, dtype: str = "bfloat16", out_step: int = 0):
    from ..checkpoint.torch_dist import load_checkpoint, save_checkpoint
    eng = build_engine(model, dtype=dtype)
    load_checkpoint(eng, src, step, load_optim=False, load_rng=False)
    save_checkpoint(eng, dst, out_step, save_optim=False)
    return dst


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("direction", choices=["hf2mcore", "mcore2hf", "policy2critic", "strip"])
    ap.add_argument("--model", required=True, help="preset name or path of a ModelConfig json")
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--step", type=int, default=None)
    ap.add_argument("--dtype", default="bfloat16")
    a = ap.parse_args(argv)
    if a.direction == "hf2mcore":
        print(hf_to_mcore(a.model, a.src, a.dst, a.step or 0, a.dtype))
    elif a.direction == "policy2critic":
        print(policy_to_critic(a.model, a.src, a.dst, a.step, a.dtype))
    elif a.direction == "strip":
        print(strip_checkpoint(a.model, a.src, a.dst, a.step, a.dtype))
    else:
        print(mcore_to_hf(a.model, a.src, a.dst, a.step, a.dtype))


if __name__ == "__main__":
    main()
