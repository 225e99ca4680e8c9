"""Casts the linear weights of a Hugging Face bf16 checkpoint to block-scaled fp8 (e4m3 values + one fp32
``weight_scale_inv`` per 128x128 block, the DeepSeek-V3 on-disk convention), leaving embeddings, norms, the router
and the output head in bf16 (the reference's fp8 casting tools under ``tools/`` and
gpatch_v4/generation_backend/sglang_model_specific/sglang_weight_update_dsv4.py:267-321).

    python -m gcore_b200.tools.fp8_cast --hf-dir in --out-dir out
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict

import torch

from ..ops.quant import dequant_128x128, quant_weight_128x128

SKIP = ("embed_tokens", "lm_head", "norm", "mlp.gate.weight", "e_score_correction_bias")


def cast_state_dict(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        if v.dim() == 2 and k.endswith(".weight") and not any(s in k for s in SKIP):
            q, s = quant_weight_128x128(v.to(torch.bfloat16).contiguous())
            out[k] = q
            out[k[:-len("weight")] + "weight_scale_inv"] = s
        else:
            out[k] = v
    return out


def uncast_state_dict(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        if k.endswith("weight_scale_inv"):
            continue
        sk = k[:-len("weight")] + "weight_scale_inv" if k.endswith(".weight") else None
        out[k] = dequant_128x128(v, sd[sk]).to(torch.bfloat16) if sk in sd else v
    return out


def main(argv=None):
    from safetensors.torch import save_file

    from ..checkpoint.hf import read_hf_dir
    ap = argparse.ArgumentParser()
    ap.add_argument("--hf-dir", required=True)
    ap.add_argument("--out-dir", required=True)
    a = ap.parse_args(argv)
    sd = cast_state_dict(read_hf_dir(a.hf_dir))
    os.makedirs(a.out_dir, exist_ok=True)
    save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(a.out_dir, "model.safetensors"))
    cfg_path = os.path.join(a.hf_dir, "config.json")
    if os.path.exists(cfg_path):
        cfg = json.load(open(cfg_path))
        cfg["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128],
                                      "activation_scheme": "dynamic"}
        json.dump(cfg, open(os.path.join(a.out_dir, "config.json"), "w"), indent=1)


if __name__ == "__main__":
    main()
