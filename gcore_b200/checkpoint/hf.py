"""HuggingFace safetensors export / import of a (TP / EP sharded) model.

Export follows the reference's ``bridge_save_hf`` sidecars (gpatch_v4/training_backend/megatron_backend/checkpoint.py:
218-300, 704): ``hf/{step}/`` full weights (LoRA merged when ``save_merged_lora_weights``), ``hf/{step}_adapter/``
adapter-only PEFT layout.  Shards are capped in size and indexed by ``model.safetensors.index.json``; only rank 0 of
each gather group writes.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist
from safetensors.torch import load_file, save_file

from ..core import parallel_state as ps
from .layout import export_full_weights, load_hf_weights


def hf_config_dict(cfg) -> dict:
    arch = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM",
            "qwen3_moe": "Qwen3MoeForCausalLM", "qwen2_moe": "Qwen2MoeForCausalLM", "deepseek_v3": "DeepseekV3ForCausalLM",
            "mistral": "MistralForCausalLM", "gpt_oss": "GptOssForCausalLM",
            "seed_oss": "SeedOssForCausalLM"}.get(cfg.arch, "LlamaForCausalLM")
    d = {"architectures": [arch], "model_type": cfg.arch if cfg.arch != "llama" else "llama",
         "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
         "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_kv_heads,
         "head_dim": cfg.head_dim, "intermediate_size": cfg.ffn_hidden_size, "vocab_size": cfg.vocab_size,
         "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta,
         "tie_word_embeddings": cfg.tie_word_embeddings, "max_position_embeddings": cfg.max_position_embeddings,
         "torch_dtype": cfg.dtype, "hidden_act": "silu"}
    if cfg.is_moe:
        d.update(num_experts=cfg.num_experts, n_routed_experts=cfg.num_experts, num_experts_per_tok=cfg.moe_top_k,
                 moe_intermediate_size=cfg.moe_ffn_hidden_size, norm_topk_prob=cfg.moe_norm_topk_prob,
                 router_aux_loss_coef=cfg.moe_aux_loss_coef)
        if getattr(cfg, "moe_shared_expert_gate", False):
            d["shared_expert_intermediate_size"] = cfg.moe_shared_expert_ffn
    if cfg.use_mla:
        d.update(q_lora_rank=cfg.q_lora_rank or None, kv_lora_rank=cfg.kv_lora_rank,
                 qk_nope_head_dim=cfg.qk_nope_head_dim, qk_rope_head_dim=cfg.qk_rope_head_dim,
                 v_head_dim=cfg.v_head_dim, n_group=cfg.moe_n_group, topk_group=cfg.moe_topk_group,
                 first_k_dense_replace=cfg.first_k_dense, routed_scaling_factor=cfg.moe_routed_scaling_factor)
    if cfg.sliding_window:
        d["sliding_window"] = cfg.sliding_window
    return d


def save_hf(engine, out_dir: str, max_shard_bytes: int = 4 << 30, merged_lora: bool = True) -> Optional[str]:
    """Every rank takes part in the gathers; the global rank 0 writes the files."""
    is_writer = (not dist.is_initialized()) or dist.get_rank() == 0
    if is_writer:
        os.makedirs(out_dir, exist_ok=True)
    shard: Dict[str, torch.Tensor] = {}
    size = 0
    index = {}
    files = []

    def flush():
        nonlocal shard, size
        if not shard or not is_writer:
            shard, size = {}, 0
            return
        name = f"model-{len(files) + 1:05d}.safetensors"
        save_file({k: v.contiguous() for k, v in shard.items()}, os.path.join(out_dir, name), metadata={"format": "pt"})
        for k in shard:
            index[k] = name
        files.append(name)
        shard, size = {}, 0

    tied = engine.model_cfg.tie_word_embeddings
    for name, t in export_full_weights(engine):
        if tied and name == "lm_head.weight":
            continue
        if is_writer:
            shard[name] = t.detach().cpu()
            size += t.numel() * t.element_size()
            if size >= max_shard_bytes:
                flush()
    flush()
    if is_writer:
        total = len(files)
        renamed = {}
        for i, f in enumerate(files):
            new = f"model-{i + 1:05d}-of-{total:05d}.safetensors"
            os.replace(os.path.join(out_dir, f), os.path.join(out_dir, new))
            renamed[f] = new
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as fh:
            json.dump({"metadata": {}, "weight_map": {k: renamed[v] for k, v in index.items()}}, fh, indent=1)
        with open(os.path.join(out_dir, "config.json"), "w") as fh:
            json.dump(hf_config_dict(engine.model_cfg), fh, indent=1)
    if dist.is_initialized() and dist.get_world_size() > 1:
        ps.cpu_barrier()
    return out_dir if is_writer else None


def save_lora_adapter(engine, out_dir: str, lora_cfg) -> Optional[str]:
    """PEFT-style adapter-only export (``adapter_model.safetensors`` + ``adapter_config.json``)."""
    from ..models.lora import lora_state_dict
    is_writer = (not dist.is_initialized()) or dist.get_rank() == 0
    sd = {k: v.detach().cpu().contiguous() for k, v in lora_state_dict(engine.model).items()}
    if is_writer:
        os.makedirs(out_dir, exist_ok=True)
        save_file(sd, os.path.join(out_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
        with open(os.path.join(out_dir, "adapter_config.json"), "w") as fh:
            json.dump({"peft_type": "LORA", "r": lora_cfg.rank, "lora_alpha": lora_cfg.alpha,
                       "lora_dropout": lora_cfg.dropout, "target_modules": list(lora_cfg.target_modules),
                       "gcore_lora_type": lora_cfg.type}, fh, indent=1)
    return out_dir if is_writer else None


def load_lora_adapter(engine, adapter_dir: str):
    sd = load_file(os.path.join(adapter_dir, "adapter_model.safetensors"))
    params = dict(engine.model.named_parameters())
    with torch.no_grad():
        for k, v in sd.items():
            params[k].copy_(v.to(params[k].dtype))


def read_hf_dir(path: str) -> Dict[str, torch.Tensor]:
    idx = os.path.join(path, "model.safetensors.index.json")
    out: Dict[str, torch.Tensor] = {}
    if os.path.exists(idx):
        files = sorted(set(json.load(open(idx))["weight_map"].values()))
    else:
        files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
    for f in files:
        out.update(load_file(os.path.join(path, f)))
    return out


def load_hf(engine, path: str):
    """Loads full HF weights into this rank's shards and refreshes the optimizer's master copy."""
    tensors = read_hf_dir(path)
    load_hf_weights(engine.model, tensors, ps.get_tensor_model_parallel_rank(), ps.get_expert_model_parallel_rank())
    if engine.optimizer is not None:
        engine.optimizer.reload_master_from_params()
    if engine.ref_model is not None:
        load_hf_weights(engine.ref_model, tensors, ps.get_tensor_model_parallel_rank(),
                        ps.get_expert_model_parallel_rank())
