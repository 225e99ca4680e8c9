"""Analytic FLOPs and MFU (gpatch_v4/utils/flops_counter.py; actor/mixin.py:1434-1545): forward FLOPs of a packed batch
for dense, MoE and MLA models, x3 for forward + backward (x4 with full recompute)."""
from __future__ import annotations

from typing import Sequence

from ..models.config import ModelConfig


def forward_flops(cfg: ModelConfig, seq_lens: Sequence[int], causal: bool = True) -> float:
    T = float(sum(seq_lens))
    h = cfg.hidden_size
    flops = 0.0
    for i in range(cfg.num_layers):
        if cfg.use_mla:
            q = (h * cfg.q_lora_rank + cfg.q_lora_rank * cfg.num_attention_heads * cfg.qk_head_dim) if cfg.q_lora_rank \
                else h * cfg.num_attention_heads * cfg.qk_head_dim
            kv = h * (cfg.kv_lora_rank + cfg.qk_rope_head_dim) + cfg.kv_lora_rank * cfg.num_attention_heads * (
                cfg.qk_nope_head_dim + cfg.v_head_dim)
            o = cfg.num_attention_heads * cfg.v_head_dim * h
            attn_w = q + kv + o
            dqk, dv = cfg.qk_head_dim, cfg.v_head_dim
        else:
            attn_w = h * (cfg.num_attention_heads + 2 * cfg.num_kv_heads) * cfg.head_dim + \
                cfg.num_attention_heads * cfg.head_dim * h
            dqk = dv = cfg.head_dim
        flops += 2 * T * attn_w
        w = cfg.layer_window(i)
        for L in seq_lens:
            eff = L if not w else min(L, w)
            pairs = L * eff / (2.0 if causal and not w else 1.0)
            if w and causal:
                pairs = eff * (eff + 1) / 2 + max(L - eff, 0) * eff
            flops += 2 * cfg.num_attention_heads * pairs * (dqk + dv)
        if cfg.layer_is_moe(i):
            flops += 2 * T * (cfg.moe_top_k * 3 * h * cfg.moe_ffn_hidden_size + h * cfg.num_experts +
                              3 * h * cfg.moe_shared_expert_ffn)
        else:
            flops += 2 * T * 3 * h * cfg.ffn_hidden_size
    flops += 2 * T * h * cfg.vocab_size
    return flops


def train_flops(cfg: ModelConfig, seq_lens: Sequence[int], recompute: bool = False) -> float:
    return forward_flops(cfg, seq_lens) * (4.0 if recompute else 3.0)


def mfu(flops: float, seconds: float, n_gpus: int, peak_tflops: float = 2250.0) -> float:
    return flops / max(seconds, 1e-9) / (n_gpus * peak_tflops * 1e12)
