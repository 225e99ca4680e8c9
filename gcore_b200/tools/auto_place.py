"""Placement search: which (TP, PP, CP, EP, DP) layouts fit a model on a cluster, ranked by a throughput heuristic
(the reference's ``tools/auto_place.py`` and the planning notes in docs/source/estimate_resource_priv.md:13-24).

    python -m gcore_b200.tools.auto_place --model qwen2.5-7b --gpus 8 --seq-len 1280 --mb-tokens 8192

Memory model per GPU (bytes): parameters 2P/mp (+ the same for a reference model), fp32 main gradients 4P/mp, AdamW
state 12P/(mp*dp) (ZeRO-1), activations of one micro-batch (per token-layer ~ 34 H / tp bytes with recompute off, 2 H
with full recompute, divided by CP), rollout KV cache budget.  Throughput heuristic: model FLOPs over the measured
GEMM rate, discounted per parallel dimension (TP 0.92 per doubling inside NVLink, PP bubble (pp-1)/m, CP 0.9,
EP 0.85).
"""
from __future__ import annotations

import argparse
import itertools
import json
from dataclasses import asdict, dataclass
from typing import List


@dataclass
class Placement:
    tp: int
    pp: int
    cp: int
    ep: int
    dp: int
    mem_gb: float
    score: float
    recompute: str


def _divisors(n):
    return [d for d in range(1, n + 1) if n % d == 0]


def param_counts(cfg):
    total = cfg.num_parameters() if hasattr(cfg, "num_parameters") else None
    h, L, v = cfg.hidden_size, cfg.num_layers, cfg.vocab_size
    D = cfg.head_dim
    attn = h * (cfg.num_attention_heads + 2 * cfg.num_kv_heads) * D + cfg.num_attention_heads * D * h
    if cfg.num_experts:
        expert = cfg.num_experts * 3 * h * cfg.moe_ffn_hidden_size
        dense = attn * L + 2 * v * h
        return dense, expert * L
    mlp = 3 * h * cfg.ffn_hidden_size
    return (attn + mlp) * L + 2 * v * h if total is None else total, 0


def search(cfg, gpus: int, seq_len: int, mb_tokens: int, hbm_gb: float = 180.0, with_ref: bool = True,
           kv_budget_gb: float = 20.0, micro_batches: int = 8, gpus_per_node: int = 8) -> List[Placement]:
    dense, expert = param_counts(cfg)
    out = []
    for tp, pp, cp in itertools.product(_divisors(min(gpus, gpus_per_node)), _divisors(gpus), _divisors(gpus)):
        mp = tp * pp * cp
        if gpus % mp or cfg.num_attention_heads % tp or cfg.num_kv_heads % tp or cfg.num_layers % pp:
            continue
        if cp > 1 and seq_len < 8192:
            continue
        dp = gpus // mp
        eps = [e for e in _divisors(dp * cp) if cfg.num_experts and cfg.num_experts % e == 0] or [1]
        for ep in eps:
            p_dense = dense / (tp * pp)
            p_exp = expert / (pp * ep)
            P = p_dense + p_exp
            edp = max(dp * cp // ep, 1)
            for recompute in ("none", "full"):
                act_per_tok_layer = (34 if recompute == "none" else 2) * cfg.hidden_size / tp
                act = act_per_tok_layer * (cfg.num_layers / pp) * mb_tokens / cp
                if pp > 1:
                    act *= min(pp, micro_batches)  # in-flight micro-batches of the first stage
                mem = (2 * P * (2 if with_ref else 1) + 4 * P + 12 * (p_dense / (dp * cp) + p_exp / edp) + act) / 2**30
                mem += kv_budget_gb + 6.0  # KV cache + workspace / logits chunks
                if mem > hbm_gb * 0.95:
                    continue
                eff = (0.92 ** (tp.bit_length() - 1)) * (1.0 - (pp - 1) / (micro_batches + pp - 1))
                eff *= (0.9 if cp > 1 else 1.0) * (0.85 if ep > 1 else 1.0) * (0.8 if recompute == "full" else 1.0)
                out.append(Placement(tp, pp, cp, ep, dp, round(mem, 1), round(eff, 4), recompute))
                break  # recompute "none" fits: no need to list the slower variant
    out.sort(key=lambda p: (-p.score, p.tp * p.pp * p.cp))
    return out


def main(argv=None):
    from ..models.config import get_preset
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=1280)
    ap.add_argument("--mb-tokens", type=int, default=8192)
    ap.add_argument("--hbm-gb", type=float, default=180.0)
    ap.add_argument("--top", type=int, default=8)
    a = ap.parse_args(argv)
    res = search(get_preset(a.model), a.gpus, a.seq_len, a.mb_tokens, a.hbm_gb)
    for p in res[:a.top]:
        print(json.dumps(asdict(p)))
    return res


if __name__ == "__main__":
    main()
