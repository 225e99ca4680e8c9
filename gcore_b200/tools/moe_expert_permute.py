"""Offline MoE expert re-permutation for expert-parallel load balance (the reference's EPLB-style balanced bisection
tool under ``tools/``): given per-expert token counts measured on a calibration set, renumber the experts of every
layer so that the contiguous blocks of ``E / ep`` experts that land on each EP rank carry equal load, and permute the
router rows and the expert weights accordingly (the model's function is unchanged).

    python -m gcore_b200.tools.moe_expert_permute --hf-dir in --out-dir out --loads loads.json --ep 8
"""
from __future__ import annotations

import argparse
import json
import os
import re
from typing import Dict, List, Sequence

import torch


def balanced_partition(loads: Sequence[float], parts: int) -> List[List[int]]:
    """Recursive balanced bisection with equal cardinality: split the experts into two halves of equal size whose
    loads are as close as possible (greedy on the sorted list, then pairwise swaps), and recurse."""
    idx = list(range(len(loads)))

    def split(ids: List[int], k: int) -> List[List[int]]:
        if k == 1:
            return [ids]
        assert k % 2 == 0 and len(ids) % 2 == 0, "expert count and EP size must be powers of two multiples"
        order = sorted(ids, key=lambda i: -loads[i])
        a, b, la, lb = [], [], 0.0, 0.0
        half = len(ids) // 2
        for i in order:
            if (la <= lb and len(a) < half) or len(b) >= half:
                a.append(i)
                la += loads[i]
            else:
                b.append(i)
                lb += loads[i]
        improved = True
        while improved:
            improved = False
            for x in list(a):
                for y in list(b):
                    d = loads[x] - loads[y]
                    if abs((la - d) - (lb + d)) + 1e-12 < abs(la - lb):
                        a[a.index(x)], b[b.index(y)] = y, x
                        la, lb = la - d, lb + d
                        improved = True
                        break
                if improved:
                    break
        return split(a, k // 2) + split(b, k // 2)

    return split(idx, parts)


def permutation_for_layer(loads: Sequence[float], ep: int) -> List[int]:
    """new_order[j] = old expert id placed at new position j."""
    return [e for part in balanced_partition(loads, ep) for e in sorted(part)]


def imbalance(loads: Sequence[float], order: Sequence[int], ep: int) -> float:
    per = len(order) // ep
    sums = [sum(loads[e] for e in order[r * per:(r + 1) * per]) for r in range(ep)]
    return max(sums) / (sum(sums) / ep)


EXPERT_RE = re.compile(r"(.*\.layers\.(\d+)\.mlp\.experts\.)(\d+)(\..*)")
ROUTER_RE = re.compile(r".*\.layers\.(\d+)\.mlp\.gate\.(weight|e_score_correction_bias)$")


def permute_state_dict(sd: Dict[str, torch.Tensor], orders: Dict[int, List[int]]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        m = EXPERT_RE.match(k)
        if m and int(m.group(2)) in orders:
            order = orders[int(m.group(2))]
            new_pos = order.index(int(m.group(3)))
            out[f"{m.group(1)}{new_pos}{m.group(4)}"] = v
            continue
        r = ROUTER_RE.match(k)
        if r and int(r.group(1)) in orders:
            out[k] = v[torch.tensor(orders[int(r.group(1))])]
            continue
        out[k] = v
    return out


def main(argv=None):
    from ..checkpoint.hf import read_hf_dir
    ap = argparse.ArgumentParser()
    ap.add_argument("--hf-dir", required=True)
    ap.add_argument("--out-dir", required=True)
    ap.add_argument("--loads", required=True, help="json: {layer index: [tokens per expert]}")
    ap.add_argument("--ep", type=int, required=True)
    a = ap.parse_args(argv)
    loads = {int(k): v for k, v in json.load(open(a.loads)).items()}
    orders = {l: permutation_for_layer(v, a.ep) for l, v in loads.items()}
    sd = permute_state_dict(read_hf_dir(a.hf_dir), orders)
    os.makedirs(a.out_dir, exist_ok=True)
    from safetensors.torch import save_file
    save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(a.out_dir, "model.safetensors"))
    json.dump({str(k): v for k, v in orders.items()}, open(os.path.join(a.out_dir, "expert_permutation.json"), "w"))
    for l, v in loads.items():
        print(f"layer {l}: imbalance {imbalance(v, list(range(len(v))), a.ep):.3f} -> {imbalance(v, orders[l], a.ep):.3f}")


if __name__ == "__main__":
    main()
