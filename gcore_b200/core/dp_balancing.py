"""Batch shaping across data-parallel ranks and inside a rank.

* ``rebalance_across_dp_ranks`` — every rank contributes its samples' lengths, one Karmarkar-Karp partition assigns
  samples to ranks so that token counts are even, samples move rank-to-rank, and ``restore_original_order`` brings
  results (log-probs, values) back to the rank and slot they came from (gpatch_v4/core/dp_balancing.py:27-572).
  Samples travel as one flat byte buffer per (source, destination) pair through a single uneven all-to-all.
* ``smart_pad_buckets`` — orders samples by length into buckets so that padded / packed micro-batches waste little,
  with the inverse permutation for restoring (gpatch_v4/core/smart_pad_helper.py:300-1044).
* ``dynamic_micro_batches`` — token-budget micro-batches (first-fit decreasing).
"""
from __future__ import annotations

import io
import pickle
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

from .packing import ffd_pack, kk_partition


def compute_partition_plan(all_lengths: List[List[int]], equal_size: bool = False) -> List[List[Tuple[int, int]]]:
    """all_lengths[r][i] = length of sample i on rank r  ->  plan[dest] = list of (source rank, index)."""
    flat = [(r, i, ln) for r, lens in enumerate(all_lengths) for i, ln in enumerate(lens)]
    parts = kk_partition([ln for _, _, ln in flat], len(all_lengths), equal_size=equal_size)
    return [[(flat[j][0], flat[j][1]) for j in sorted(p)] for p in parts]


def _ser(samples: List[dict]) -> torch.Tensor:
    buf = io.BytesIO()
    pickle.dump(samples, buf, protocol=pickle.HIGHEST_PROTOCOL)
    return torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8)


def _de(t: torch.Tensor) -> List[dict]:
    return pickle.loads(t.cpu().numpy().tobytes()) if t.numel() else []


def _exchange(outgoing: List[List[dict]], group) -> List[List[dict]]:
    """outgoing[d] = samples for rank d -> incoming[s] = samples from rank s (one size exchange + one byte a2a)."""
    n = dist.get_world_size(group)
    dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
    bufs = [_ser(o) if o else torch.empty(0, dtype=torch.uint8) for o in outgoing]
    send_sizes = torch.tensor([b.numel() for b in bufs], dtype=torch.int64, device=dev)
    recv_sizes = torch.empty_like(send_sizes)
    dist.all_to_all_single(recv_sizes, send_sizes, group=group)
    send = torch.cat(bufs).to(dev) if sum(b.numel() for b in bufs) else torch.empty(0, dtype=torch.uint8, device=dev)
    rs = recv_sizes.tolist()
    recv = torch.empty(sum(rs), dtype=torch.uint8, device=dev)
    dist.all_to_all_single(recv, send, rs, send_sizes.tolist(), group=group)
    out, o = [], 0
    for s in rs:
        out.append(_de(recv[o:o + s]))
        o += s
    return out


def rebalance_across_dp_ranks(samples: List[dict], group, length_key: str = "tokens", equal_size: bool = False):
    """Returns (balanced samples for this rank, restore plan)."""
    n, rank = dist.get_world_size(group), dist.get_rank(group)
    lens = [len(s[length_key]) for s in samples]
    all_lens = [None] * n
    dist.all_gather_object(all_lens, lens, group=group)
    plan = compute_partition_plan(all_lens, equal_size)
    outgoing = [[] for _ in range(n)]
    for d in range(n):
        for src, i in plan[d]:
            if src == rank:
                outgoing[d].append(dict(samples[i], _origin=(rank, i)))
    incoming = _exchange(outgoing, group)
    mine = [s for part in incoming for s in part]
    return mine, dict(n_original=len(samples))


def restore_original_order(samples: List[dict], restore: dict, group, keys: Sequence[str] = ()) -> List[dict]:
    """Sends every sample (or only ``keys`` of it) back to the rank it came from, in its original slot."""
    n = dist.get_world_size(group)
    outgoing = [[] for _ in range(n)]
    for s in samples:
        src, i = s["_origin"]
        payload = {k: s[k] for k in keys} if keys else {k: v for k, v in s.items() if k != "_origin"}
        payload["_slot"] = i
        outgoing[src].append(payload)
    incoming = _exchange(outgoing, group)
    out = [None] * restore["n_original"]
    for part in incoming:
        for s in part:
            out[s.pop("_slot")] = s
    assert all(o is not None for o in out), "a sample did not return from rebalancing"
    return out


def smart_pad_buckets(lengths: Sequence[int], bucket_size: int) -> Tuple[List[List[int]], List[int]]:
    """Sort by length (descending), cut into buckets of ``bucket_size`` samples.  Returns (buckets of indices,
    inverse permutation such that ``flat[inverse[i]]`` is original sample i)."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    buckets = [order[i:i + bucket_size] for i in range(0, len(order), bucket_size)]
    inverse = [0] * len(order)
    for pos, i in enumerate(order):
        inverse[i] = pos
    return buckets, inverse


def padding_waste(lengths: Sequence[int], buckets: List[List[int]]) -> float:
    """Fraction of padded positions if every bucket were padded to its longest member."""
    used = sum(lengths)
    padded = sum(max(lengths[i] for i in b) * len(b) for b in buckets if b)
    return 1.0 - used / max(padded, 1)


def dynamic_micro_batches(lengths: Sequence[int], max_tokens: int) -> List[List[int]]:
    return ffd_pack(lengths, max_tokens)
