"""Dynamic context parallelism: per-sequence CP group sizes inside a shared DP x CP pool of ranks.

Long sequences get a large CP group, short ones a small group or a single rank, so that every rank of the pool holds
about the same number of tokens per micro-step (gpatch_v4/utils/dynamic_cp_utils.py:74-2021,
docs/source/dynamic_cp.md).  The pieces:

* ``schedule``            - global plan from all sequence lengths: CP size per sample (smallest power of two whose
                            shards fit ``max_tokens_per_rank``), then first-fit packing of (sample, rank block) pairs
                            into micro-steps; rank blocks are aligned power-of-two ranges of the pool, one process
                            group per block (``build_block_groups``).
* ``reroute_samples``     - moves every sample to all ranks of its block with ONE byte all-to-all for all fields
                            (the reference's fused uint8 reroute, dynamic_cp_utils.py:1109-1280).
* ``reverse_reroute``     - one all-to-all that returns per-sample results (log-probs) from the block's first rank
                            to the rank the sample came from (dynamic_cp_utils.py:1898-2021).
* inside a block the static machinery applies: ``parallel.cp.CPContext`` over the block's group.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch.distributed as dist

from ..core.dp_balancing import _exchange


@dataclass
class Assignment:
    gid: int          # global sample id (position in the concatenation of every rank's samples)
    block_start: int  # first pool rank of the CP block
    cp_size: int
    step: int         # micro-step index


def cp_size_for(length: int, max_tokens_per_rank: int, pool: int, min_cp: int = 1) -> int:
    need = max(min_cp, -(-length // max_tokens_per_rank))
    cp = 1
    while cp < need:
        cp *= 2
    if cp > pool:
        raise ValueError(f"a sequence of {length} tokens needs CP {cp} but the pool has {pool} ranks; raise "
                         f"max_seqlen_per_dp_cp_rank ({max_tokens_per_rank})")
    return cp


def schedule(global_lens: Sequence[int], pool: int, max_tokens_per_rank: int, min_cp: int = 1) -> List[Assignment]:
    """Deterministic on every rank (pure function of the gathered lengths)."""
    assert pool & (pool - 1) == 0, "the DP x CP pool must be a power of two"
    order = sorted(range(len(global_lens)), key=lambda g: (-global_lens[g], g))
    steps: List[List[int]] = []  # per micro-step: tokens already placed on every pool rank
    out: List[Assignment] = []
    for g in order:
        cp = cp_size_for(global_lens[g], max_tokens_per_rank, pool, min_cp)
        share = -(-global_lens[g] // cp)
        placed = False
        for si, load in enumerate(steps):
            best, best_load = None, None
            for b in range(0, pool, cp):
                peak = max(load[b:b + cp])
                if peak + share <= max_tokens_per_rank and (best is None or peak < best_load):
                    best, best_load = b, peak
            if best is not None:
                for r in range(best, best + cp):
                    load[r] += share
                out.append(Assignment(g, best, cp, si))
                placed = True
                break
        if not placed:
            load = [0] * pool
            for r in range(cp):
                load[r] += share
            steps.append(load)
            out.append(Assignment(g, 0, cp, len(steps) - 1))
    return out


def imbalance(plan: List[Assignment], global_lens: Sequence[int], pool: int) -> float:
    """max over ranks of total tokens / mean."""
    tot = [0.0] * pool
    for a in plan:
        for r in range(a.block_start, a.block_start + a.cp_size):
            tot[r] += global_lens[a.gid] / a.cp_size
    return max(tot) / max(sum(tot) / pool, 1e-9)


def build_block_groups(pool_group) -> Dict[Tuple[int, int], object]:
    """One process group per aligned power-of-two block of the pool: {(start, size): group}.  Collective: every rank
    of the default group must call it (``dist.new_group`` contract)."""
    ranks = dist.get_process_group_ranks(pool_group)
    n = len(ranks)
    groups = {}
    size = 2
    while size <= n:
        for start in range(0, n, size):
            groups[(start, size)] = dist.new_group([ranks[i] for i in range(start, start + size)],
                                                   backend=dist.get_backend(pool_group))
        size *= 2
    return groups


def gather_lengths(samples: List[dict], group, key: str = "tokens") -> Tuple[List[int], List[int]]:
    """-> (all lengths in rank order, offset of every rank's first sample)."""
    n = dist.get_world_size(group)
    lens = [len(s[key]) for s in samples]
    allv = [None] * n
    dist.all_gather_object(allv, lens, group=group)
    offsets = [0]
    for l in allv:
        offsets.append(offsets[-1] + len(l))
    return [x for l in allv for x in l], offsets


def reroute_samples(samples: List[dict], plan: List[Assignment], offsets: List[int], group) -> List[List[dict]]:
    """Returns, per micro-step, the samples this rank takes part in (whole samples; the CP shard is cut at pack
    time).  Every sample carries ``_gid``, ``_origin`` and its ``Assignment``."""
    n, rank = dist.get_world_size(group), dist.get_rank(group)
    by_gid = {a.gid: a for a in plan}
    outgoing = [[] for _ in range(n)]
    for i, s in enumerate(samples):
        gid = offsets[rank] + i
        a = by_gid[gid]
        for r in range(a.block_start, a.block_start + a.cp_size):
            outgoing[r].append(dict(s, _gid=gid, _origin=rank, _slot=i, _block=(a.block_start, a.cp_size),
                                    _step=a.step))
    incoming = _exchange(outgoing, group)
    nsteps = max((a.step for a in plan), default=-1) + 1
    steps: List[List[dict]] = [[] for _ in range(nsteps)]
    for part in incoming:
        for s in part:
            steps[s["_step"]].append(s)
    for st in steps:
        st.sort(key=lambda s: s["_gid"])
    return steps


def reverse_reroute(results: List[dict], n_original: int, group, keys: Sequence[str] = ("logprobs",)) -> List[dict]:
    """``results``: computed samples held by this rank (any rank of a block may hold them; only the block's first
    rank sends).  Returns this rank's original samples' results in their original order."""
    n, rank = dist.get_world_size(group), dist.get_rank(group)
    outgoing = [[] for _ in range(n)]
    for s in results:
        if s["_block"][0] != rank:
            continue
        payload = {k: s[k] for k in keys if k in s}
        payload["_slot"] = s["_slot"]
        outgoing[s["_origin"]].append(payload)
    incoming = _exchange(outgoing, group)
    out: List[Optional[dict]] = [None] * n_original
    for part in incoming:
        for s in part:
            out[s.pop("_slot")] = s
    assert all(o is not None for o in out), "a sample's result did not come back from its compute block"
    return out
