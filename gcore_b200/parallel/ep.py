"""Expert-parallel token exchange (NCCL / gloo path).

Each EP rank owns ``E / ep`` experts.  A forward pass is: sort (token, k) pairs by destination rank -> exchange
per-rank per-expert counts (one small all-to-all) -> uneven all-to-all of the token rows and their local expert
ids -> expert-sorted padded layout -> grouped GEMMs -> reverse all-to-all -> weighted sum over k.  The autograd
transpose of an uneven all-to-all is the all-to-all with split sizes swapped, as in the reference
(gpatch_v4/models/deepseek_v4/a2a.py:23-134).  This is the unfused twin of the peer-memory dispatch kernel and the
oracle for it.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from ..core import parallel_state as ps


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits: List[int], in_splits: List[int], group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = torch.empty((sum(out_splits),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty((sum(ctx.in_splits),) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return out, None, None, None


def all_to_all_uneven(x, out_splits, in_splits, group):
    return _AllToAll.apply(x, out_splits, in_splits, group)


CHECK_A2A = {"enabled": False}   # switched on by ``debug.check_a2a_legality``: every exchange is validated first


def check_a2a_legality(in_splits, out_splits, group):
    """Debug check: every rank's send sizes must equal its peers' receive sizes
    (gpatch_v4/utils/dynamic_cp_utils.py:441-555 does the same before a fused reroute)."""
    n = dist.get_world_size(group)
    mine = [list(in_splits), list(out_splits)]
    allv = [None] * n
    dist.all_gather_object(allv, mine, group=group)
    r = dist.get_rank(group)
    for peer in range(n):
        if allv[peer][0][r] != out_splits[peer]:
            raise RuntimeError(f"all-to-all mismatch: rank {peer} sends {allv[peer][0][r]} rows to rank {r}, "
                               f"which expects {out_splits[peer]}")


def ep_moe_forward(layer, x, idx, w):
    """``layer``: MoELayer; x [T, H]; idx / w [T, K].  Returns the combined expert output [T, H]."""
    from ..models.moe import build_dispatch_plan, padded_rows_bound
    group = ps.get_expert_model_parallel_group()
    ep = dist.get_world_size(group)
    T, H = x.shape
    K = idx.shape[1]
    E_local = layer.num_local
    from .ep_fused import fused_ep_moe_forward, get_fused_ep
    fe = get_fused_ep(group, H, E_local * ep, K, T, x)
    if fe is not None:
        return fused_ep_moe_forward(fe, layer, x, idx, w)
    flat_e = idx.reshape(-1)
    dest_rank = flat_e // E_local
    order = torch.argsort(dest_rank * (E_local * ep) + flat_e, stable=True)  # by rank, then by expert
    token_of = torch.arange(T, device=x.device).repeat_interleave(K)
    send_rows = x[token_of[order]]
    send_e = (flat_e[order] % E_local)
    # counts [ep, E_local] -> exchange so that every rank knows what it receives per (source, local expert)
    cnt = torch.bincount(flat_e, minlength=E_local * ep).view(ep, E_local)
    recv_cnt = torch.empty_like(cnt)
    dist.all_to_all_single(recv_cnt, cnt, group=group)
    in_splits = cnt.sum(1).tolist()       # rows this rank sends to each peer (host sync, like the reference)
    out_splits = recv_cnt.sum(1).tolist()  # rows this rank receives from each peer
    if CHECK_A2A["enabled"]:               # debug.check_a2a_legality
        check_a2a_legality(in_splits, out_splits, group)
    recv_rows = all_to_all_uneven(send_rows, out_splits, in_splits, group)
    recv_e = torch.empty(sum(out_splits), dtype=send_e.dtype, device=x.device)
    dist.all_to_all_single(recv_e, send_e.contiguous(), out_splits, in_splits, group=group)
    # local expert-sorted padded layout
    dest, offsets = build_dispatch_plan(recv_e, E_local)
    rows = padded_rows_bound(recv_rows.shape[0], E_local)
    x_perm = torch.zeros(rows, H, dtype=x.dtype, device=x.device).index_copy(0, dest, recv_rows)
    y_perm = layer.experts(x_perm, offsets)
    y_rows = y_perm[dest]
    back = all_to_all_uneven(y_rows, in_splits, out_splits, group)  # rows return in `order`
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    y = back[inv].view(T, K, H)
    return (y * w.to(x.dtype)[:, :, None]).sum(1)
