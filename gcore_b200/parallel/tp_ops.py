"""Autograd-aware tensor-parallel / sequence-parallel collectives and the eager vocab-parallel log-prob + entropy.

These are the unfused NCCL (or gloo) twins of the fused kernels: the call sites match where Megatron-Core issues
them for the reference (column-parallel: all-gather -> GEMM, row-parallel: GEMM -> reduce-scatter, configured in
gpatch_v4/training_backend/megatron_backend/mixin.py:404-410; vocab parallel CE: gpatch_v4/utils/training_utils.py:1139-1208, gpatch_v4/training_backend/vocab_parallel_entropy.py:12-81).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _ws(group):
    return dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1


def all_gather_dim0(x: torch.Tensor, group) -> torch.Tensor:
    n = _ws(group)
    if n == 1:
        return x
    out = torch.empty((x.shape[0] * n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def reduce_scatter_dim0(x: torch.Tensor, group) -> torch.Tensor:
    n = _ws(group)
    if n == 1:
        return x
    assert x.shape[0] % n == 0
    out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
    return out


class _GatherFromSP(torch.autograd.Function):
    """fwd: all-gather along tokens; bwd: reduce-scatter (the gathered tensor feeds a column-parallel GEMM)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_dim0(g, ctx.group), None


class _ReduceScatterToSP(torch.autograd.Function):
    """fwd: reduce-scatter along tokens (output of a row-parallel GEMM); bwd: all-gather."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return reduce_scatter_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        return all_gather_dim0(g, ctx.group), None


class _CopyToTP(torch.autograd.Function):
    """fwd: identity; bwd: all-reduce."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        if _ws(ctx.group) > 1:
            g = g.contiguous()
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """fwd: all-reduce; bwd: identity."""

    @staticmethod
    def forward(ctx, x, group):
        if _ws(group) > 1:
            x = x.contiguous()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _ScatterToSP(torch.autograd.Function):
    """fwd: keep this rank's token slice; bwd: all-gather."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = _ws(group)
        if n == 1:
            return x
        r = dist.get_rank(group)
        c = x.shape[0] // n
        return x[r * c:(r + 1) * c].contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather_dim0(g, ctx.group), None


class _SliceOfGathered(torch.autograd.Function):
    """fwd: this rank's token slice of a tensor that came out of ``gather_from_sequence_parallel``; bwd: the gradient
    in that slice, zeros elsewhere.  The gather's own backward sums the ranks' gradients (reduce-scatter), so a branch
    that re-shards its output must hand back only its own share; ``scatter_to_sequence_parallel`` (all-gather in the
    backward) is for tensors that every rank computed in full, such as the output of the vocabulary-parallel
    embedding."""

    @staticmethod
    def forward(ctx, x, group):
        n = _ws(group)
        r = dist.get_rank(group)
        c = x.shape[0] // n
        ctx.meta = (r * c, c, x.shape[0])
        return x[r * c:(r + 1) * c].contiguous()

    @staticmethod
    def backward(ctx, g):
        lo, c, total = ctx.meta
        full = g.new_zeros((total,) + tuple(g.shape[1:]))
        full[lo:lo + c] = g
        return full, None


class _ScaleGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, factor):
        ctx.factor = factor
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g * ctx.factor, None


def replicated_consumer_of_gathered(x, group):
    """Marks a tensor that came out of ``gather_from_sequence_parallel`` as the input of a computation every TP rank
    repeats in full (a replicated head): each rank then sends back the whole gradient, and the gather's backward would
    add the copies up, so each copy is scaled by 1 / TP size."""
    n = _ws(group)
    return _ScaleGrad.apply(x, 1.0 / n) if n > 1 else x


def slice_of_gathered(x, group):
    return _SliceOfGathered.apply(x, group) if _ws(group) > 1 else x


def gather_from_sequence_parallel(x, group):
    return _GatherFromSP.apply(x, group) if _ws(group) > 1 else x


def reduce_scatter_to_sequence_parallel(x, group):
    return _ReduceScatterToSP.apply(x, group) if _ws(group) > 1 else x


def copy_to_tensor_parallel(x, group):
    return _CopyToTP.apply(x, group) if _ws(group) > 1 else x


def reduce_from_tensor_parallel(x, group):
    return _ReduceFromTP.apply(x, group) if _ws(group) > 1 else x


def scatter_to_sequence_parallel(x, group):
    return _ScatterToSP.apply(x, group) if _ws(group) > 1 else x


# ------------------------------------------------------------------------------------------------ vocab parallel
class _VocabParallelLogprobEntropy(torch.autograd.Function):
    """z: [T, V_local] fp32 (already divided by temperature).  Three reductions over TP: max, sum-exp and the
    pair (sum p*z, target z) packed in one buffer."""

    @staticmethod
    def forward(ctx, z, targets, vocab_start, group):
        V = z.shape[-1]
        m = z.max(-1).values
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(z - m[:, None])
        packed = torch.empty(3, z.shape[0], dtype=torch.float32, device=z.device)
        packed[0] = e.sum(-1)
        packed[1] = (e * z).sum(-1)
        local = targets - vocab_start
        mine = (local >= 0) & (local < V)
        idx = local.clamp(0, V - 1)
        packed[2] = torch.where(mine, z.gather(-1, idx[:, None]).squeeze(-1), torch.zeros_like(m))
        dist.all_reduce(packed, group=group)
        s, sz, zt = packed[0], packed[1], packed[2]
        lse = m + torch.log(s)
        logp = zt - lse
        ent = lse - sz / s
        ctx.save_for_backward(z, lse, ent, idx, mine)
        return logp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        z, lse, ent, idx, mine = ctx.saved_tensors
        p = torch.exp(z - lse[:, None])
        d = -g_lp[:, None] * p
        d.scatter_add_(-1, idx[:, None], (g_lp * mine.float())[:, None])
        if g_ent is not None:
            d = d - g_ent[:, None] * p * (z - lse[:, None] + ent[:, None])
        return d, None, None, None


def vocab_parallel_logprob_entropy(z, targets, vocab_start, group):
    if _ws(group) == 1:
        lse = torch.logsumexp(z, -1)
        logp = z.gather(-1, targets[:, None]).squeeze(-1) - lse
        p = torch.softmax(z, -1)
        return logp, lse - (p * z).sum(-1)
    return _VocabParallelLogprobEntropy.apply(z, targets, vocab_start, group)


class _VocabParallelEmbedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, vocab_start, group):
        V = weight.shape[0]
        local = ids - vocab_start
        mine = (local >= 0) & (local < V)
        idx = local.clamp(0, V - 1)
        out = weight[idx] * mine[:, None].to(weight.dtype)
        if _ws(group) > 1:
            dist.all_reduce(out, group=group)
        ctx.save_for_backward(idx, mine)
        ctx.vshape = weight.shape
        return out

    @staticmethod
    def backward(ctx, g):
        idx, mine = ctx.saved_tensors
        dw = torch.zeros(ctx.vshape, dtype=torch.float32, device=g.device)
        dw.index_add_(0, idx, g.float() * mine[:, None].float())
        return None, dw.to(g.dtype), None, None


def vocab_parallel_embedding(ids, weight, vocab_start, group):
    """Embedding lookup with the table sharded over the vocabulary; out-of-shard ids contribute zero and the
    partial rows are summed over the TP group."""
    if _ws(group) == 1:
        return torch.nn.functional.embedding(ids, weight)
    return _VocabParallelEmbedding.apply(ids, weight, vocab_start, group)
