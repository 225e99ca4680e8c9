"""Context parallelism for packed (THD) batches.

Sharding: the packed token stream of a micro-batch (documents back to back, padded to a multiple of ``cp``) is cut
into ``cp`` contiguous chunks; rank ``r`` owns tokens ``[r*s, (r+1)*s)`` and every per-token tensor (ids, positions,
targets, masks) is sliced the same way, so everything outside attention is embarrassingly parallel and the loss is a
sum over ranks.  Attention needs, for the queries a rank owns, the keys/values of the same document that precede them:
rows ``[k0, (r+1)*s)`` of the global stream, where ``k0`` is the start of the first document that reaches into the
rank's chunk (clipped to ``window - 1`` rows before the chunk for sliding-window layers, which turns the exchange into
a neighbour halo).  Because those queries are a suffix of their key range, the single-GPU varlen kernel computes the
shard exactly when given per-document ``(cu_q, cu_k)`` with ``lk >= lq``.

Key/value acquisition and the return of dK/dV run over NVLink peer memory (``gk_peer_rows`` in ``ops/csrc/comm.cu``):
each rank publishes its K/V rows in a symmetric buffer, pulls the foreign rows it needs straight from their owners
into local memory, and in the backward pass every owner pulls and sums (fixed order, deterministic) the partial
dK/dV rows that later ranks computed for it.  The plan (who pulls which rows from whom) is derived on the host from the
document boundaries, which every rank of the group knows.  The gloo / NCCL twin uses a differentiable all-gather.

Reference behaviour: zigzag / contiguous CP gathers with reduce-scatter backward (gpatch_v4/core/mappings.py:19-355),
contiguous CP with a sliding-window halo (gpatch_v4/models/deepseek_v4/cp.py:51-176,514-548), all-gather-KV varlen
attention (tests/test_gpatch_v4/test_welm_v45_myfa_packed_cp.py:1-14).
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import attention as attn_ops

LAUNCHES = {"cp": 0}


# ------------------------------------------------------------------------------------------------ planning (host)
@dataclass
class CPPlan:
    k0: int                      # first global row of the gathered K/V range
    rows: int                    # gathered rows = (rank + 1) * s - k0
    cu_q: List[int]
    cu_k: List[int]
    max_q: int
    max_k: int
    pulls: List[Tuple[int, int, int, int]]    # (source rank, source local row, destination row, n rows)
    returns: List[Tuple[int, int, int, int]]  # (source rank, row inside its gathered range, local row, n rows)


def _first_row(cu: List[int], a: int, b: int, window: int) -> int:
    """Start of the gathered key range of the rank that owns tokens [a, b)."""
    for d in range(len(cu) - 1):
        ds, de = cu[d], cu[d + 1]
        if de > a and ds < b:
            ks = ds
            if window and window > 0:
                ks = max(ds, max(ds, a) - (window - 1))
            return min(ks, a)
    return a


def plan_cp(cu: List[int], s: int, cp: int, rank: int, window: int = 0) -> CPPlan:
    """``cu``: document boundaries of the whole packed stream (cu[-1] == cp * s)."""
    assert cu[-1] == cp * s, (cu[-1], cp, s)
    a, b = rank * s, (rank + 1) * s
    k0 = _first_row(cu, a, b, window)
    cu_q, cu_k = [0], [0]
    for d in range(len(cu) - 1):
        ds, de = cu[d], cu[d + 1]
        qs, qe = max(ds, a), min(de, b)
        if qs >= qe:
            continue
        ks = max(ds, k0)  # only the first document can start before `a`; later ones start where the previous ended
        assert ks - k0 == cu_k[-1], "key ranges of consecutive documents must be contiguous"
        cu_q.append(qe - a)
        cu_k.append(qe - k0)
    max_q = max(cu_q[i + 1] - cu_q[i] for i in range(len(cu_q) - 1))
    max_k = max(cu_k[i + 1] - cu_k[i] for i in range(len(cu_k) - 1))
    pulls = []
    for r in range(rank + 1):
        lo, hi = max(k0, r * s), min(b, (r + 1) * s)
        if lo < hi:
            pulls.append((r, lo - r * s, lo - k0, hi - lo))
    returns = []
    for r in range(rank, cp):
        k0r = k0 if r == rank else _first_row(cu, r * s, (r + 1) * s, window)
        lo = max(a, k0r)
        if lo < b:
            returns.append((r, lo - k0r, lo - a, b - lo))
    return CPPlan(k0, b - k0, cu_q, cu_k, max_q, max_k, pulls, returns)


@dataclass
class CPContext:
    """What a model forward needs to run attention on one CP shard of a packed micro-batch.  Passed to the model in
    place of ``cu_seqlens``."""
    group: object
    cp: int
    rank: int
    cu_global: List[int]
    s: int
    device: torch.device
    _plans: Dict[int, CPPlan] = field(default_factory=dict)
    _tensors: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)

    def plan(self, window: int) -> CPPlan:
        w = int(window or 0)
        if w not in self._plans:
            self._plans[w] = plan_cp(self.cu_global, self.s, self.cp, self.rank, w)
        return self._plans[w]

    def cu_tensors(self, window: int):
        w = int(window or 0)
        if w not in self._tensors:
            p = self.plan(w)
            self._tensors[w] = (torch.tensor(p.cu_q, dtype=torch.int32, device=self.device),
                                torch.tensor(p.cu_k, dtype=torch.int32, device=self.device))
        return self._tensors[w]


def shard_packed_batch(mb, group, device, halo: int = 0):
    """Slices every per-token tensor of a host-side ``PackedBatch`` to this rank's contiguous chunk and attaches the
    ``CPContext``.  The batch must already be padded to a multiple of the group size.  ``halo`` > 0 also keeps the
    ids, targets, mask and sequence index of that many positions behind the chunk (look-ahead of the multi-token
    prediction blocks; sequence index -1 past the end of the stream)."""
    from dataclasses import replace
    cp, rank = dist.get_world_size(group), dist.get_rank(group)
    T = mb.tokens.numel()
    assert T % cp == 0, "packed batch must be padded to a multiple of the context-parallel size"
    s = T // cp
    sl = slice(rank * s, (rank + 1) * s)
    ctx = CPContext(group, cp, rank, [int(c) for c in mb.cu_seqlens.tolist()], s, torch.device(device))
    out = replace(mb, tokens=mb.tokens[sl], position_ids=mb.position_ids[sl], targets=mb.targets[sl],
                  loss_mask=mb.loss_mask[sl], seq_ids=mb.seq_ids[sl],
                  fields={k: v[sl] for k, v in mb.fields.items()})
    out.cp_ctx = ctx
    if halo > 0:
        lo, hi = (rank + 1) * s, min((rank + 1) * s + halo, T)

        def behind(x, fill):
            pad = x.new_full((halo - (hi - lo),), fill)
            return torch.cat([x[lo:hi], pad])
        out.halo = {"tokens": behind(mb.tokens, 0), "targets": behind(mb.targets, 0),
                    "loss_mask": behind(mb.loss_mask, 0), "seq_ids": behind(mb.seq_ids, -1)}
    return out


# ------------------------------------------------------------------------------------------------ peer-memory runtime
class PeerCP:
    """Symmetric K/V and dK/dV staging buffers of one context-parallel group (double-buffered by call parity: a rank
    can be at most one exchange ahead of its peers, because every exchange contains a group barrier)."""

    def __init__(self, group, width: int, s_max: int, device):
        from .symm import SymmBuffer
        self.group, self.width, self.s_max = group, width, s_max
        self.cp, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = device
        self.kv = [SymmBuffer(s_max * width, torch.bfloat16, group, device) for _ in range(2)]
        self.dkv = [SymmBuffer(self.cp * s_max * width, torch.bfloat16, group, device) for _ in range(2)]
        self.flags = SymmBuffer(64 * 8, torch.int32, group, device)
        self.flags.t.zero_()
        self.flag_ptrs = torch.tensor(self.flags.ptrs, dtype=torch.int64, device=device)
        self.epoch = 0
        self.calls = 0
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def _barrier(self):
        self.epoch += 1
        LAUNCHES["cp"] += 1
        _lib.check(_lib.kernels().gk_peer_barrier(_lib.ptr(self.flag_ptrs), self.rank, self.cp, 0, self.epoch,
                                                  _lib.ptr(_lib.err_flag(self.device)), _lib.stream_ptr()), "cp_barrier")

    def _rows(self, dst: torch.Tensor, segs: List[Tuple[int, int, int]]):
        arr = (ctypes.c_ulonglong * (3 * len(segs)))(*[v for seg in segs for v in seg])
        LAUNCHES["cp"] += 1
        _lib.check(_lib.kernels().gk_peer_rows(_lib.ptr(dst), dst.numel(), len(segs), arr, _lib.stream_ptr()),
                   "peer_rows")

    def gather_kv(self, k: torch.Tensor, v: torch.Tensor, plan: CPPlan) -> torch.Tensor:
        """k, v [s, Hk, D] -> [rows, 2*Hk, D]: the K/V rows this rank's queries can see, pulled from their owners."""
        s, hk, D = k.shape
        W = self.width
        assert 2 * hk * D == W and s <= self.s_max
        buf = self.kv[self.calls & 1]
        stage = buf.t[:s * W].view(s, 2 * hk, D)
        stage[:, :hk].copy_(k)
        stage[:, hk:].copy_(v)
        self._barrier()
        out = torch.empty(plan.rows, 2 * hk, D, dtype=torch.bfloat16, device=self.device)
        segs = [(buf.ptrs[r] + src_row * W * 2, dst_row * W, (dst_row + n) * W) for r, src_row, dst_row, n in plan.pulls]
        self._rows(out, segs)
        self.calls += 1
        return out

    def return_dkv(self, dkv: torch.Tensor, plan: CPPlan, s: int) -> torch.Tensor:
        """dkv [rows, 2*Hk, D] partial gradients for the gathered range -> [s, 2*Hk, D] summed over every rank that
        attended to this rank's rows."""
        W = self.width
        buf = self.dkv[self.calls & 1]
        assert dkv.numel() <= buf.t.numel()
        buf.t[:dkv.numel()].copy_(dkv.reshape(-1))
        self._barrier()
        out = torch.empty(s, dkv.shape[1], dkv.shape[2], dtype=torch.bfloat16, device=self.device)
        segs = [(buf.ptrs[r] + src_row * W * 2, dst_row * W, (dst_row + n) * W) for r, src_row, dst_row, n in plan.returns]
        self._rows(out, segs)
        self.calls += 1
        return out


_PEER: Dict = {}


def _get_peer(ctx: CPContext, width: int, s: int) -> Optional[PeerCP]:
    if ctx.device.type != "cuda" or not _lib.use_native() or os.environ.get("GCORE_FUSED_CP", "1") == "0":
        return None
    if ctx.cp > 8 or not hasattr(_lib.kernels(), "gk_peer_rows"):
        return None
    key = (id(ctx.group), width)
    peer = _PEER.get(key)
    if peer is None or peer.s_max < s:
        s_max = int(os.environ.get("GCORE_CP_MAX_TOKENS", "0")) or max(s, 4096)
        s_max = max(s_max, s)
        peer = PeerCP(ctx.group, width, s_max, ctx.device)  # collective: s is the same on every rank of the group
        _PEER[key] = peer
    return peer


class _PeerCPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, sinks, cpx: CPContext, peer: PeerCP, window, scale):
        plan = cpx.plan(window)
        cu_q, cu_k = cpx.cu_tensors(window)
        hk = k.shape[1]
        kv = peer.gather_kv(k, v, plan)
        kg, vg = kv[:, :hk], kv[:, hk:]
        out, lse = attn_ops._native_fwd(q, kg, vg, cu_q, cu_k, plan.max_q, True, window, sinks, scale)
        ctx.save_for_backward(q, kv, out, lse, sinks if sinks is not None else torch.empty(0))
        ctx.misc = (cpx, peer, window, scale, sinks is not None, k.shape[0])
        return out

    @staticmethod
    def backward(ctx, do):
        q, kv, out, lse, sinks = ctx.saved_tensors
        cpx, peer, window, scale, has_sinks, s = ctx.misc
        plan = cpx.plan(window)
        cu_q, cu_k = cpx.cu_tensors(window)
        hk = kv.shape[1] // 2
        from ..ops.attention_bwd import attn_bwd
        dq, dk, dv, dsinks = attn_bwd(do.contiguous(), q, kv[:, :hk], kv[:, hk:], out, lse, sinks if has_sinks else None,
                                      cu_q, cu_k, plan.max_q, plan.max_k, True, window, scale)
        dkv = peer.return_dkv(torch.cat([dk, dv], dim=1), plan, s)
        return dq, dkv[:, :hk], dkv[:, hk:], dsinks, None, None, None, None


def cp_attention(q, k, v, cpx: CPContext, window=0, sinks=None, scale=None):
    """Causal varlen attention of this rank's query shard ``q`` [s, Hq, D] against the document prefixes that live on
    this and earlier ranks.  ``k`` / ``v`` [s, Hk, D] are this rank's rows."""
    import math
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s, hk, D = k.shape
    peer = _get_peer(cpx, 2 * hk * D, s) if (q.dtype == torch.bfloat16 and D in (64, 128)) else None
    if peer is not None:
        return _PeerCPAttention.apply(q.contiguous(), k, v, sinks, cpx, peer, int(window or 0), scale)
    # collective twin (gloo / NCCL): differentiable all-gather of K and V, then the same per-document call
    plan = cpx.plan(window)
    cu_q, cu_k = cpx.cu_tensors(window)
    kg = gather_from_cp(k.contiguous(), cpx.group)[plan.k0:plan.k0 + plan.rows]
    vg = gather_from_cp(v.contiguous(), cpx.group)[plan.k0:plan.k0 + plan.rows]
    return attn_ops.flash_attn_varlen(q, kg.contiguous(), vg.contiguous(), cu_q, cu_k, plan.max_q, plan.max_k,
                                      causal=True, window=window, sinks=sinks, scale=scale)


# ------------------------------------------------------------------------------------------------ mappings
def zigzag_order(cp: int) -> List[int]:
    """Chunk order after a rank-major gather of zigzag shards: rank r holds chunks r and 2cp-1-r."""
    order = []
    for r in range(cp):
        order += [r, 2 * cp - 1 - r]
    return order


def split_for_cp(x: torch.Tensor, cp: int, rank: int, dim: int = 0, zigzag: bool = False) -> torch.Tensor:
    """This rank's shard of ``x`` along ``dim``: one contiguous chunk, or chunks ``rank`` and ``2cp-1-rank`` of
    ``2cp`` (zigzag, balances causal work; gpatch_v4/utils/training_utils.py:450-498)."""
    if not zigzag:
        return x.chunk(cp, dim=dim)[rank].contiguous()
    ch = x.chunk(2 * cp, dim=dim)
    return torch.cat([ch[rank], ch[2 * cp - 1 - rank]], dim=dim)


class _GatherFromCP(torch.autograd.Function):
    """All-gather along ``dim`` (optionally undoing the zigzag placement); backward keeps this rank's slice of the
    gradient summed over ranks (reduce-scatter), scaled by ``grad_scale`` (1/cp gives the reference's AVG)."""

    @staticmethod
    def forward(ctx, x, group, dim, zigzag, grad_scale):
        cp = dist.get_world_size(group)
        ctx.misc = (group, dim, zigzag, grad_scale, cp, dist.get_rank(group))
        parts = [torch.empty_like(x) for _ in range(cp)]
        dist.all_gather(parts, x.contiguous(), group=group)
        if not zigzag:
            return torch.cat(parts, dim=dim)
        chunks = [None] * (2 * cp)
        for r, p in enumerate(parts):
            a, b = p.chunk(2, dim=dim)
            chunks[r], chunks[2 * cp - 1 - r] = a, b
        return torch.cat(chunks, dim=dim)

    @staticmethod
    def backward(ctx, g):
        group, dim, zigzag, grad_scale, cp, rank = ctx.misc
        g = g.contiguous()
        if zigzag:
            ch = g.chunk(2 * cp, dim=dim)
            parts = [torch.cat([ch[r], ch[2 * cp - 1 - r]], dim=dim).contiguous() for r in range(cp)]
        else:
            parts = [p.contiguous() for p in g.chunk(cp, dim=dim)]
        out = torch.empty_like(parts[rank])
        dist.reduce_scatter(out, parts, group=group)
        if grad_scale != 1.0:
            out = out * grad_scale
        return out, None, None, None, None


def gather_from_cp(x, group, dim: int = 0, zigzag: bool = False, grad_scale: float = 1.0):
    if group is None or dist.get_world_size(group) == 1:
        return x
    return _GatherFromCP.apply(x, group, dim, zigzag, grad_scale)


class _AllReduceIdentityBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def all_reduce_cp(x, group):
    """Sum over the CP group whose backward is the identity (gpatch_v4/core/mappings.py:19-47)."""
    if group is None or dist.get_world_size(group) == 1:
        return x
    return _AllReduceIdentityBwd.apply(x, group)
