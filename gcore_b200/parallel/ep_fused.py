"""Expert-parallel dispatch / combine over NVLink peer memory (``ops/csrc/ep_comm.cu``).

``FusedEP`` owns, per expert-parallel group, two symmetric row buffers (tokens arriving at this rank's experts and
expert outputs waiting to be collected), the count tables and the flags.  The autograd pair ``dispatch`` /
``combine`` replaces the count all-to-all, the three uneven all-to-alls, the host-side split computation and the
local permutations of the NCCL path (``parallel/ep.py``; reference: gpatch_v4/models/deepseek_v4/a2a.py:23-134,
modeling_deepseek_v4.py:1221-1289): tokens are written by the sending rank directly to their final expert-sorted row
in the owner's buffer, and collected by the token's owner with the top-k weighted sum in the same pass.  The backward
of each is the other's kernel (scaled push / unweighted pull).  No host synchronisation happens per layer.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from .symm import SymmBuffer

LAUNCHES = {"ep": 0}
SEG = 128


def _ptr_array(*lists):
    flat = [p for l in lists for p in l]
    return (ctypes.c_ulonglong * len(flat))(*flat)


class FusedEP:
    def __init__(self, group, hidden: int, num_experts: int, top_k: int, max_tokens: int, capacity_factor: float = 2.0,
                 device=None):
        self.group = group
        self.ep = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.H, self.E, self.K = hidden, num_experts, top_k
        self.E_local = num_experts // self.ep
        self.max_tokens = max_tokens
        worst = self.ep * max_tokens * top_k
        rows = min(worst, int(capacity_factor * max_tokens * top_k))
        self.R_max = (rows + self.E_local * (SEG - 1) + SEG - 1) // SEG * SEG
        self.recv = SymmBuffer(self.R_max * hidden, torch.bfloat16, group, self.device)
        self.yout = SymmBuffer(self.R_max * hidden, torch.bfloat16, group, self.device)
        self.cnt = SymmBuffer(2 * self.ep * num_experts, torch.int32, group, self.device)
        self.pflags = SymmBuffer(64, torch.int32, group, self.device)
        self.bflags = SymmBuffer(64 * 8, torch.int32, group, self.device)
        for b in (self.cnt, self.pflags, self.bflags):
            b.t.zero_()
        self.plan_ptrs = _ptr_array(self.cnt.ptrs, self.pflags.ptrs)
        self.recv_ptrs = _ptr_array(self.recv.ptrs)
        self.yout_ptrs = _ptr_array(self.yout.ptrs)
        self.bflag_ptrs = torch.tensor(self.bflags.ptrs, dtype=torch.int64, device=self.device)
        self.plan_calls = 0
        self.barrier_epoch = 0
        # call / epoch counters on the device ([0] plans, [1] barriers), advanced by the kernels themselves: the whole
        # dispatch -> experts -> combine sequence can then be captured in a CUDA graph and replayed (decode steps of
        # an expert-parallel rollout engine)
        self.dev_ctr = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.dev_epochs = hasattr(_lib.kernels(), "gk_ep_plan_dev") and hasattr(_lib.kernels(), "gk_peer_barrier_dev")
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def _err(self):
        return _lib.ptr(_lib.err_flag(self.device))

    def barrier(self):
        self.barrier_epoch += 1
        LAUNCHES["ep"] += 1
        if self.dev_epochs:
            _lib.check(_lib.kernels().gk_peer_barrier_dev(_lib.ptr(self.bflag_ptrs), self.rank, self.ep, 0,
                                                          _lib.ptr(self.dev_ctr[1:]), self._err(), _lib.stream_ptr()),
                       "ep_barrier")
            return
        _lib.check(_lib.kernels().gk_peer_barrier(_lib.ptr(self.bflag_ptrs), self.rank, self.ep, 0, self.barrier_epoch,
                                                  self._err(), _lib.stream_ptr()), "ep_barrier")

    def plan(self, idx: torch.Tensor):
        """idx [T, K] global expert ids -> routing state shared by dispatch, combine and their backward passes."""
        T, K = idx.shape
        if T > self.max_tokens:
            raise RuntimeError(f"expert-parallel buffers were sized for {self.max_tokens} tokens per micro-batch, got "
                               f"{T}; set GCORE_EP_MAX_TOKENS")
        flat = idx.reshape(-1)
        n = flat.numel()
        if n <= LOCAL_PLAN_MAX and flat.dtype == torch.int64 and hasattr(_lib.kernels(), "gk_ep_local_plan"):
            # small batches (decode steps): histogram, in-expert positions and the cleared per-call outputs from one
            # single-CTA kernel; all per-call int32 arrays are slices of one allocation
            flat = flat.contiguous()
            buf = torch.empty(3 * n + 2 * self.E + 2 * self.E_local + 1, dtype=torch.int32, device=self.device)
            o = [0, n, 2 * n, 3 * n, 3 * n + self.E, 3 * n + 2 * self.E, 3 * n + 2 * self.E + self.E_local + 1]
            idx32, pos, dst_row, cnt, send_base, offsets, tot_local = (buf[a:b] for a, b in zip(o, o[1:] + [buf.numel()]))
            LAUNCHES["ep"] += 1
            _lib.check(_lib.kernels().gk_ep_local_plan(_lib.ptr(flat), n, self.E, self.E_local, _lib.ptr(idx32),
                                                       _lib.ptr(pos), _lib.ptr(cnt), _lib.ptr(offsets),
                                                       _lib.ptr(tot_local), _lib.stream_ptr()), "ep_local_plan")
            st = dict(T=T, K=K, idx=idx32, pos=pos, cnt=cnt, send_base=send_base, offsets=offsets, tot_local=tot_local,
                      dst_row=dst_row, _keep=(flat, buf))
        else:
            # histogram without a host synchronisation (bincount sizes its output on the host)
            cnt = torch.zeros(self.E, dtype=torch.int64, device=flat.device).scatter_add_(0, flat, torch.ones_like(flat))
            order = torch.argsort(flat, stable=True)
            starts = cnt.cumsum(0) - cnt
            pos = torch.empty_like(flat)
            pos[order] = torch.arange(flat.numel(), device=flat.device) - starts[flat[order]]
            st = dict(T=T, K=K, idx=flat.to(torch.int32), pos=pos.to(torch.int32), cnt=cnt.to(torch.int32),
                      send_base=torch.empty(self.E, dtype=torch.int32, device=self.device),
                      offsets=torch.zeros(self.E_local + 1, dtype=torch.int32, device=self.device),
                      tot_local=torch.zeros(self.E_local, dtype=torch.int32, device=self.device),
                      dst_row=torch.empty(T * K, dtype=torch.int32, device=self.device))
        LAUNCHES["ep"] += 1
        if self.dev_epochs:
            _lib.check(_lib.kernels().gk_ep_plan_dev(_lib.ptr(st["cnt"]), self.plan_ptrs, self.rank, self.ep, self.E, SEG,
                                                     self.R_max, _lib.ptr(self.dev_ctr), _lib.ptr(st["send_base"]),
                                                     _lib.ptr(st["offsets"]), _lib.ptr(st["tot_local"]), self._err(),
                                                     _lib.stream_ptr()), "ep_plan")
        else:
            _lib.check(_lib.kernels().gk_ep_plan(_lib.ptr(st["cnt"]), self.plan_ptrs, self.rank, self.ep, self.E, SEG,
                                                 self.R_max, self.plan_calls, _lib.ptr(st["send_base"]),
                                                 _lib.ptr(st["offsets"]), _lib.ptr(st["tot_local"]), self._err(),
                                                 _lib.stream_ptr()), "ep_plan")
        self.plan_calls += 1
        return st

    def push(self, x: torch.Tensor, scale: Optional[torch.Tensor], st) -> torch.Tensor:
        """Writes every (token, k) row of ``x`` (times ``scale``) to its expert-sorted row on the owning rank, waits
        for everyone's rows and returns a private copy of this rank's receive buffer [R_max, H]."""
        x = x.contiguous()
        LAUNCHES["ep"] += 1
        _lib.check(_lib.kernels().gk_ep_push(_lib.ptr(x), _lib.ptr(scale), _lib.ptr(st["idx"]), _lib.ptr(st["pos"]),
                                             _lib.ptr(st["send_base"]), _lib.ptr(st["offsets"]),
                                             _lib.ptr(st["tot_local"]), self.recv_ptrs, _lib.ptr(st["dst_row"]),
                                             self.rank, self.ep, self.E_local, SEG, self.R_max, st["K"], self.H,
                                             st["T"], _lib.stream_ptr()), "ep_push")
        self.barrier()
        if st.get("forward_only"):
            # forward-only passes read the receive buffer in place: a peer overwrites it with the next layer's rows
            # only after the group barrier of this layer's combine, which this rank reaches after its expert GEMMs
            return self.recv.t[:self.R_max * self.H].view(self.R_max, self.H)
        out = torch.empty(self.R_max, self.H, dtype=torch.bfloat16, device=self.device)
        self._copy_rows(self.recv.t, out, st)
        return out

    def _copy_rows(self, src, dst, st):
        """Copies the rows below the last padded offset (a device-side count: no host synchronisation)."""
        LAUNCHES["ep"] += 1
        _lib.check(_lib.kernels().gk_ep_copy_rows(_lib.ptr(src), _lib.ptr(dst), _lib.ptr(st["offsets"][self.E_local:]),
                                                  self.H, _lib.stream_ptr()), "ep_copy_rows")

    def pull(self, rows: torch.Tensor, weight: Optional[torch.Tensor], st, want_gathered: bool):
        """Publishes ``rows`` [R_max, H] (this rank's expert-side rows), waits for the peers and collects, for every
        local token, the weighted sum of its k rows."""
        self._copy_rows(rows.contiguous(), self.yout.t, st)
        self.barrier()
        T, K = st["T"], st["K"]
        y = torch.empty(T, self.H, dtype=torch.bfloat16, device=self.device)
        gathered = torch.empty(T * K, self.H, dtype=torch.bfloat16, device=self.device) if want_gathered else None
        LAUNCHES["ep"] += 1
        _lib.check(_lib.kernels().gk_ep_pull(self.yout_ptrs, _lib.ptr(st["dst_row"]), _lib.ptr(weight), _lib.ptr(y),
                                             _lib.ptr(gathered), self.ep, K, self.H, self.R_max, T,
                                             _lib.stream_ptr()), "ep_pull")
        return y, gathered


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, fe: FusedEP, st):
        ctx.fe, ctx.st = fe, st
        return fe.push(x, None, st)

    @staticmethod
    def backward(ctx, d_rows):
        dx, _ = ctx.fe.pull(d_rows.contiguous(), None, ctx.st, False)
        return dx, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_rows, w, fe: FusedEP, st):
        w32 = w.detach().float().contiguous()
        y, gathered = fe.pull(y_rows, w32.reshape(-1), st, w.requires_grad)
        ctx.fe, ctx.st, ctx.wdtype = fe, st, w.dtype
        ctx.save_for_backward(w32, gathered if gathered is not None else torch.empty(0))
        return y

    @staticmethod
    def backward(ctx, dy):
        w32, gathered = ctx.saved_tensors
        fe, st = ctx.fe, ctx.st
        dy = dy.contiguous()
        dw = None
        if ctx.needs_input_grad[1] and gathered.numel():
            T, K = st["T"], st["K"]
            dw = torch.bmm(gathered.view(T, K, fe.H), dy.view(T, fe.H, 1)).view(T, K).to(ctx.wdtype)
        d_rows = fe.push(dy, w32.reshape(-1), st)
        return d_rows, dw, None, None


_INSTANCES = {}


LOCAL_PLAN_MAX = 8192      # (token, k) pairs up to which the single-kernel local plan is used
_SMALL = {"tokens": 0}


@contextlib.contextmanager
def small_batch(tokens: int):
    """Inside this context expert-parallel layers with at most ``tokens`` tokens per rank use an instance whose peer
    buffers (and with them the row capacity the grouped expert GEMMs and the activation between them run over) are
    sized for ``tokens`` tokens in the worst case of every rank sending all its pairs to one rank, instead of for a
    training micro-batch.  The rollout engine's decode steps enter it with their static batch size, which is the
    same on every rank of the group; a decode step then moves a few thousand rows of capacity per layer, not a few
    hundred thousand."""
    prev = _SMALL["tokens"]
    _SMALL["tokens"] = int(tokens)
    try:
        yield
    finally:
        _SMALL["tokens"] = prev


def get_fused_ep(group, hidden: int, num_experts: int, top_k: int, tokens: int, x: torch.Tensor) -> Optional[FusedEP]:
    """The per-group instance, created on first use (a collective over the group).  The choice between this path and
    the NCCL one depends only on values that are equal on every rank."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and _lib.use_native(x)):
        return None
    if os.environ.get("GCORE_FUSED_EP", "1") == "0" or dist.get_world_size(group) > 8 or hidden % 8:
        return None
    if not hasattr(_lib.kernels(), "gk_ep_plan"):
        return None
    small = _SMALL["tokens"] if 0 < tokens <= _SMALL["tokens"] else 0
    key = (id(group), hidden, num_experts, top_k, small)
    if key not in _INSTANCES:
        if small:
            _INSTANCES[key] = FusedEP(group, hidden, num_experts, top_k, small, device=x.device,
                                      capacity_factor=float(dist.get_world_size(group)))
        else:
            max_tokens = int(os.environ.get("GCORE_EP_MAX_TOKENS", "0")) or max(16384, 2 * tokens)
            _INSTANCES[key] = FusedEP(group, hidden, num_experts, top_k, max_tokens, device=x.device)
    return _INSTANCES[key]


def fused_ep_moe_forward(fe: FusedEP, layer, x, idx, w):
    st = fe.plan(idx)
    # read here: an autograd function always runs its forward with grad mode off
    st["forward_only"] = not torch.is_grad_enabled() and os.environ.get("GCORE_EP_RECV_INPLACE", "1") != "0"
    rows = _Dispatch.apply(x, fe, st)
    y_rows = layer.experts(rows, st["offsets"])
    return _Combine.apply(y_rows, w, fe, st)
