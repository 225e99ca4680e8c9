"""Symmetric-memory runtime for the fused compute + collective kernels.

Every rank of a tensor-parallel group allocates the same communication buffers with
``torch.distributed._symmetric_memory`` (CUDA VMM allocations whose handles are exchanged once at rendezvous), which
gives each rank device pointers to every peer's copy.  The kernels in ``ops/csrc/gemm_comm.cu`` then move data with
peer stores / TMA loads and order it with epoch flags that live in the same symmetric space.

``FusedTP`` exposes the two tensor-parallel primitives as autograd functions with the NCCL twins' contract
(``parallel/tp_ops.py``):  ``ag_linear``  = all-gather(x over tokens) -> x W^T (+ bias)   and
``linear_rs`` = x W^T -> reduce-scatter over tokens.  Their backward passes are each other's fused kernel
(dgrad of a column-parallel layer is a GEMM -> reduce-scatter, dgrad of a row-parallel one an all-gather -> GEMM);
the weight gradients reuse the gathered operand that the forward / backward already materialised.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import linear_wgrad

LAUNCHES = {"fused_comm": 0}
_MAX_FLAGS = 1 << 16


class SymmBuffer:
    def __init__(self, numel: int, dtype, group, device):
        import torch.distributed._symmetric_memory as symm_mem
        self.t = symm_mem.empty(numel, dtype=dtype, device=device)
        self.hdl = symm_mem.rendezvous(self.t, group=group)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.rank = self.hdl.rank
        self.world = self.hdl.world_size


class FusedTP:
    """Per-TP-group communication state: two gathered buffers and two inboxes (call parity) plus flag arrays."""

    def __init__(self, group, max_rows_per_rank: int, max_width: int, device=None, ncomm: int = 16):
        self.group = group
        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.max_rows = max_rows_per_rank
        self.max_width = max_width
        self.ncomm = ncomm
        n = self.tp * max_rows_per_rank * max_width
        self.ag = [SymmBuffer(n, torch.bfloat16, group, self.device) for _ in range(2)]
        self.rs = [SymmBuffer(n, torch.bfloat16, group, self.device) for _ in range(2)]
        self.ag_flags = [SymmBuffer(_MAX_FLAGS, torch.int32, group, self.device) for _ in range(2)]
        self.rs_flags = [SymmBuffer(_MAX_FLAGS, torch.int32, group, self.device) for _ in range(2)]
        for f in self.ag_flags + self.rs_flags:
            f.t.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group)
        self.ag_calls = 0
        self.rs_calls = 0

    # ------------------------------------------------------------------ raw launches
    def _ptr_array(self, buf: SymmBuffer, flags: SymmBuffer):
        arr = (ctypes.c_ulonglong * (2 * self.tp))(*(buf.ptrs + flags.ptrs))
        return arr

    def gathered_view(self, rows_per_rank: int, width: int, parity: int) -> torch.Tensor:
        """The local gathered buffer viewed as [tp * rows_per_rank, width]; a producer may write this rank's rows
        (``[rank * rows_per_rank, (rank + 1) * rows_per_rank)``) directly into it."""
        return self.ag[parity].t[:self.tp * rows_per_rank * width].view(self.tp * rows_per_rank, width)

    def ag_gemm(self, x_local: torch.Tensor, w: torch.Tensor, bias=None, b_mn: bool = False):
        """Returns ``(y [tp*Tl, N], x_gathered [tp*Tl, K])``; ``x_gathered`` stays valid until the call after next."""
        Tl, K = x_local.shape
        assert Tl % 128 == 0 and Tl <= self.max_rows and K <= self.max_width, (Tl, K)
        N = w.shape[1] if b_mn else w.shape[0]
        parity = self.ag_calls & 1
        self.ag_calls += 1
        epoch = (self.ag_calls + 1) // 2  # grows once per use of each parity
        chunks = Tl // 128
        assert self.tp * chunks <= _MAX_FLAGS
        gathered = self.gathered_view(Tl, K, parity)
        mine = gathered[self.rank * Tl:(self.rank + 1) * Tl]
        if x_local.data_ptr() != mine.data_ptr():
            mine.copy_(x_local)
        y = torch.empty(self.tp * Tl, N, dtype=torch.bfloat16, device=x_local.device)
        LAUNCHES["fused_comm"] += 1
        rc = _lib.kernels().gk_gemm_comm(
            1, _lib.ptr(gathered), K, _lib.ptr(w), w.stride(0), w.shape[0], int(b_mn), _lib.ptr(y), N,
            _lib.ptr(bias), self.tp * Tl, N, K, self.rank, self.tp, Tl, self.ncomm, epoch,
            self._ptr_array(self.ag[parity], self.ag_flags[parity]), K, _lib.ptr(_lib.err_flag(x_local.device)),
            _lib.stream_ptr())
        _lib.check(rc, "gk_gemm_comm[AG]")
        return y, gathered

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, b_mn: bool = False) -> torch.Tensor:
        """``a`` [tp*Tl, K_local] (all tokens, this rank's slice of the contraction) -> ``y_local`` [Tl, N]."""
        T, K = a.shape
        assert T % (128 * self.tp) == 0, T
        Tl = T // self.tp
        N = w.shape[1] if b_mn else w.shape[0]
        assert Tl <= self.max_rows and N <= self.max_width, (Tl, N)
        parity = self.rs_calls & 1
        self.rs_calls += 1
        epoch = (self.rs_calls + 1) // 2
        assert self.tp * (Tl // 128) * ((N + 127) // 128) <= _MAX_FLAGS
        y = torch.empty(Tl, N, dtype=torch.bfloat16, device=a.device)
        LAUNCHES["fused_comm"] += 1
        rc = _lib.kernels().gk_gemm_comm(
            2, _lib.ptr(a), a.stride(0), _lib.ptr(w), w.stride(0), w.shape[0], int(b_mn), _lib.ptr(y), N, None,
            T, N, K, self.rank, self.tp, Tl, 0, epoch, self._ptr_array(self.rs[parity], self.rs_flags[parity]), N,
            _lib.ptr(_lib.err_flag(a.device)), _lib.stream_ptr())
        _lib.check(rc, "gk_gemm_comm[RS]")
        return y

    # ------------------------------------------------------------------ autograd
    def ag_linear(self, x_local, w, bias=None, main_grad=None):
        return _AGLinear.apply(x_local, w, bias, self, main_grad)

    def linear_rs(self, a, w, main_grad=None):
        return _LinearRS.apply(a, w, self, main_grad)


class _AGLinear(torch.autograd.Function):
    """Column-parallel linear with sequence parallelism: y = gather(x) W^T + b."""

    @staticmethod
    def forward(ctx, x_local, w, bias, ftp: FusedTP, main_grad):
        y, gathered = ftp.ag_gemm(x_local.contiguous(), w, bias)
        # the gathered activation is needed for wgrad; it lives in a double-buffered comm buffer, so keep a copy only
        # if the backward may run after two more fused calls (always the case in a transformer stack)
        ctx.save_for_backward(x_local, w)
        ctx.ftp, ctx.main_grad, ctx.has_bias = ftp, main_grad, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x_local, w = ctx.saved_tensors
        ftp = ctx.ftp
        dy = dy.contiguous()
        # dgrad: dx_local = reduce_scatter(dy W)  -> fused GEMM -> RS with the weight read MN-major
        dx = ftp.gemm_rs(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = db = None
        if ctx.needs_input_grad[1]:
            # wgrad needs gather(x): re-gather through the comm buffer (identity-weight trick is avoided: plain push)
            xg = _regather(ftp, x_local)
            if ctx.main_grad is not None:
                linear_wgrad(dy, xg, out=ctx.main_grad, accumulate=True)
            else:
                dw = linear_wgrad(dy, xg).to(w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(0).to(dy.dtype)
        return dx, dw, db, None, None


class _LinearRS(torch.autograd.Function):
    """Row-parallel linear with sequence parallelism: y_local = reduce_scatter(a W^T)."""

    @staticmethod
    def forward(ctx, a, w, ftp: FusedTP, main_grad):
        ctx.save_for_backward(a, w)
        ctx.ftp, ctx.main_grad = ftp, main_grad
        return ftp.gemm_rs(a.contiguous(), w)

    @staticmethod
    def backward(ctx, dy_local):
        a, w = ctx.saved_tensors
        ftp = ctx.ftp
        # dgrad: da = gather(dy) W -> fused AG -> GEMM with the weight read MN-major; its gathered dy feeds wgrad
        da, dyg = ftp.ag_gemm(dy_local.contiguous(), w, None, b_mn=True)
        dw = None
        if ctx.needs_input_grad[1]:
            if ctx.main_grad is not None:
                linear_wgrad(dyg, a, out=ctx.main_grad, accumulate=True)
            else:
                dw = linear_wgrad(dyg, a).to(w.dtype)
        return (da if ctx.needs_input_grad[0] else None), dw, None, None


def _regather(ftp: FusedTP, x_local: torch.Tensor) -> torch.Tensor:
    out = torch.empty(ftp.tp * x_local.shape[0], x_local.shape[1], dtype=x_local.dtype, device=x_local.device)
    dist.all_gather_into_tensor(out, x_local.contiguous(), group=ftp.group)
    return out


class PeerAllReduce:
    """One-shot all-reduce over peer memory for small bf16 tensors (``ops/csrc/comm.cu``); in place, usable inside a
    CUDA graph (the call epoch is kept on the device)."""

    def __init__(self, group, max_elems: int, device=None):
        self.group = group
        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.slot = (max_elems + 7) // 8 * 8
        lib = _lib.kernels()
        lib.gk_allreduce_ctas.restype = ctypes.c_int
        self.ctas = lib.gk_allreduce_ctas()
        self.inbox = SymmBuffer(2 * self.tp * self.slot, torch.bfloat16, group, self.device)
        self.flags = SymmBuffer(2 * self.tp * self.ctas, torch.int32, group, self.device)
        self.flags.t.zero_()
        self.state = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.ptrs = (ctypes.c_ulonglong * (2 * self.tp))(*(self.inbox.ptrs + self.flags.ptrs))
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        n = x.numel()
        if n > self.slot or n % 8 or x.dtype != torch.bfloat16 or not x.is_contiguous():
            dist.all_reduce(x, group=self.group)
            return x
        LAUNCHES["fused_comm"] += 1
        rc = _lib.kernels().gk_allreduce_oneshot(_lib.ptr(x), _lib.ptr(x), n, self.rank, self.tp, self.slot, self.ptrs,
                                                 _lib.ptr(self.state), _lib.ptr(_lib.err_flag(x.device)),
                                                 _lib.stream_ptr())
        _lib.check(rc, "gk_allreduce_oneshot")
        return x


    def all_reduce_rmsnorm(self, partial: torch.Tensor, residual, gamma: torch.Tensor, eps: float):
        """``(y, new_residual)`` with ``new_residual = all_reduce(partial) + residual`` and ``y = RMSNorm(new_residual)
        * gamma``, one kernel; ``None`` when the shape is outside the kernel's limits (the caller then runs the two
        steps separately)."""
        rows, H = partial.shape
        if (rows * H > self.slot or H % 8 or partial.dtype != torch.bfloat16 or not partial.is_contiguous()
                or gamma.dtype != torch.bfloat16 or (residual is not None and not residual.is_contiguous())
                or not hasattr(_lib.kernels(), "gk_allreduce_rmsnorm")):
            return None
        y = torch.empty_like(partial)
        res_out = torch.empty_like(partial)
        LAUNCHES["fused_comm"] += 1
        rc = _lib.kernels().gk_allreduce_rmsnorm(_lib.ptr(partial), _lib.ptr(residual), _lib.ptr(gamma), _lib.ptr(res_out),
                                                 _lib.ptr(y), rows, H, float(eps), self.rank, self.tp, self.slot,
                                                 self.ptrs, _lib.ptr(self.state), _lib.ptr(_lib.err_flag(partial.device)),
                                                 _lib.stream_ptr())
        _lib.check(rc, "gk_allreduce_rmsnorm")
        return y, res_out


_FUSED: dict = {}


def get_fused_tp(group, max_rows_per_rank: int, max_width: int) -> Optional[FusedTP]:
    """One ``FusedTP`` per (group, capacity); ``None`` when the group is trivial or symmetric memory is unavailable."""
    if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return None
    key = (id(group), max_rows_per_rank, max_width)
    if key not in _FUSED:
        _FUSED[key] = FusedTP(group, max_rows_per_rank, max_width)
    return _FUSED[key]
