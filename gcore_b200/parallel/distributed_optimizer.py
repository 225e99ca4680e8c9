"""Contiguous parameter / main-gradient buffers with bucketed gradient reduction, and the ZeRO-1 distributed
optimizer on top of them (sharded fp32 master weights + Adam moments, bf16 parameter all-gather).

Behavioural contract = Megatron-Core's ``DistributedDataParallel`` + ``DistributedOptimizer`` as configured by the
reference (gpatch_v4/training_backend/megatron_backend/mixin.py:311-348, optimizer.py:53-169): fp32 gradient
accumulation and reduction, bucket size ``max(40e6, 1e6 * dp_size)`` elements, reduce-scatter when the optimizer is
distributed (all-reduce otherwise), gradient averaging over DP x CP, global-norm clipping across model-parallel
ranks with replicated parameters counted once, linear / cosine / WSD learning-rate schedules with warm-up.

Dense parameters reduce over the DP x CP group; expert parameters over the expert-data-parallel group.
The update itself is one fused kernel per shard (``ops.optim.adam_step``): unscale + clip + AdamW + bf16 write.

On GPUs of one NVLink domain the buffers live in symmetric memory and the collective halves of the step move into
the optimizer kernel (``ops/csrc/zero1.cu``): the shard owner pulls its gradient shard from every peer, applies
AdamW and pushes the bf16 parameters into every peer's buffer; NCCL moves no gradient or parameter bytes
(``GCORE_FUSED_DP=0`` restores the reduce-scatter / all-gather path).
"""
from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..core import parallel_state as ps
from ..ops import _lib
from ..ops import optim as optim_ops


LAUNCHES = {"zero1": 0}


def _peer_memory_ok(group, dev, dt, grad_dtype) -> bool:
    if dev.type != "cuda" or not dist.is_initialized() or os.environ.get("GCORE_FUSED_DP", "1") == "0":
        return False
    n = _group_size(group)
    if n < 2 or n > 8 or dt != torch.bfloat16 or grad_dtype != torch.float32 or not _lib.use_native():
        return False
    return hasattr(_lib.kernels(), "gk_zero1_step")


def _group_size(g):
    return dist.get_world_size(g) if (g is not None and dist.is_initialized()) else 1


def _group_rank(g):
    return dist.get_rank(g) if (g is not None and dist.is_initialized()) else 0


@dataclass
class Bucket:
    start: int
    end: int
    params: List[torch.nn.Parameter]
    pending: int = 0
    handle: Optional[object] = None


class ParamAndGradBuffer:
    """All parameters of one reduction domain in one flat bf16 buffer and their main grads in one flat fp32 buffer."""

    def __init__(self, params: List[torch.nn.Parameter], names: List[str], group, grad_dtype=torch.float32,
                 bucket_size: Optional[int] = None, use_distributed_optimizer: bool = True, alloc_grads: bool = True):
        self.group = group
        self.dp = _group_size(group)
        self.dp_rank = _group_rank(group)
        self.params, self.names = params, names
        self.use_distributed_optimizer = use_distributed_optimizer
        self.grad_dtype = grad_dtype
        dev = params[0].device
        dt = params[0].dtype
        if bucket_size is None:
            bucket_size = max(40_000_000, 1_000_000 * self.dp)
        align = 128 * self.dp
        # layout: parameters in reverse registration order so buckets fill in roughly backward order
        self.offsets: Dict[int, int] = {}
        self.buckets: List[Bucket] = []
        off, bstart, bparams = 0, 0, []
        for p in reversed(params):
            self.offsets[id(p)] = off
            off += p.numel()
            bparams.append(p)
            if off - bstart >= bucket_size:
                off = (off + align - 1) // align * align
                self.buckets.append(Bucket(bstart, off, bparams))
                bstart, bparams = off, []
        if bparams:
            off = (off + align - 1) // align * align
            self.buckets.append(Bucket(bstart, off, bparams))
        self.numel = off
        # Peer-memory mode: parameter and gradient buffers live in symmetric memory so that the optimizer kernel of
        # every rank can pull gradient shards from, and push parameter shards to, its data-parallel peers.
        self.peer = (use_distributed_optimizer and _peer_memory_ok(group, dev, dt, grad_dtype))
        self.param_sym = self.grad_sym = self.flag_sym = None
        if self.peer:
            from .symm import SymmBuffer
            self.param_sym = SymmBuffer(self.numel, dt, group, dev)
            self.param_data = self.param_sym.t.zero_()
            self.flag_sym = SymmBuffer(64 * 8, torch.int32, group, dev)
            self.flag_sym.t.zero_()
            self.flag_ptrs = torch.tensor(self.flag_sym.ptrs, dtype=torch.int64, device=dev)
            self.barrier_epoch = 0
            self.pending_scale = None
        else:
            self.param_data = torch.zeros(self.numel, dtype=dt, device=dev)
        self.grad_data = None
        self.param_to_bucket: Dict[int, Bucket] = {}
        for b in self.buckets:
            for p in b.params:
                self.param_to_bucket[id(p)] = b
        with torch.no_grad():
            for p in params:
                o = self.offsets[id(p)]
                view = self.param_data[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
        if alloc_grads:
            self.allocate_grads()

    # ---- gradient storage can be released between training phases (colocated rollout needs the memory)
    def allocate_grads(self):
        if self.grad_data is None:
            if self.peer:
                if self.grad_sym is None:
                    from .symm import SymmBuffer
                    self.grad_sym = SymmBuffer(self.numel, self.grad_dtype, self.group, self.param_data.device)
                    self.ptrs = (ctypes.c_ulonglong * (2 * self.dp))(*(self.grad_sym.ptrs + self.param_sym.ptrs))
                self.grad_data = self.grad_sym.t.zero_()
            else:
                self.grad_data = torch.zeros(self.numel, dtype=self.grad_dtype, device=self.param_data.device)
        for p in self.params:
            o = self.offsets[id(p)]
            p.main_grad = self.grad_data[o:o + p.numel()].view(p.shape) if p.requires_grad else None

    def release_grads(self):
        if self.peer:
            return  # symmetric buffers are rendezvoused once and stay mapped on the peers
        self.grad_data = None
        for p in self.params:
            p.main_grad = None

    # ---- peer-memory optimizer path (ops/csrc/zero1.cu)
    def peer_barrier(self):
        """Device-side barrier over the reduction group on the current stream (bounded wait, error word on expiry)."""
        self.barrier_epoch += 1
        _lib.check(_lib.kernels().gk_peer_barrier(_lib.ptr(self.flag_ptrs), self.dp_rank, self.dp, 0,
                                                  self.barrier_epoch, _lib.ptr(_lib.err_flag(self.param_data.device)),
                                                  _lib.stream_ptr()), "peer_barrier")
        LAUNCHES["zero1"] += 1

    def zero1(self, mode: int, sh: dict, scale: float, clip, sumsq, lr=0.0, cfg=None, step=1, wd=0.0):
        s, e = sh["s"], sh["e"]
        _lib.check(_lib.kernels().gk_zero1_step(
            mode, self.ptrs, self.dp_rank, self.dp, s, e - s, _lib.ptr(self.grad_data[s:e]), _lib.ptr(sh["master"]),
            _lib.ptr(sh["m"]), _lib.ptr(sh["v"]), float(scale), _lib.ptr(clip), _lib.ptr(sumsq), float(lr),
            float(cfg.adam_beta1 if cfg else 0.9), float(cfg.adam_beta2 if cfg else 0.999),
            float(cfg.adam_eps if cfg else 1e-8), float(wd), int(step), 0, _lib.stream_ptr()), "zero1_step")
        LAUNCHES["zero1"] += 1

    def zero_grad(self):
        if self.grad_data is not None:
            self.grad_data.zero_()
        for p in self.params:
            p.grad = None

    def shard_range(self, bucket: Bucket):
        n = (bucket.end - bucket.start) // self.dp
        s = bucket.start + self.dp_rank * n
        return s, s + n

    def reduce_bucket(self, bucket: Bucket, scale: float, async_op: bool = False):
        g = self.grad_data[bucket.start:bucket.end]
        if scale != 1.0:
            g.mul_(scale)
        if self.dp == 1:
            return None
        if self.use_distributed_optimizer:
            s, e = self.shard_range(bucket)
            return dist.reduce_scatter_tensor(self.grad_data[s:e], g, group=self.group, async_op=async_op)
        return dist.all_reduce(g, group=self.group, async_op=async_op)

    def gather_params(self, bucket: Bucket, async_op: bool = False):
        if self.dp == 1 or not self.use_distributed_optimizer:
            return None
        s, e = self.shard_range(bucket)
        return dist.all_gather_into_tensor(self.param_data[bucket.start:bucket.end], self.param_data[s:e],
                                           group=self.group, async_op=async_op)


class DistributedDataParallel:
    """Owns the buffers of a model, routes autograd gradients into ``main_grad`` and runs the bucketed reduction."""

    def __init__(self, model: torch.nn.Module, grad_reduce_in_fp32: bool = True, bucket_size: Optional[int] = None,
                 use_distributed_optimizer: bool = True, overlap_grad_reduce: bool = False,
                 average_in_collective: bool = True, alloc_grads: bool = True):
        self.model = model
        self.overlap = overlap_grad_reduce
        dense_p, dense_n, exp_p, exp_n = [], [], [], []
        for n, p in model.named_parameters():
            if not p.requires_grad:
                continue  # frozen weights (LoRA base, frozen towers) keep their own storage and get no grad / state
            if getattr(p, "is_expert", False):
                exp_p.append(p), exp_n.append(n)
            else:
                dense_p.append(p), dense_n.append(n)
        gdt = torch.float32 if grad_reduce_in_fp32 else None
        self.buffers: List[ParamAndGradBuffer] = []
        by_dtype: Dict = {}
        for plist, nlist, group in ((dense_p, dense_n, ps.get_data_parallel_group(with_context_parallel=True)),
                                    (exp_p, exp_n, ps.get_expert_data_parallel_group())):
            # one buffer per (domain, dtype): fp32 router weights do not share storage with bf16 weights
            split: Dict = {}
            for p, n in zip(plist, nlist):
                key = (p.dtype, p.dim() >= 2)  # biases and norm gains take no weight decay
                split.setdefault(key, ([], []))
                split[key][0].append(p)
                split[key][1].append(n)
            for (dt, decays), (pl, nl) in split.items():
                buf = ParamAndGradBuffer(pl, nl, group, gdt or dt, bucket_size, use_distributed_optimizer,
                                         alloc_grads)
                buf.weight_decay_mult = 1.0 if decays else 0.0
                self.buffers.append(buf)
        self._hooks = []
        for buf in self.buffers:
            for p in buf.params:
                if p.requires_grad:
                    self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(buf, p)))
        self.grad_scale_extra = 1.0

    def _make_hook(self, buf: ParamAndGradBuffer, p):
        def hook(param):
            if param.grad is not None and param.main_grad is not None:
                param.main_grad.add_(param.grad.to(param.main_grad.dtype))
            param.grad = None
        return hook

    def zero_grad_buffer(self):
        for b in self.buffers:
            b.zero_grad()

    def allocate_grads(self):
        for b in self.buffers:
            b.allocate_grads()

    def release_grads(self):
        for b in self.buffers:
            b.release_grads()

    def finish_grad_sync(self, extra_scale: float = 1.0):
        """Reduces every bucket: the sum over the buffer's reduction group times ``extra_scale`` / (dense data-parallel
        size), i.e. the average over the data-parallel replicas for ``extra_scale = 1`` and the plain sum for
        ``extra_scale = dense DP size`` (losses already normalised by global counts).  The divisor is the *dense* group
        size for every buffer: an expert buffer reduces over its own group (whose size differs: expert parallelism
        removes ranks from it, tensor-parallel ranks holding whole experts join it), but every token still
        contributes exactly once to an expert's gradient, so the normalisation is that of the batch, not of the group.
        (Dividing by the expert group's own size scaled expert gradients by the expert-parallel size.)"""
        dense_dp = ps.get_data_parallel_world_size(with_context_parallel=True)
        tp_group = ps.get_tensor_model_parallel_group()
        if ps.get_tensor_model_parallel_world_size() > 1:
            # gains / router weights that act on sequence-parallel activations see only this rank's tokens; replicated
            # adapter halves on sharded projections see only this rank's shard of the other half
            sp = getattr(self.model, "sequence_parallel", False)
            sp_grads = [p.main_grad for buf in self.buffers for p in buf.params if p.main_grad is not None
                        and ((sp and getattr(p, "sequence_parallel", False)) or getattr(p, "tp_partial_grad", False))]
            if sp_grads:
                flat = torch.cat([g.reshape(-1) for g in sp_grads])
                dist.all_reduce(flat, group=tp_group)
                o = 0
                for g in sp_grads:
                    g.copy_(flat[o:o + g.numel()].view_as(g))
                    o += g.numel()
        handles = []
        for buf in self.buffers:
            scale = extra_scale / max(dense_dp, 1)
            if buf.peer:
                # reduce-scatter happens inside the optimizer kernels (peer pulls); only order the ranks here
                buf.pending_scale = scale
                buf.peer_barrier()
                continue
            for bucket in buf.buckets:
                h = buf.reduce_bucket(bucket, scale, async_op=True)
                if h is not None:
                    handles.append(h)
        for h in handles:
            h.wait()

    def parameters(self):
        return self.model.parameters()

    def __call__(self, *a, **kw):
        return self.model(*a, **kw)


def lr_at_step(cfg, step: int, total_steps: Optional[int]) -> float:
    """``OptimizerParamScheduler`` semantics: linear warm-up from ``lr_warmup_init`` then constant / linear / cosine /
    inverse-square-root / WSD decay to ``min_lr`` over ``lr_decay_steps``."""
    warm = cfg.lr_warmup_steps
    if cfg.lr_warmup_step_frac and total_steps:
        warm = int(cfg.lr_warmup_step_frac * total_steps)
    if warm > 0 and step <= warm:
        return cfg.lr_warmup_init + (cfg.lr - cfg.lr_warmup_init) * step / warm
    decay_steps = cfg.lr_decay_steps or total_steps
    if cfg.lr_decay_style == "constant" or not decay_steps:
        return cfg.lr
    if step > decay_steps:
        return cfg.min_lr
    if cfg.lr_decay_style == "inverse-square-root":
        return max(cfg.min_lr, cfg.lr * math.sqrt(max(warm, 1)) / math.sqrt(max(step, 1)))
    frac = (step - warm) / max(decay_steps - warm, 1)
    frac = min(max(frac, 0.0), 1.0)
    if cfg.lr_decay_style == "linear":
        coeff = 1.0 - frac
    elif cfg.lr_decay_style == "cosine":
        coeff = 0.5 * (math.cos(math.pi * frac) + 1.0)
    elif cfg.lr_decay_style == "WSD":
        wsd = cfg.lr_wsd_decay_steps or 0
        anneal_start = decay_steps - wsd
        if step <= anneal_start:
            coeff = 1.0
        else:
            f = (step - anneal_start) / max(wsd, 1)
            coeff = {"linear": 1 - f, "cosine": 0.5 * (math.cos(math.pi * f) + 1), "exponential": 2 ** (-f * 10)
                     if False else (0.5 ** (f * 10))}.get(cfg.lr_wsd_decay_style, 1 - f)
    else:
        coeff = 1.0
    return cfg.min_lr + coeff * (cfg.lr - cfg.min_lr)


class DistributedOptimizer:
    """AdamW with state sharded over the buffer's reduction group (ZeRO-1)."""

    def __init__(self, ddp: DistributedDataParallel, cfg, total_steps: Optional[int] = None):
        self.ddp, self.cfg, self.total_steps = ddp, cfg, total_steps
        self.step_count = 0
        self.shards = []  # per (buffer, bucket): dict(master, m, v, range)
        for buf in ddp.buffers:
            for bucket in buf.buckets:
                s, e = buf.shard_range(bucket) if buf.use_distributed_optimizer else (bucket.start, bucket.end)
                master = buf.param_data[s:e].float()
                self.shards.append(dict(buf=buf, bucket=bucket, s=s, e=e, master=master,
                                        m=torch.zeros_like(master), v=torch.zeros_like(master)))
        self._wd_mask_cache = None
        self.last_grad_norm = None
        self.offloaded = False

    # ------------------------------------------------------------------ grad norm / clip
    def _local_sumsq(self, skip_peer: bool = False) -> torch.Tensor:
        """Sum of squares of this rank's gradient shards, with parameters replicated across TP counted on TP rank 0
        only (their shard values are identical on every TP rank)."""
        dev = self.shards[0]["master"].device
        total = torch.zeros(1, dtype=torch.float32, device=dev)
        tp_rank = ps.get_tensor_model_parallel_rank()
        for sh in self.shards:
            buf, s, e = sh["buf"], sh["s"], sh["e"]
            if skip_peer and buf.peer:
                continue
            if not buf.use_distributed_optimizer and buf.dp > 1 and buf.dp_rank != 0:
                continue  # every rank of the reduction group holds the whole bucket: count it once
            g = buf.grad_data[s:e]
            if tp_rank == 0 or ps.get_tensor_model_parallel_world_size() == 1:
                optim_ops.sumsq(g, total)
            else:
                # subtract nothing here; replicated params are masked below
                for p in sh["bucket"].params:
                    if getattr(p, "tp_mode", "none") in ("column", "row", "expert"):
                        o = buf.offsets[id(p)]
                        lo, hi = max(o, s), min(o + p.numel(), e)
                        if hi > lo:
                            optim_ops.sumsq(buf.grad_data[lo:hi], total)
        return total

    def grad_norm(self, skip_peer: bool = False, extra=None) -> torch.Tensor:
        total = self._local_sumsq(skip_peer)
        if extra is not None:
            total += extra
        if dist.is_initialized() and ps.get_world_size() > 1:
            # shards partition the DP x CP group, model-parallel ranks hold different parameters: sum over everyone
            # (of this role: with disaggregated placement the rollout ranks are not part of it)
            dist.all_reduce(total, group=ps.get_world_group())
        return total.sqrt()

    # ------------------------------------------------------------------ step
    def step(self, lr: Optional[float] = None):
        cfg = self.cfg
        self.step_count += 1
        if lr is None:
            lr = lr_at_step(cfg, self.step_count, self.total_steps)
        clipping = bool(cfg.max_grad_norm and cfg.max_grad_norm > 0)
        peer_shards = [sh for sh in self.shards if sh["buf"].peer and sh["buf"].pending_scale is not None]
        fused_sumsq = None
        if peer_shards:
            if clipping:
                # without tensor parallelism no parameter is replicated, so the kernel's own sum of squares is exact
                if ps.get_tensor_model_parallel_world_size() == 1:
                    fused_sumsq = torch.zeros(1, dtype=torch.float32, device=peer_shards[0]["master"].device)
                for sh in peer_shards:  # pull + sum + scale -> own fp32 shard
                    sh["buf"].zero1(1, sh, sh["buf"].pending_scale, None, fused_sumsq)
            else:
                fused_sumsq = torch.zeros(1, dtype=torch.float32, device=peer_shards[0]["master"].device)
                for sh in peer_shards:  # pull + Adam + push in one pass
                    buf = sh["buf"]
                    buf.zero1(3, sh, buf.pending_scale, None, fused_sumsq, lr, cfg, self.step_count,
                              cfg.weight_decay * getattr(buf, "weight_decay_mult", 1.0))
        if fused_sumsq is None:
            norm = self.grad_norm()
        else:
            norm = self.grad_norm(skip_peer=True, extra=fused_sumsq)
        self.last_grad_norm = norm
        clip = None
        if clipping:
            clip = torch.clamp(cfg.max_grad_norm / (norm + 1e-6), max=1.0)
        for sh in self.shards:
            buf, s, e = sh["buf"], sh["s"], sh["e"]
            if buf.peer and buf.pending_scale is not None:
                if clipping:  # Adam on the reduced shard + push of the bf16 parameters to every rank
                    buf.zero1(2, sh, 1.0, clip, None, lr, cfg, self.step_count,
                              cfg.weight_decay * getattr(buf, "weight_decay_mult", 1.0))
                continue
            optim_ops.adam_step(sh["master"], sh["m"], sh["v"], buf.grad_data[s:e], buf.param_data[s:e], lr=lr,
                                beta1=cfg.adam_beta1, beta2=cfg.adam_beta2, eps=cfg.adam_eps,
                                weight_decay=cfg.weight_decay * getattr(buf, "weight_decay_mult", 1.0),
                                step=self.step_count, grad_scale=clip)
        handles = []
        for sh in self.shards:
            if sh["buf"].peer and sh["buf"].pending_scale is not None:
                continue
            h = sh["buf"].gather_params(sh["bucket"], async_op=True)
            if h is not None:
                handles.append(h)
        for h in handles:
            h.wait()
        for buf in self.ddp.buffers:
            if buf.peer and buf.pending_scale is not None:
                buf.pending_scale = None
                buf.peer_barrier()  # every peer's parameter pushes have landed; gradients may be overwritten
        return float(lr)

    def reload_master_from_params(self):
        for sh in self.shards:
            sh["master"].copy_(sh["buf"].param_data[sh["s"]:sh["e"]].float())

    # ------------------------------------------------------------------ host offload (time-sharing with rollout)
    def offload(self):
        """Moves master weights and moments to pinned host memory (CPU swap of the reference:
        gpatch_v4/training_backend/megatron_backend/mcore_swap_impl.py:24-207)."""
        if self.offloaded:
            return
        for sh in self.shards:
            for k in ("master", "m", "v"):
                t = sh[k]
                host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=t.is_cuda)
                host.copy_(t, non_blocking=True)
                sh[k + "_dev"] = t.device
                sh[k] = host
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
        self.offloaded = True

    def onload(self):
        if not self.offloaded:
            return
        for sh in self.shards:
            for k in ("master", "m", "v"):
                sh[k] = sh[k].to(sh.pop(k + "_dev"), non_blocking=True)
        self.offloaded = False

    # ------------------------------------------------------------------ state
    def state_dict(self):
        return {"step": self.step_count,
                "shards": [dict(s=sh["s"], e=sh["e"], master=sh["master"], m=sh["m"], v=sh["v"]) for sh in self.shards]}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        for sh, src in zip(self.shards, sd["shards"]):
            for k in ("master", "m", "v"):
                sh[k].copy_(src[k])
