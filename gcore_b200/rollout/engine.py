"""Continuous-batching rollout decoder with a paged KV cache.

Replaces the vLLM / SGLang engines the reference wraps (``InferEngine``, gpatch_v4/generation_backend/
infer_engine.py:158-768) and keeps its verbs: ``generate``, ``abort_all_requests``, ``flush_cache``, ``sleep`` /
``wake_up`` (``weights`` / ``kv_cache`` tags), ``update_weights``, ``get_load``.

B200-first choices:
  * The engine lives in the trainer's process and, when the tensor-parallel layouts match, reads the trainer's bf16
    parameter buffer directly: a weight "resync" is a pointer hand-over, not a copy.  Other layouts go through
    ``rollout/weight_sync.py``.
  * A decode step is one CUDA graph: embedding, per layer (RMSNorm, swap-AB split-K tcgen05 GEMMs, RoPE-fused cache
    append, split-KV paged attention, SwiGLU), vocabulary GEMM, Gumbel-max sampling, and the state advance
    (positions, context lengths, slot computation, output ring write), so the host only replays it.
  * The host synchronises every ``sync_interval`` steps: it then reads the tokens produced, retires finished
    requests, admits waiting ones (prefill) and tops up block tables for the next interval.  Requests that hit EOS
    inside an interval produce a few discarded tokens instead of forcing a sync per token.
  * ``n`` samples per prompt share the prompt's KV blocks (copy-on-write of the last partial block).
  * Tensor-parallel ranks run the same host logic on the same inputs (SPMD) and agree on sampled tokens because the
    sampler's random stream depends only on (seed, step, token id).
"""
from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..core import parallel_state as ps
from ..models.config import ModelConfig
from ..ops import _lib, fused
from ..ops.attention import flash_attn_varlen, kv_append_rope, mla_paged_decode, paged_decode_append
from ..ops.gemm import linear_forward
from ..ops.vocab import apply_top_k_top_p, sample, sample_filtered
from ..utils import io_counters


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    min_p: float = 0.0
    max_new_tokens: int = 128
    seed: int = 42
    stop_token_ids: Sequence[int] = ()
    greedy: bool = False
    # logits of tokens already in the prompt or the output are divided (positive) / multiplied (negative) by this
    repetition_penalty: float = 1.0


@dataclass
class Request:
    rid: int
    prompt: List[int]
    params: SamplingParams
    seed: int
    out_tokens: List[int] = field(default_factory=list)
    out_logprobs: List[float] = field(default_factory=list)
    finished: bool = False
    finish_reason: str = ""
    parent: Optional[int] = None
    slot: int = -1
    routed_experts: Optional[list] = None
    prompt_index: int = 0


class _Sched:
    """ctypes face of the C++ scheduler / block manager (``runtime/csrc/scheduler.cpp``)."""

    def __init__(self, num_blocks, block_size, max_running, max_prefill_tokens):
        self.lib = _lib.runtime()
        L = self.lib
        L.gkrt_sched_create.restype = ctypes.c_void_p
        L.gkrt_sched_create.argtypes = [ctypes.c_int] * 4
        for fn, args, res in (
            ("gkrt_sched_destroy", [ctypes.c_void_p], None),
            ("gkrt_sched_add", [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int], ctypes.c_int),
            ("gkrt_sched_fork", [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                 ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)], ctypes.c_int),
            ("gkrt_sched_step", [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64), ctypes.c_int,
                                 ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int64), ctypes.c_int,
                                 ctypes.POINTER(ctypes.c_int)], ctypes.c_int),
            ("gkrt_sched_commit", [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int], None),
            ("gkrt_sched_finish", [ctypes.c_void_p, ctypes.c_int64], None),
            ("gkrt_sched_abort_all", [ctypes.c_void_p], None),
            ("gkrt_sched_reserve", [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int], ctypes.c_int),
            ("gkrt_sched_advance", [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int], None),
            ("gkrt_sched_batch_tables", [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64), ctypes.c_int,
                                         ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.POINTER(ctypes.c_int)],
             ctypes.c_int),
            ("gkrt_sched_stats", [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64)], None),
        ):
            f = getattr(L, fn)
            f.argtypes, f.restype = args, res
        self.h = L.gkrt_sched_create(num_blocks, block_size, max_running, max_prefill_tokens)

    def __del__(self):
        try:
            self.lib.gkrt_sched_destroy(self.h)
        except Exception:
            pass

    def add(self, rid, prompt_len, max_new):
        return self.lib.gkrt_sched_add(self.h, rid, prompt_len, max_new)

    def fork(self, parent, child, max_new):
        a, b = ctypes.c_int(), ctypes.c_int()
        rc = self.lib.gkrt_sched_fork(self.h, parent, child, max_new, ctypes.byref(a), ctypes.byref(b))
        return rc, a.value, b.value

    def step(self, cap_prefill, cap_decode):
        pre = (ctypes.c_int64 * max(cap_prefill, 1))()
        dec = (ctypes.c_int64 * max(cap_decode, 1))()
        npre, ndec = ctypes.c_int(), ctypes.c_int()
        self.lib.gkrt_sched_step(self.h, pre, cap_prefill, ctypes.byref(npre), dec, cap_decode, ctypes.byref(ndec))
        return list(pre[:npre.value]), list(dec[:ndec.value])

    def commit(self, rid, is_prefill):
        self.lib.gkrt_sched_commit(self.h, rid, int(is_prefill))

    def reserve(self, rid, tokens):
        return self.lib.gkrt_sched_reserve(self.h, rid, tokens)

    def advance(self, rid, tokens):
        self.lib.gkrt_sched_advance(self.h, rid, tokens)

    def finish(self, rid):
        self.lib.gkrt_sched_finish(self.h, rid)

    def abort_all(self):
        self.lib.gkrt_sched_abort_all(self.h)

    def tables(self, rids, max_blocks):
        n = len(rids)
        ids = (ctypes.c_int64 * max(n, 1))(*rids)
        tab = (ctypes.c_int * (max(n, 1) * max_blocks))()
        cached = (ctypes.c_int * max(n, 1))()
        rc = self.lib.gkrt_sched_batch_tables(self.h, ids, n, tab, max_blocks, cached)
        assert rc == 0
        return (torch.frombuffer(tab, dtype=torch.int32).view(max(n, 1), max_blocks)[:n].clone(),
                torch.frombuffer(cached, dtype=torch.int32)[:n].clone())

    def stats(self):
        out = (ctypes.c_int64 * 8)()
        self.lib.gkrt_sched_stats(self.h, out)
        return dict(free_blocks=out[0], running=out[1], waiting=out[2], preemptions=out[3], num_blocks=out[4])


def _count_launches() -> int:
    from ..ops import attention, gemm, optim, rl, vocab
    return sum(sum(m.LAUNCHES.values()) for m in (attention, fused, gemm, optim, rl, vocab))


class LayerWeights:
    __slots__ = ("ln1", "qkv_w", "qkv_b", "o_w", "ln2", "fc1_w", "fc2_w", "q_ln", "k_ln", "sinks", "window", "moe",
                 "mla", "fp8")  # fp8: {"qkv_w": (e4m3 codes, 128x128 fp32 scales), ...} when the engine serves in block fp8


class RolloutWeights:
    """Views of one model shard's parameters in the layout the decoder consumes.  ``from_model`` shares storage with
    a ``GPTModel`` (zero-copy); ``clone_from_model`` owns its tensors (separate rollout copy, needed when the engine
    must keep serving while the trainer's weights move)."""

    def __init__(self):
        self.layers: List[LayerWeights] = []
        self.embed = self.final_ln = self.head = None

    @staticmethod
    def _serving_module(module, clone: bool):
        """The trainer's module itself (shared storage) or, for a separate rollout copy, a deep copy whose parameters
        are plain tensors of their own (no gradient buffers, no optimizer hooks)."""
        if not clone:
            return module
        if any(getattr(p, "is_lora", False) for p in module.parameters()):
            raise NotImplementedError("a separate rollout copy of a latent-attention or MoE module that carries LoRA "
                                      "adapters is not supported: use policy.share_rollout_weights=true")
        import copy
        own = copy.deepcopy(module)
        for p in own.parameters():
            p.requires_grad_(False)
            for attr in ("main_grad", "grad"):
                if getattr(p, attr, None) is not None:
                    setattr(p, attr, None)
        return own

    @classmethod
    def from_model(cls, model, clone: bool = False):
        f = (lambda t: t.detach().clone()) if clone else (lambda t: t.detach())
        w = cls()
        model = getattr(model, "language_model", model)  # vision-language wrapper: the decoder is what serves
        w.embed = f(model.embedding.word_embeddings.weight)
        w.final_ln = f(model.decoder.final_layernorm.weight)
        w.head = f(model.output_weight())
        for layer in model.decoder.layers:
            lw = LayerWeights()
            lw.fp8 = None
            a = layer.self_attention
            lw.ln1 = f(layer.input_layernorm.weight)
            lw.mla = None
            if hasattr(a, "linear_kv_down_proj"):
                # multi-head latent attention: the module itself serves (its projections carry LoRA adapters and
                # fp8 wrappers as they are); the cache holds the latent and the shared rotated key
                lw.mla = cls._serving_module(a, clone)
                lw.qkv_w = lw.qkv_b = lw.o_w = lw.q_ln = lw.k_ln = lw.sinks = None
                lw.window = 0
                lw.ln2 = f(layer.pre_mlp_layernorm.weight)
                if layer.is_moe:
                    lw.moe = cls._serving_module(layer.mlp, clone)
                    lw.fc1_w = lw.fc2_w = None
                else:
                    lw.moe = None
                    lw.fc1_w = f(layer.mlp.linear_fc1.weight)
                    lw.fc2_w = f(layer.mlp.linear_fc2.weight)
                w.layers.append(lw)
                continue
            lw.qkv_w = f(a.linear_qkv.weight)
            lw.qkv_b = f(a.linear_qkv.bias) if a.linear_qkv.bias is not None else None
            lw.o_w = f(a.linear_proj.weight)
            lw.ln2 = f(layer.pre_mlp_layernorm.weight)
            lw.q_ln = f(a.q_layernorm.weight) if hasattr(a, "q_layernorm") else None
            lw.k_ln = f(a.k_layernorm.weight) if hasattr(a, "k_layernorm") else None
            lw.sinks = f(a.sinks) if getattr(a, "sinks", None) is not None else None
            lw.window = a.window
            if layer.is_moe:
                # the module serves as it is (router + experts); a separate rollout copy owns a deep copy of it
                lw.moe = cls._serving_module(layer.mlp, clone)
                lw.fc1_w = lw.fc2_w = None
            else:
                lw.moe = None
                lw.fc1_w = f(layer.mlp.linear_fc1.weight)
                lw.fc2_w = f(layer.mlp.linear_fc2.weight)
            w.layers.append(lw)
        return w

    def tensors(self):
        for t in (self.embed, self.final_ln, self.head):
            yield t
        for lw in self.layers:
            for k in ("ln1", "qkv_w", "qkv_b", "o_w", "ln2", "fc1_w", "fc2_w", "q_ln", "k_ln", "sinks"):
                t = getattr(lw, k)
                if t is not None:
                    yield t


class InferEngine:
    def __init__(self, cfg: ModelConfig, weights: RolloutWeights, tp_size: int = 1, tp_group=None,
                 max_running_requests: int = 64, max_model_len: int = 2048, kv_block_size: int = 16,
                 num_kv_blocks: Optional[int] = None, gpu_memory_utilization: float = 0.7,
                 max_prefill_tokens: int = 16384, use_cuda_graph: bool = True, sync_interval: int = 8,
                 eos_token_id: Optional[int] = None, device=None, max_sync_interval: int = 64):
        self.cfg, self.w = cfg, weights
        self.tp, self.tp_group = tp_size, tp_group
        self.device = device or weights.embed.device
        self.max_running = max_running_requests
        self.max_model_len = max_model_len
        self.bs = kv_block_size
        self.max_blocks = (max_model_len + kv_block_size - 1) // kv_block_size + 1
        self.hq = cfg.num_attention_heads // tp_size
        self.hk = cfg.num_kv_heads // tp_size
        self.D = cfg.head_dim
        self.mla_dim = (cfg.kv_lora_rank + cfg.qk_rope_head_dim) if getattr(cfg, "use_mla", False) else 0
        self._mla_abs: Dict[int, list] = {}   # id(attention module) -> [absorbed up-projection, stale]
        self.vocab_local = weights.head.shape[0]
        self.vocab_start = self.vocab_local * (dist.get_rank(tp_group) if (tp_group is not None and tp_size > 1) else 0)
        # the library (eager) backend launches its decode ops one by one (its GPU path has no host synchronisation, so
        # the launch queue stays ahead of the device)
        self.use_graph = use_cuda_graph and self.device.type == "cuda" and not _lib.force_eager()
        self.ep_group = None  # set when experts are parallel: engines of the group then run their passes in lockstep
        if any(getattr(lw.moe, "ep_size", 1) > 1 for lw in weights.layers if lw.moe is not None):
            self.ep_group = ps.get_expert_model_parallel_group()
            # The NCCL dispatch sizes its exchanges on the host, so a decode step over it cannot be replayed from a
            # captured graph.  The peer-memory dispatch plans on the device and keeps its call / barrier epochs in
            # device memory (parallel/ep_fused.py), so its decode steps are captured like the dense ones; the
            # engines of the group replay in lockstep (same number of steps between two host agreements).
            fused_ep = (self.device.type == "cuda" and not _lib.force_eager()
                        and os.environ.get("GCORE_FUSED_EP", "1") != "0"
                        and os.environ.get("GCORE_EP_DECODE_GRAPH", "1") != "0"
                        and hasattr(_lib.kernels(), "gk_ep_plan_dev") and dist.get_world_size(self.ep_group) <= 8
                        and cfg.hidden_size % 8 == 0)
            if not fused_ep:
                self.use_graph = False
        # decode steps between two host synchronisations: ``sync_interval`` while requests wait for a slot (a finished
        # request should hand its slot over soon), up to ``max_sync_interval`` when nothing waits (then only the
        # discarded tokens after an early stop are at stake, and every synchronisation costs the GPU an idle gap)
        self.sync_interval = max(1, sync_interval)
        self.max_sync_interval = max(self.sync_interval, max_sync_interval)
        self.eos = eos_token_id
        self.gpu_memory_utilization = gpu_memory_utilization
        self._num_blocks_cfg = num_kv_blocks
        self.max_prefill_tokens = max_prefill_tokens
        self.k_cache: List[torch.Tensor] = []
        self.v_cache: List[torch.Tensor] = []
        self.sched: Optional[_Sched] = None
        self.requests: Dict[int, Request] = {}
        self._next_rid = 0
        self._graphs: Dict[int, tuple] = {}
        self._state = None
        self.asleep = {"weights": False, "kv_cache": True}
        self.stats = dict(decode_steps=0, prefill_tokens=0, generated_tokens=0, graph_replays=0)
        self.record_routed_experts = False
        self._peer_ar = None
        self.weight_scales: dict = {}  # name -> fp32 128x128 block scales when weights are held in e4m3

    # ------------------------------------------------------------------ memory
    def _kv_bytes_per_block(self):
        if self.mla_dim:
            return len(self.w.layers) * self.bs * self.mla_dim * 2
        return 2 * len(self.w.layers) * self.bs * self.hk * self.D * 2

    def wake_up(self, tags: Sequence[str] = ("weights", "kv_cache")):
        """Allocates the KV cache (tag ``kv_cache``); weights are shared storage and are always resident."""
        if "kv_cache" in tags and self.asleep["kv_cache"]:
            n = self._num_blocks_cfg
            if n is None:
                need = self.max_running * self.max_blocks + 8
                if self.device.type == "cuda":
                    free, total = torch.cuda.mem_get_info(self.device)
                    budget = int(free * self.gpu_memory_utilization)
                    n = max(min(need, budget // self._kv_bytes_per_block()), self.max_blocks + 1)
                else:
                    n = need
            self.num_blocks = n
            dt = self.w.embed.dtype
            if self.mla_dim:
                # latent cache: one row of (kv_lora + rope) values per token, shared by all heads; block ``n`` is a
                # sink for the rows of inactive batch slots
                self.k_cache = [torch.zeros(n + 1, self.bs, 1, self.mla_dim, dtype=dt, device=self.device)
                                for _ in self.w.layers]
                self.v_cache = [torch.zeros(n + 1, 0, dtype=dt, device=self.device) for _ in self.w.layers]
            else:
                self.k_cache = [torch.zeros(n, self.bs, self.hk, self.D, dtype=dt, device=self.device)
                                for _ in self.w.layers]
                self.v_cache = [torch.zeros(n, self.bs, self.hk, self.D, dtype=dt, device=self.device)
                                for _ in self.w.layers]
            self.sched = _Sched(n, self.bs, self.max_running, self.max_prefill_tokens)
            self.asleep["kv_cache"] = False
            self._graphs.clear()
        if "weights" in tags:
            self.asleep["weights"] = False

    def sleep(self, tags: Sequence[str] = ("kv_cache",)):
        """Releases the KV cache (and the captured graphs that reference it) so the trainer can use the memory."""
        if "kv_cache" in tags and not self.asleep["kv_cache"]:
            self._graphs.clear()
            self._state = None
            self.k_cache, self.v_cache = [], []
            self.sched = None
            self.asleep["kv_cache"] = True
            if self.device.type == "cuda":
                torch.cuda.empty_cache()
        if "weights" in tags:
            self.asleep["weights"] = True
            if getattr(self, "owns_weights", False):
                # a separate rollout copy is only needed while the engine serves: drop it, the next weight update
                # rebuilds it (the reference's engines release their weights in sleep mode the same way)
                self.w = None
                self._graphs.clear()
                if self.device.type == "cuda":
                    torch.cuda.empty_cache()

    def load_weights_from(self, model, bucket_mb: int = 512):
        """Rebuilds an owned rollout copy from ``model`` through a staging bucket of ``bucket_mb``: every tensor is
        copied into the bucket and from the bucket into the engine's own storage - the byte traffic of the reference's
        export -> flattened bucket -> engine ``load_weights`` hand-over on one GPU
        (gpatch_v4/client/update_weight_factory.py:271-379)."""
        w = RolloutWeights.from_model(model, clone=False)
        own = RolloutWeights.from_model(model, clone=False)
        stage = torch.empty(bucket_mb << 20, dtype=torch.uint8, device=self.device)
        moved = 0

        def via_bucket(t):
            nonlocal moved
            if t is None or not isinstance(t, torch.Tensor):
                return t
            n = t.numel() * t.element_size()
            moved += n
            if n > stage.numel():
                return t.detach().clone()
            b = stage[:n].view(t.dtype).view(t.shape)
            b.copy_(t)
            return b.clone()

        own.embed, own.final_ln, own.head = via_bucket(w.embed), via_bucket(w.final_ln), via_bucket(w.head)
        for lo, lw in zip(own.layers, w.layers):
            for k in ("ln1", "qkv_w", "qkv_b", "o_w", "ln2", "fc1_w", "fc2_w", "q_ln", "k_ln", "sinks"):
                setattr(lo, k, via_bucket(getattr(lw, k)))
        del stage
        self.w = own
        self.owns_weights = True
        self.asleep["weights"] = False
        self._graphs.clear()
        self._mla_abs.clear()   # the latent-attention modules of the new copy get fresh absorbed matrices
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        return moved

    def flush_cache(self):
        if self.sched is not None:
            self.sched.abort_all()
        self.requests.clear()

    def abort_all_requests(self):
        self.flush_cache()

    def get_load(self):
        return self.sched.stats() if self.sched is not None else dict(running=0, waiting=0)

    def update_weights(self, weights: Optional[RolloutWeights] = None):
        """Shared storage: nothing moves; a new ``RolloutWeights`` re-points the engine (captured graphs are dropped
        because they hold the old addresses)."""
        if weights is not None and weights is not self.w:
            same = all(a.data_ptr() == b.data_ptr() for a, b in zip(self.w.tensors(), weights.tensors()))
            self.w = weights
            if not same:
                self._graphs.clear()
        if getattr(self, "fp8_enabled", False):
            self.quantize_weights_fp8()
        for ent in self._mla_abs.values():
            ent[1] = True
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()

    # ------------------------------------------------------------------ block-fp8 serving
    def quantize_weights_fp8(self):
        """(Re)builds e4m3 + 128x128-scale copies of every dense projection whose contraction length is a multiple of
        128; called after each weight hand-over when the engine serves in fp8 (the reference's fp8 rollout:
        gpatch_v4/generation_backend/sglang_model_specific/sglang_weight_update_dsv4.py:267-321)."""
        from ..ops.quant import quant_weight_128x128
        self.fp8_enabled = True
        for lw in self.w.layers:
            lw.fp8 = {}
            for name in ("qkv_w", "o_w", "fc1_w", "fc2_w"):
                w = getattr(lw, name)
                if w is not None and w.dim() == 2 and w.shape[1] % 128 == 0:
                    lw.fp8[name] = quant_weight_128x128(w.to(torch.bfloat16).contiguous())
        self._graphs.clear()

    def _lin(self, h, lw: LayerWeights, name: str, bias=None):
        if lw.fp8 and name in lw.fp8:
            from ..ops import quant
            q, sc = lw.fp8[name]
            aq, asc = quant.quant_act_1x128(h.to(torch.bfloat16).contiguous())
            y = quant.gemm_fp8_blockscaled(aq, asc, q, sc, out_dtype=torch.bfloat16).to(h.dtype)
            return y + bias if bias is not None else y
        return linear_forward(h, getattr(lw, name), bias)

    # ------------------------------------------------------------------ model math (no autograd)
    def _ensure_peer_ar(self, x):
        if self._peer_ar is None and self.device.type == "cuda" and not _lib.force_eager() \
                and x.dtype == torch.bfloat16 and os.environ.get("GCORE_PEER_ALLREDUCE", "1") != "0":
            from ..parallel.symm import PeerAllReduce
            self._peer_ar = PeerAllReduce(self.tp_group, self.max_running * self.cfg.hidden_size, self.device)

    def _allreduce(self, x):
        if self.tp > 1:
            self._ensure_peer_ar(x)
            if self._peer_ar is not None and x.numel() <= self._peer_ar.slot and x.is_contiguous():
                return self._peer_ar.all_reduce(x)  # one-shot push over NVLink peer memory (decode-sized tensors)
            dist.all_reduce(x, group=self.tp_group)
        return x

    def _reduce_norm(self, partial, gamma, res, pending: bool):
        """``RMSNorm(all_reduce(partial) + res)`` and the new residual.  ``pending``: ``partial`` still holds this
        rank's partial sums; on the peer-memory path the all-reduce, the residual add and the norm are then one
        kernel that reads the peers' partials (tensor-parallel decode), otherwise all-reduce and norm run one after
        the other."""
        if pending and self.tp > 1:
            self._ensure_peer_ar(partial)
            # opt-in: in the two-GPU GRPO step the single kernel measured 2 % behind the one-shot all-reduce followed
            # by the norm kernel (rollout 5.91 s against 5.80 s, and 5.71 s against 5.60 s with its first version)
            if self._peer_ar is not None and os.environ.get("GCORE_FUSED_AR_NORM", "0") == "1":
                out = self._peer_ar.all_reduce_rmsnorm(partial, res, gamma, self.cfg.rms_norm_eps)
                if out is not None:
                    return out
            partial = self._allreduce(partial)
        return fused.rmsnorm(partial, gamma, self.cfg.rms_norm_eps, res)

    def _mlp(self, lw: LayerWeights, h, reduce: bool = True):
        """Feed-forward block; with ``reduce=False`` a dense block returns this rank's partial sums (second value
        True) and leaves the all-reduce to the caller."""
        if lw.moe is not None:
            was = lw.moe.training
            lw.moe.eval()
            y, _ = lw.moe(h)
            if was:
                lw.moe.train()
            return y if reduce else (y, False)
        g = self._lin(h, lw, "fc1_w")
        y = self._lin(fused.swiglu(g), lw, "fc2_w")
        return self._allreduce(y) if reduce else (y, self.tp > 1)

    def _embed(self, tokens):
        if self.tp == 1:
            return torch.nn.functional.embedding(tokens, self.w.embed)
        local = tokens - self.vocab_start
        mine = (local >= 0) & (local < self.vocab_local)
        x = self.w.embed[local.clamp(0, self.vocab_local - 1)] * mine[:, None].to(self.w.embed.dtype)
        return self._allreduce(x)

    def _qk_norm(self, lw, qkv, T):
        if lw.q_ln is None:
            return qkv
        return fused.qk_headnorm_(qkv, lw.q_ln, lw.k_ln, self.hq, self.hk, self.D, self.cfg.rms_norm_eps)

    @torch.no_grad()
    def _prefill(self, tokens, pos, cu, max_len, slots, embed_rows=None):
        """Packed prompts through all layers; K/V go to the cache; returns the last-token hidden of every prompt.
        ``embed_rows = (row_index, rows)`` overwrites embedding rows (image features at placeholder tokens)."""
        cfg = self.cfg
        T = tokens.numel()
        x = self._embed(tokens)
        if embed_rows is not None:
            x = x.index_copy(0, embed_rows[0], embed_rows[1].to(x.dtype))
        res = None
        for li, lw in enumerate(self.w.layers):
            h, res = fused.rmsnorm(x, lw.ln1, cfg.rms_norm_eps, res)
            if lw.mla is not None:
                q_nope, q_rope, c_kv, k_rope = lw.mla.project(h, pos)
                sink = (self.k_cache[li].shape[0] - 1) * self.bs  # rows without a slot land in the spare block
                self.k_cache[li].view(-1, self.mla_dim).index_copy_(
                    0, torch.where(slots >= 0, slots, torch.full_like(slots, sink)).long(),
                    torch.cat([self._mla_cached_latent(lw.mla, c_kv), k_rope], -1))
                a = self._allreduce(lw.mla.linear_proj(lw.mla.attend(q_nope, q_rope, c_kv, k_rope, cu, max_len)))
                h, res = fused.rmsnorm(a, lw.ln2, cfg.rms_norm_eps, res)
                x = self._mlp(lw, h)
                continue
            qkv = self._lin(h, lw, "qkv_w", lw.qkv_b)
            qkv = self._qk_norm(lw, qkv, T)
            kv_append_rope(qkv, pos, slots, self.k_cache[li], self.v_cache[li], self.hq, self.hk, self.D,
                           cfg.rope_theta, cfg.rotary_dim)
            v3 = qkv.view(T, self.hq + 2 * self.hk, self.D)
            o = flash_attn_varlen(v3[:, :self.hq], v3[:, self.hq:self.hq + self.hk], v3[:, self.hq + self.hk:], cu, cu,
                                  max_len, max_len, causal=True, window=lw.window, sinks=lw.sinks)
            a = self._allreduce(self._lin(o.reshape(T, self.hq * self.D), lw, "o_w"))
            h, res = fused.rmsnorm(a, lw.ln2, cfg.rms_norm_eps, res)
            x = self._mlp(lw, h)
        last = (cu[1:] - 1).long()
        hl, _ = fused.rmsnorm(x[last], self.w.final_ln, cfg.rms_norm_eps, res[last])
        return hl

    @torch.no_grad()
    def _decode_math(self, st):
        """One token for every row of the batch state ``st`` (all tensors static: graph-capturable).  The chain of
        ~10 short kernels per layer is launched with programmatic dependent launch: each kernel's set-up (and, for the
        cluster GEMM, its first weight tiles) overlaps the tail of the one before (``GCORE_PDL=0`` disables)."""
        pdl = (self.device.type == "cuda" and not _lib.force_eager() and os.environ.get("GCORE_PDL", "1") != "0"
               and hasattr(_lib.kernels(), "gk_set_pdl"))
        if pdl:
            _lib.kernels().gk_set_pdl(1)
        try:
            if self.ep_group is not None:
                # expert-parallel layers of a decode step run on peer buffers sized for the (static, rank-uniform)
                # decode batch instead of a training micro-batch
                from ..parallel.ep_fused import small_batch
                with small_batch(st["tokens"].numel()):
                    self._decode_layers(st)
            else:
                self._decode_layers(st)
        finally:
            if pdl:
                _lib.kernels().gk_set_pdl(0)

    def _decode_layers(self, st):
        cfg = self.cfg
        B = st["tokens"].numel()
        pos = st["pos"]
        blk = st["block_table"].gather(1, (pos // self.bs).long()[:, None]).squeeze(1)
        slots = torch.where(st["active"], blk * self.bs + pos % self.bs, torch.full_like(pos, -1))
        ctx = torch.where(st["active"], pos + 1, torch.zeros_like(pos))
        x = self._embed(st["tokens"])
        res = None
        if self.mla_dim:
            sink = (self.k_cache[0].shape[0] - 1) * self.bs
            lat_slots = torch.where(slots >= 0, slots, torch.full_like(slots, sink)).long()
            lat_idx = lat_mask = None
            if not self._mla_native():
                # eager form: latent rows of every request, gathered once per step for all layers' index arithmetic
                p_all = torch.arange(self.max_model_len, device=pos.device)
                lat_idx = (st["block_table"].long()[:, p_all // self.bs] * self.bs + p_all % self.bs)  # [B, Lmax]
                lat_mask = p_all[None, :] < ctx[:, None]
        pending = False   # x still holds this rank's partial sums of the previous block's row-parallel projection
        for li, lw in enumerate(self.w.layers):
            h, res = self._reduce_norm(x, lw.ln1, res, pending)
            if lw.mla is not None:
                o = self._mla_decode(lw.mla, h, pos, self.k_cache[li], lat_slots, lat_idx, lat_mask,
                                     paged=(st["block_table"], ctx))
                h, res = self._reduce_norm(lw.mla.linear_proj(o), lw.ln2, res, self.tp > 1)
                x, pending = self._mlp(lw, h, reduce=False)
                continue
            qkv = self._lin(h, lw, "qkv_w", lw.qkv_b)
            qkv = self._qk_norm(lw, qkv, B)
            # rotary embedding, cache append and attention: one kernel where the tensor-core decode kernel serves
            # the shape, else the two kernels in sequence
            o = paged_decode_append(qkv, pos, slots, self.k_cache[li], self.v_cache[li], st["block_table"], ctx,
                                    self.max_model_len, self.hq, self.hk, self.D, cfg.rope_theta, cfg.rotary_dim,
                                    window=lw.window, sinks=lw.sinks)
            h, res = self._reduce_norm(self._lin(o.view(B, self.hq * self.D), lw, "o_w"), lw.ln2, res, self.tp > 1)
            x, pending = self._mlp(lw, h, reduce=False)
        hl, _ = self._reduce_norm(x, self.w.final_ln, res, pending)
        self._sample_into(hl, st)
        # state advance
        st["pos"].add_(st["active"].to(pos.dtype))
        st["steps"].add_(1)
        st["ring_idx"].add_(1)

    def _ep_any(self, *flags):
        """Logical OR of each flag over the engines of the expert-parallel group (one small all-reduce)."""
        dev = self.device if dist.get_backend(self.ep_group) == "nccl" else torch.device("cpu")
        t = torch.tensor([float(bool(f)) for f in flags], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.ep_group)
        return [bool(x) for x in t.tolist()]

    @staticmethod
    def _mla_cached_latent(mla, c_kv):
        """What the cache keeps of the latent.  When the kv up-projection computes in block fp8 the trainer multiplies
        the 1x128-quantised latent with the 128x128-quantised weight; the absorbed decode reproduces that product
        exactly by caching the quantise -> dequantise image of the latent (and absorbing the dequantised weight)."""
        up = mla.linear_kv_up_proj
        if getattr(up, "precision", None) == "fp8" and c_kv.shape[-1] % 128 == 0:
            from ..ops import quant
            q, sc = quant.quant_act_1x128(c_kv.to(torch.bfloat16).contiguous())
            return quant.dequant_1x128(q, sc).to(c_kv.dtype)
        return c_kv

    @staticmethod
    def _mla_up_weight(mla):
        up = mla.linear_kv_up_proj
        w = up.weight
        if getattr(up, "precision", None) == "fp8" and w.shape[1] % 128 == 0:
            from ..ops import quant
            q, sc = quant.quant_weight_128x128(w.detach().to(torch.bfloat16).contiguous())
            w = quant.dequant_128x128(q, sc)[:w.shape[0], :w.shape[1]].to(up.weight.dtype)
        return w

    def _mla_absorbed(self, mla):
        """The kv up-projection as ``[heads, nope + v, kv_lora]`` with adapters folded in (and, for block-fp8 layers,
        after the quantise -> dequantise round trip): what the absorbed decode multiplies the query and the latent
        output with.  Derived once per weight version, not per decode step: ``update_weights`` marks the copies stale
        and ``generate`` rewrites them in place before it decodes (captured graphs keep reading the same storage)."""
        cfg = self.cfg
        dn, dv, C = cfg.qk_nope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        ent = self._mla_abs.get(id(mla))
        if ent is None or ent[1]:
            w_up = self._mla_up_weight(mla).view(mla.h, dn + dv, C)
            up_lora = getattr(mla.linear_kv_up_proj, "lora", None)
            if up_lora is not None:  # adapters on the up-projection: fold their delta into the absorbed matrices
                w_up = w_up + up_lora.delta_weight().view(mla.h, dn + dv, C).to(w_up.dtype)
            if ent is None:
                ent = [w_up.contiguous().clone(), False]
                self._mla_abs[id(mla)] = ent
            else:
                ent[0].copy_(w_up)
                ent[1] = False
        return ent[0]

    def _mla_native(self) -> bool:
        """Whether the decode step runs the latent-attention kernel (bf16 cache on a GPU, a built geometry)."""
        cfg = self.cfg
        if self.device.type != "cuda" or _lib.force_eager() or os.environ.get("GCORE_MLA_DECODE", "1") == "0":
            return False
        if self.k_cache is None or self.k_cache[0].dtype != torch.bfloat16:
            return False
        lib = _lib.kernels()
        return hasattr(lib, "gk_mla_decode_supported") and \
            bool(lib.gk_mla_decode_supported(cfg.kv_lora_rank, cfg.qk_rope_head_dim))

    def _mla_decode(self, mla, h, pos, cache, slots, lat_idx, lat_mask, paged=None):
        """One token per request of multi-head latent attention on the latent cache, in the absorbed form: the key
        up-projection is folded into the query and the value up-projection is applied after the weighted sum, so a
        step reads ``kv_lora + rope`` values per cached token instead of per-head keys and values
        (the role of the latent decode kernels the reference reaches through its serving engines)."""
        cfg = self.cfg
        dn, dr, dv, C = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        B = h.shape[0]
        q_nope, q_rope, c_kv, k_rope = mla.project(h, pos)
        flat = cache.view(-1, self.mla_dim)
        flat.index_copy_(0, slots, torch.cat([self._mla_cached_latent(mla, c_kv), k_rope], -1))
        w_up = self._mla_absorbed(mla)
        if lat_idx is None:
            # latent decode kernel straight on the paged cache: the two absorbed projections are head-batched GEMMs
            # in head-major layout, which the kernel reads and writes through strides
            block_table, ctx = paged
            q_lat = torch.bmm(q_nope.transpose(0, 1), w_up[:, :dn])                   # [h, B, C]
            o_lat = torch.empty_like(q_lat)
            mla_paged_decode(q_lat.transpose(0, 1), q_rope, cache.view(-1, self.bs, self.mla_dim), block_table, ctx,
                             self.max_model_len, 1.0 / math.sqrt(dn + dr), out=o_lat.transpose(0, 1))
            o = torch.bmm(o_lat, w_up[:, dn:].transpose(1, 2))                        # [h, B, dv]
            return o.transpose(0, 1).reshape(B, mla.h * dv)
        lat = flat[lat_idx]                                            # [B, Lmax, C + dr]
        q_abs = torch.einsum("bhd,hdc->bhc", q_nope.float(), w_up[:, :dn].float())
        s = torch.einsum("bhc,blc->bhl", q_abs, lat[..., :C].float())
        s = s + torch.einsum("bhr,blr->bhl", q_rope.float(), lat[..., C:].float())
        s = (s / math.sqrt(dn + dr)).masked_fill(~lat_mask[:, None, :], float("-inf"))
        p = torch.softmax(s, -1)
        p = torch.where(lat_mask[:, None, :], p, torch.zeros_like(p))   # rows of inactive slots: all masked -> zeros
        o_lat = torch.einsum("bhl,blc->bhc", p, lat[..., :C].float())
        o = torch.einsum("bhc,hvc->bhv", o_lat, w_up[:, dn:].float())
        return o.reshape(B, mla.h * dv).to(h.dtype)

    def _sample_into(self, hidden, st):
        logits = linear_forward(hidden, self.w.head, out_dtype=torch.float32)
        sp = st["params"]
        penalise = sp.get("repetition_penalty", 1.0) != 1.0
        if penalise:
            logits = self._penalise_seen(logits, st, self.vocab_start if self.tp > 1 else 0)
        if sp["filtered"]:
            tp_group, vocab_start = (self.tp_group, self.vocab_start) if self.tp > 1 else (None, 0)
            if self.tp > 1:
                # top-k / top-p / min-p are properties of the whole distribution: the k-th value and the nucleus
                # threshold of a vocabulary shard are not those of the vocabulary.  Gather the shards, filter the
                # full row on every rank (same result everywhere: the sampler's random stream depends only on
                # seed, step and token id), and sample without a cross-rank merge.
                parts = [torch.empty_like(logits) for _ in range(self.tp)]
                dist.all_gather(parts, logits.contiguous(), group=self.tp_group)
                logits = torch.cat(parts, dim=1)
                tp_group, vocab_start = None, 0
            tok, lp = sample_filtered(logits.contiguous(), sp["temperature"], sp["top_k"], sp["top_p"], sp["min_p"],
                                      st["seeds"], st["steps"], sp["greedy"])
        else:
            tok, lp = sample(logits, sp["temperature"], st["seeds"], st["steps"], sp["greedy"],
                             self.tp_group if self.tp > 1 else None, self.vocab_start)
        st["tokens"].copy_(tok)
        if penalise:
            st["seen"].scatter_(1, tok[:, None], True)
        idx = st["ring_idx"] % st["ring_tok"].shape[0]
        st["ring_tok"].index_copy_(0, idx, tok[None])
        st["ring_lp"].index_copy_(0, idx, lp[None])

    # ------------------------------------------------------------------ state / graphs
    def _new_state(self, B, params: SamplingParams):
        dev = self.device
        R = self.max_sync_interval
        return dict(
            tokens=torch.zeros(B, dtype=torch.int64, device=dev), pos=torch.zeros(B, dtype=torch.int32, device=dev),
            active=torch.zeros(B, dtype=torch.bool, device=dev),
            block_table=torch.zeros(B, self.max_blocks, dtype=torch.int32, device=dev),
            seeds=torch.zeros(B, dtype=torch.int64, device=dev), steps=torch.zeros(B, dtype=torch.int32, device=dev),
            ring_tok=torch.zeros(R, B, dtype=torch.int64, device=dev),
            ring_lp=torch.zeros(R, B, dtype=torch.float32, device=dev),
            ring_idx=torch.zeros(1, dtype=torch.int64, device=dev),
            params=dict(temperature=params.temperature, top_k=params.top_k, top_p=params.top_p, min_p=params.min_p,
                        greedy=params.greedy, repetition_penalty=float(params.repetition_penalty),
                        filtered=(params.top_k and params.top_k > 0) or params.top_p < 1.0 or params.min_p > 0.0),
            **({"seen": torch.zeros(B, self._vocab_total(), dtype=torch.bool, device=dev)}
               if params.repetition_penalty != 1.0 else {}))

    def _vocab_total(self) -> int:
        return self.w.head.shape[0] * self.tp

    def _penalise_seen(self, logits, st, start: int):
        """Repetition penalty on ``logits`` [B, n] = vocabulary ids ``start .. start + n`` (static shapes, no host
        synchronisation: part of the captured decode step)."""
        pen = st["params"]["repetition_penalty"]
        seen = st["seen"][:, start:start + logits.shape[1]]
        return torch.where(seen, torch.where(logits > 0, logits / pen, logits * pen), logits)

    def _run_decode(self, st):
        B = st["tokens"].numel()
        if not self.use_graph:
            self._decode_math(st)
            return
        g = self._graphs.get(B)
        if g is None or g[1] is not st:
            # warm up once eagerly on a side stream (allocates scratch, configures kernels), then capture
            keep = {k: v.clone() for k, v in st.items() if isinstance(v, torch.Tensor)}
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._decode_math(st)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            for k, v in keep.items():
                st[k].copy_(v)
            graph = torch.cuda.CUDAGraph()
            before = _count_launches()
            with torch.cuda.graph(graph):
                self._decode_math(st)
            self.graph_launches = _count_launches() - before  # our kernels inside one replay
            for k, v in keep.items():
                st[k].copy_(v)
            self._graphs[B] = (graph, st)
            g = self._graphs[B]
        g[0].replay()
        self.stats["graph_replays"] += 1

    # ------------------------------------------------------------------ public generate
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams, n: int = 1,
                 seeds: Optional[Sequence[int]] = None, image_embeds: Optional[Sequence] = None,
                 image_token_id: Optional[int] = None) -> List[Request]:
        """Generates ``n`` samples for every prompt; returns requests ordered ``[p0s0, p0s1, ..., p1s0, ...]``.
        Request ``(i, j)`` uses seed ``params.seed + i * n + j`` unless ``seeds`` is given
        (gpatch_v4/extended_model/llm.py:57-68).  Vision-language prompts: ``image_embeds[i]`` holds one row of
        merged vision features per ``image_token_id`` placeholder of prompt ``i`` (or None); the rows replace the
        placeholder embeddings in the prefill, decoding is unchanged."""
        if self.asleep["kv_cache"]:
            self.wake_up(("kv_cache",))
        if self.mla_dim:
            for lw in self.w.layers:   # re-derive stale absorbed matrices here, outside any graph capture
                if lw.mla is not None:
                    self._mla_absorbed(lw.mla)
        dev = self.device
        reqs: List[Request] = []
        if isinstance(prompts, torch.Tensor):
            prompts = prompts.tolist()
        vocab = self.cfg.vocab_size
        for i, p in enumerate(prompts):
            if len(p) and not (0 <= min(p) and max(p) < vocab):
                # checked on the host: an id outside the embedding table would otherwise trip a device-side assert
                raise ValueError(f"prompt {i} holds token ids outside [0, {vocab})")
        for i, p in enumerate(prompts):
            for j in range(n):
                rid = self._next_rid
                self._next_rid += 1
                sd = seeds[i * n + j] if seeds is not None else params.seed + i * n + j
                r = Request(rid, list(p), params, sd)
                r.prompt_index = i
                r.parent = reqs[i * n].rid if j > 0 else None
                reqs.append(r)
                self.requests[rid] = r
        parents = [r for r in reqs if r.parent is None]
        children: Dict[int, List[Request]] = {}
        for r in reqs:
            if r.parent is not None:
                children.setdefault(r.parent, []).append(r)
        for r in parents:
            rc = self.sched.add(r.rid, len(r.prompt), params.max_new_tokens)
            if rc != 0:
                raise ValueError(f"request of {len(r.prompt)} + {params.max_new_tokens} tokens cannot fit the KV cache")
        B = self.max_running
        st = self._state
        if st is None or st["tokens"].numel() != B or st["params"] != self._new_state(1, params)["params"]:
            st = self._new_state(B, params)
            self._state = st
            self._graphs.clear()
        slots_free = list(range(B - 1, -1, -1))
        slot_req: Dict[int, Request] = {}
        stop_ids = set(params.stop_token_ids) | ({self.eos} if self.eos is not None else set())
        host_tok = torch.zeros(B, dtype=torch.int64)
        host_pos = torch.zeros(B, dtype=torch.int32)
        host_active = torch.zeros(B, dtype=torch.bool)
        host_seed = torch.zeros(B, dtype=torch.int64)
        host_step = torch.zeros(B, dtype=torch.int32)
        host_bt = torch.zeros(B, self.max_blocks, dtype=torch.int32)
        if dev.type == "cuda":
            host_tok, host_pos, host_active, host_seed, host_step, host_bt = (
                t.pin_memory() for t in (host_tok, host_pos, host_active, host_seed, host_step, host_bt))
        # numpy views: scalar writes through a tensor cost microseconds each, and there are hundreds per interval
        n_tok, n_pos, n_active, n_seed, n_step = (t.numpy() for t in (host_tok, host_pos, host_active, host_seed,
                                                                      host_step))

        def place(r: Request, first_tok: int, first_lp: float):
            """Request enters the decode batch after its first token is known."""
            r.out_tokens.append(first_tok)
            r.out_logprobs.append(first_lp)
            if first_tok in stop_ids or len(r.out_tokens) >= params.max_new_tokens:
                r.finished, r.finish_reason = True, "stop" if first_tok in stop_ids else "length"
                self.sched.finish(r.rid)
                return
            s = slots_free.pop()
            r.slot = s
            slot_req[s] = r
            n_tok[s] = first_tok
            n_pos[s] = len(r.prompt)
            n_active[s] = True
            n_seed[s] = r.seed
            n_step[s] = 1
            if "seen" in st:   # the slot's table restarts from this request's prompt and first token
                st["seen"][s].zero_()
                st["seen"][s, torch.tensor(list(r.prompt) + [first_tok], dtype=torch.int64, device=dev)] = True

        while True:
            # ---- admit: a prompt enters only when its whole sample group fits the batch
            cap = len(slots_free) // max(n, 1)
            pre_ids, _ = self.sched.step(cap, 0) if cap > 0 else ([], [])
            if self.ep_group is not None and self._ep_any(bool(pre_ids))[0] and not pre_ids:
                # another engine of the expert-parallel group prefills now: join its all-to-alls with one dummy token
                self._prefill(torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, dtype=torch.int32, device=dev),
                              torch.tensor([0, 1], dtype=torch.int32, device=dev), 1,
                              torch.full((1,), -1, dtype=torch.int32, device=dev))
            if pre_ids:
                pre = [self.requests[i] for i in pre_ids]
                toks = torch.tensor([t for r in pre for t in r.prompt], dtype=torch.int64)
                lens = [len(r.prompt) for r in pre]
                cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
                pos = torch.cat([torch.arange(l, dtype=torch.int32) for l in lens])
                bt, _ = self.sched.tables(pre_ids, self.max_blocks)
                bidx = torch.repeat_interleave(torch.arange(len(pre)), torch.tensor(lens))
                slots = bt[bidx, (pos // self.bs).long()] * self.bs + pos % self.bs
                slots = slots.to(torch.int32)
                if dev.type == "cuda":
                    toks, pos, cu, slots = toks.pin_memory(), pos.pin_memory(), cu.pin_memory(), slots.pin_memory()
                io_counters.add_h2d(io_counters.tensor_bytes(toks, pos, cu, slots))
                embed_rows = None
                if image_embeds is not None:
                    rows_idx, feats, base = [], [], 0
                    for r, l in zip(pre, lens):
                        fe = image_embeds[r.prompt_index]
                        if fe is not None:
                            where = [base + k for k, t in enumerate(r.prompt) if t == image_token_id]
                            if len(where) != fe.shape[0]:
                                raise ValueError(f"prompt {r.prompt_index}: {len(where)} image placeholder tokens for "
                                                 f"{fe.shape[0]} vision feature rows")
                            rows_idx += where
                            feats.append(fe)
                        base += l
                    if rows_idx:
                        embed_rows = (torch.tensor(rows_idx, dtype=torch.int64, device=dev),
                                      torch.cat(feats).to(dev))
                hl = self._prefill(toks.to(dev, non_blocking=True), pos.to(dev, non_blocking=True),
                                   cu.to(dev, non_blocking=True), max(lens), slots.to(dev, non_blocking=True),
                                   embed_rows)
                self.stats["prefill_tokens"] += int(toks.numel())
                for r in pre:
                    self.sched.commit(r.rid, True)
                # the first token of a prompt's samples all come from the same last-position hidden state
                rows, owners = [], []
                for k, r in enumerate(pre):
                    for c in [r] + children.get(r.rid, []):
                        rows.append(k)
                        owners.append(c)
                hsel = hl[torch.tensor(rows, device=dev)]
                sd = torch.tensor([c.seed for c in owners], dtype=torch.int64, device=dev)
                tmp = dict(tokens=torch.zeros(len(owners), dtype=torch.int64, device=dev), seeds=sd,
                           steps=torch.zeros(len(owners), dtype=torch.int32, device=dev),
                           ring_tok=torch.zeros(1, len(owners), dtype=torch.int64, device=dev),
                           ring_lp=torch.zeros(1, len(owners), dtype=torch.float32, device=dev),
                           ring_idx=torch.zeros(1, dtype=torch.int64, device=dev), params=st["params"])
                if "seen" in st:
                    tmp["seen"] = torch.zeros(len(owners), self._vocab_total(), dtype=torch.bool, device=dev)
                    for k, c in enumerate(owners):
                        tmp["seen"][k, torch.tensor(c.prompt, dtype=torch.int64, device=dev)] = True
                self._sample_into(hsel, tmp)
                ft, fl = tmp["ring_tok"][0].tolist(), tmp["ring_lp"][0].tolist()
                io_counters.add_d2h(12 * len(owners))
                first = {c.rid: (t, l) for c, t, l in zip(owners, ft, fl)}
                # fork the samples before anything of the group can finish, then enter the decode batch
                copies = []
                for r in pre:
                    for c in children.get(r.rid, []):
                        rc, src, dst = self.sched.fork(r.rid, c.rid, params.max_new_tokens)
                        if rc != 0:
                            raise RuntimeError("KV cache exhausted while forking samples of a prompt; raise "
                                               "num_kv_blocks or lower max_running_requests")
                        if src >= 0:
                            copies.append((src, dst))
                if copies:
                    src = torch.tensor([a for a, _ in copies], device=dev)
                    dst = torch.tensor([b for _, b in copies], device=dev)
                    for li in range(len(self.w.layers)):
                        self.k_cache[li][dst] = self.k_cache[li][src]
                        self.v_cache[li][dst] = self.v_cache[li][src]
                for c in owners:
                    place(c, *first[c.rid])
            if self.ep_group is not None:
                # expert-parallel engines agree on what the group does next: decode if anyone has running requests,
                # stop only when everyone is done; an engine without requests decodes an all-inactive batch so that
                # its experts keep serving the others' tokens
                any_decode, any_left = self._ep_any(bool(slot_req), bool(slot_req) or self.sched.stats()["waiting"] > 0)
                if not any_left:
                    break
                if not slot_req:
                    if any_decode:
                        st["active"].zero_()
                        for _ in range(self.sync_interval):
                            self._run_decode(st)
                    continue
            if not slot_req:
                st_ = self.sched.stats()
                if st_["waiting"] == 0:
                    break
                if st_["running"] == 0 and not pre_ids:
                    raise RuntimeError("rollout engine cannot make progress: KV cache too small for one request")
                continue
            # ---- reserve KV for the next interval and push the batch state
            interval = self.sync_interval
            if self.sched.stats()["waiting"] == 0 and self.ep_group is None:
                # nobody waits for a slot: run until the first request reaches its length limit
                left = min(params.max_new_tokens - len(r.out_tokens) for r in slot_req.values())
                interval = max(interval, min(left, self.max_sync_interval))
            for s, r in list(slot_req.items()):
                remaining = params.max_new_tokens - len(r.out_tokens)
                self.sched.reserve(r.rid, min(interval, remaining) + 1)
            rids = [slot_req[s].rid if s in slot_req else -1 for s in range(B)]
            live = [s for s in range(B) if s in slot_req]
            bt, _ = self.sched.tables([rids[s] for s in live], self.max_blocks)
            host_bt.zero_()
            host_bt[torch.tensor(live)] = bt
            for k, src in (("tokens", host_tok), ("pos", host_pos), ("active", host_active), ("seeds", host_seed),
                           ("steps", host_step), ("block_table", host_bt)):
                st[k].copy_(src, non_blocking=True)
                io_counters.add_h2d(io_counters.tensor_bytes(src))
            st["ring_idx"].zero_()
            for _ in range(interval):
                self._run_decode(st)
            self.stats["decode_steps"] += interval
            ring_tok = st["ring_tok"].cpu()
            ring_lp = st["ring_lp"].cpu()
            io_counters.add_d2h(io_counters.tensor_bytes(ring_tok, ring_lp))
            # ---- harvest: one column of the ring per request, cut at its first stop token or at its length limit
            tok_np = ring_tok[:interval].t().contiguous().numpy()     # [B, interval]
            lp_np = ring_lp[:interval].t().contiguous().numpy()
            stop_hit = None
            if stop_ids:
                import numpy as np
                stop_hit = np.isin(tok_np, np.fromiter(stop_ids, dtype=tok_np.dtype))
            for s in live:
                r = slot_req[s]
                room = params.max_new_tokens - len(r.out_tokens)
                took = min(interval, room)
                reason = "length" if took == room else ""
                if stop_hit is not None:
                    hits = stop_hit[s, :took].nonzero()[0]
                    if hits.size:
                        took, reason = int(hits[0]) + 1, "stop"
                r.out_tokens.extend(tok_np[s, :took].tolist())
                r.out_logprobs.extend(lp_np[s, :took].tolist())
                self.stats["generated_tokens"] += took
                if reason:
                    r.finished, r.finish_reason = True, reason
                    self.sched.finish(r.rid)
                    del slot_req[s]
                    slots_free.append(s)
                    n_active[s] = False
                    n_pos[s] = 0
                else:
                    self.sched.advance(r.rid, interval)
                    n_tok[s] = r.out_tokens[-1]
                    n_pos[s] += interval
                    n_step[s] += interval
        for r in reqs:
            self.requests.pop(r.rid, None)
        return reqs
