"""Training engine: owns the model shard, the gradient / parameter buffers and the distributed optimizer of one rank.

Public verbs are those of the reference's ``BaseEngine`` (gpatch_v4/training_backend/base_engine.py:8-102):
``setup_model_and_get_optimizer``, ``compute_log_probs``, ``rl_train_actor``, ``finetune_step``, ``compute_values``,
``rl_train_value``, ``offload_* / onload_*``, ``export_weights``.  One implementation serves both back ends:
``native`` runs the sm_100a kernels, ``nccl_eager`` forces the PyTorch / library path of every op (the measured
baseline); collectives sit at the same call sites in both.

All sequence data is packed (THD).  Losses are normalised globally: per-token losses divide by the token count of the
whole global batch (all micro-batches, all DP ranks), per-sequence losses by the number of sequences.
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..core import parallel_state as ps
from ..core.packing import PackedBatch, make_microbatches, pack_samples
from ..loss import policy_loss as PL
from ..models.config import ModelConfig, build_model_config
from ..models.gpt import GPTModel
from ..models.lora import apply_lora, verify_lora_weight_consistency
from ..ops.rl import grpo_loss as fused_grpo_loss
from ..ops.vocab import linear_logprob_entropy
from ..utils import io_counters
from ..parallel.distributed_optimizer import DistributedDataParallel, DistributedOptimizer, lr_at_step


def _device():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


class FillerBatch(list):
    """Sample indices of a micro-batch that exists only so that every rank of a group runs the same number of
    micro-batches (each one carries the group's per-layer collectives).  It is packed like any other micro-batch,
    with its loss mask zeroed: it adds nothing to the loss, the gradients or the metrics, and its forward-only
    results are dropped."""


@contextlib.contextmanager
def backend_scope(backend: str):
    """``nccl_eager`` forces the eager implementation of every op for the duration of the call."""
    if backend != "nccl_eager":
        yield
        return
    old = os.environ.get("GCORE_B200_FORCE_EAGER")
    os.environ["GCORE_B200_FORCE_EAGER"] = "1"
    try:
        yield
    finally:
        if old is None:
            os.environ.pop("GCORE_B200_FORCE_EAGER", None)
        else:
            os.environ["GCORE_B200_FORCE_EAGER"] = old


class CPBatch(list):
    """Sample indices of a micro-batch that runs on its own context-parallel group (dynamic context parallelism:
    the group is the block of pool ranks its sequences were scheduled on; ``None`` = this rank alone)."""
    cp_group = None


class TrainingEngine:
    router_bias_violation = None
    _dcp = None       # dynamic context parallelism: {"pool": group, "groups": {(start, size): group}}
    _cur_cpg = None   # context-parallel group of the micro-batch packed last (dynamic context parallelism)   # (max, mean) load violation of the last router-bias update, when it is on

    def __init__(self, policy_cfg, optimizer_cfg, training_cfg, ppo_cfg=None, model_cfg: Optional[ModelConfig] = None,
                 role: str = "policy", value_head: bool = False, total_steps: Optional[int] = None,
                 vision_cfg=None, image_token_id: Optional[int] = None):
        self.policy_cfg, self.opt_cfg, self.train_cfg, self.ppo_cfg = policy_cfg, optimizer_cfg, training_cfg, ppo_cfg
        self.role = role
        if vision_cfg is None and getattr(policy_cfg, "vision_config", None):
            from ..models.vlm import VisionConfig
            vision_cfg = VisionConfig(**dict(policy_cfg.vision_config))
            image_token_id = policy_cfg.image_token_id if image_token_id is None else image_token_id
        self.vision_cfg, self.image_token_id = vision_cfg, image_token_id  # set: the model is a vision-language model
        self.value_head = value_head
        self.total_steps = total_steps
        self.backend = training_cfg.training_backend
        self.device = _device()
        self.model_cfg = model_cfg or build_model_config(policy_cfg.model_arch, policy_cfg.model_config)
        self.model: Optional[GPTModel] = None
        self.ref_model: Optional[GPTModel] = None
        self.ddp: Optional[DistributedDataParallel] = None
        self.optimizer: Optional[DistributedOptimizer] = None
        self.adapters = {}
        self.step = 0
        self.temperature = 1.0
        self.metrics_hooks: List[Callable] = []
        self.timers: Dict[str, float] = {}

    # ------------------------------------------------------------------ setup
    def _build(self, seed=None, value_head=False, recompute=None) -> GPTModel:
        d = self.policy_cfg.dist_config
        st = ps.get_state()
        tp = st.tp if st.initialized else 1
        ep = st.ep if st.initialized else 1
        if self.device.type == "cpu" and self.model_cfg.dtype == "bfloat16" and os.environ.get("GCORE_CPU_FP32", "1") == "1":
            pass
        pp = st.pp if st.initialized else 1
        stage_kw = {}
        if pp > 1:
            from ..parallel.pp import stage_layer_range
            stage = ps.get_pipeline_model_parallel_rank()
            assert not self.model_cfg.tie_word_embeddings, "tied embeddings are not supported across pipeline stages"
            vpp = d.virtual_pipeline_model_parallel_size or 1
            if vpp > 1:
                # interleaved stages: this rank holds chunks v = 0 .. vpp-1, chunk v being virtual stage v * pp + stage
                assert d.num_layers_in_first_pipeline_stage is None and d.num_layers_in_last_pipeline_stage is None, \
                    "uneven first / last stages are not combined with virtual pipeline stages"
                assert self.model_cfg.num_layers % (pp * vpp) == 0, "layers must divide evenly over pp * vpp chunks"
                rng = [stage_layer_range(self.model_cfg.num_layers, pp * vpp, v * pp + stage) for v in range(vpp)]
            else:
                rng = stage_layer_range(self.model_cfg.num_layers, pp, stage, d.num_layers_in_first_pipeline_stage,
                                        d.num_layers_in_last_pipeline_stage)
            stage_kw = dict(pre_process=stage == 0, post_process=stage == pp - 1, layer_range=rng)
        if self.vision_cfg is not None:
            from ..models.vlm import VLModel
            assert tp == 1 and pp == 1, "vision-language models run with TP = PP = 1"
            kw = dict(device=self.device, recompute=recompute if recompute is not None else self.policy_cfg.recompute,
                      value_head=value_head)
            if self.model_cfg.mrope_sections is not None:
                # multi-axis rotary ids: the Qwen3-VL family (images + videos, deepstack features)
                from ..models.qwen3_vl import Qwen3VLModel
                vopt = dict(getattr(self.policy_cfg, "vision_options", None) or {})
                m = Qwen3VLModel(self.model_cfg, self.vision_cfg, self.image_token_id,
                                 video_token_id=vopt.get("video_token_id"),
                                 deepstack_layers=tuple(vopt.get("deepstack_layers", (0,))),
                                 temporal_patch=int(vopt.get("temporal_patch", 2)), **kw)
            else:
                m = VLModel(self.model_cfg, self.vision_cfg, self.image_token_id, **kw)
        else:
            m = GPTModel(self.model_cfg, tp_size=tp, ep_size=ep, sequence_parallel=d.sequence_parallel,
                         recompute=recompute if recompute is not None else self.policy_cfg.recompute,
                         device=self.device, value_head=value_head, **stage_kw)
        m.recompute_num_layers = getattr(self.policy_cfg, "recompute_num_layers", None)
        if seed is not None:
            m.reset_parameters(seed)
        return m

    def setup_model_and_get_optimizer(self, seed: Optional[int] = None, with_ref: Optional[bool] = None):
        with_ref = (not self.policy_cfg.without_ref) if with_ref is None else with_ref
        seed = self.train_cfg.seed if seed is None else seed
        self.model = self._build(seed, self.value_head)
        if with_ref and not self.value_head:
            # the reference policy starts as a frozen copy of the initial weights
            self.ref_model = self._build(seed, False, recompute="none")
            for p in self.ref_model.parameters():
                p.requires_grad_(False)
            self.ref_model.eval()
        if self.policy_cfg.lora.enabled:
            self.adapters = apply_lora(self.model, self.policy_cfg.lora, seed)
            if self.policy_cfg.lora.verify_weight_consistency:
                assert verify_lora_weight_consistency(self.adapters, ps.get_tensor_model_parallel_group()), \
                    "LoRA replicated halves differ across the TP group"
        self._apply_freeze()
        self._apply_precision()
        self._maybe_enable_fused_tp()
        self._setup_dynamic_cp()
        if not self.policy_cfg.without_optim:
            oc = self.opt_cfg
            self.ddp = DistributedDataParallel(self.model, oc.grad_reduce_in_fp32, oc.bucket_size,
                                               oc.use_distributed_optimizer, oc.overlap_grad_reduce)
            self.optimizer = DistributedOptimizer(self.ddp, oc, self.total_steps)
        return self.model, self.optimizer

    def _setup_dynamic_cp(self):
        """``dist_config.dynamic_context_parallel``: the data-parallel ranks form a pool; every step each sequence is
        given a block of 1, 2, 4, ... pool ranks by its length (``max_seqlen_per_dp_cp_rank`` tokens per rank), the
        samples travel to their blocks in one byte all-to-all, and results travel back
        (gpatch_v4/extended_model/llm.py:1056-1430, utils/dynamic_cp_utils.py:1109,1471,1898).  Collective: builds one
        process group per aligned power-of-two block of the pool."""
        d = self.policy_cfg.dist_config
        if not d.dynamic_context_parallel or not dist.is_initialized():
            return
        pool = ps.get_data_parallel_group(with_context_parallel=True)
        if pool is None or dist.get_world_size(pool) <= 1:
            return
        assert ps.get_context_parallel_world_size() == 1, \
            "dynamic context parallelism sizes its own groups: set context_parallel_size to 1"
        assert ps.get_pipeline_model_parallel_world_size() == 1 and not self.model_cfg.is_moe, \
            "dynamic context parallelism is built for dense models without pipeline stages"
        from ..parallel.dynamic_cp import build_block_groups
        self._dcp = {"pool": pool, "groups": build_block_groups(pool)}

    def _dynamic_cp_plan(self, samples, forward_only: bool):
        """-> (this rank's share of the rerouted samples, micro-batches over them).  Micro-batches are ordered by
        (micro-step, block size descending): blocks are aligned power-of-two ranges, so every rank meets the groups it
        belongs to in the same order."""
        from ..parallel import dynamic_cp as D
        d = self.policy_cfg.dist_config
        pool = self._dcp["pool"]
        budget = (d.max_seqlen_per_dp_cp_rank_fwd_only if forward_only else None) or d.max_seqlen_per_dp_cp_rank
        lens, offsets = D.gather_lengths(samples, pool)
        plan = D.schedule(lens, dist.get_world_size(pool), budget, d.min_dynamic_context_parallel_size)
        steps = D.reroute_samples(list(samples), plan, offsets, pool)
        flat, batches = [], []
        for st in steps:
            by_block: Dict[tuple, list] = {}
            for smp in st:
                by_block.setdefault(tuple(smp["_block"]), []).append(smp)
            for blk in sorted(by_block, key=lambda b: (-b[1], b[0])):
                b = CPBatch(range(len(flat), len(flat) + len(by_block[blk])))
                b.cp_group = self._dcp["groups"][blk] if blk[1] > 1 else None
                flat += by_block[blk]
                batches.append(b)
        return flat, batches

    def _apply_precision(self):
        """``policy.fp8`` / ``fp8_qat`` / ``fp4_qat``: the decoder's projections whose contraction length is a multiple
        of 128 switch to the block-fp8 GEMM or to quantisation-aware training (router, embedding and head stay bf16)."""
        pc = self.policy_cfg
        kind = "fp8" if pc.fp8 else ("fp8_qat" if pc.fp8_qat else ("fp4_qat" if pc.fp4_qat else None))
        self.lowp_modules = []
        if kind is None:
            return
        from ..models.gpt import ParallelLinear
        from ..models.moe import Experts
        for name, mod in self.model.named_modules():
            if isinstance(mod, ParallelLinear) and "decoder.layers" in name and mod.in_local % 128 == 0 \
                    and mod.out_local > 1:
                mod.precision = kind
                self.lowp_modules.append(name)
            elif isinstance(mod, Experts) and kind == "fp8":
                # grouped expert projections on the grouped block-fp8 GEMM (shapes that are not multiples of 128
                # stay bf16 inside grouped_linear)
                mod.precision = kind
                self.lowp_modules.append(name)

    def _maybe_enable_fused_tp(self):
        """TP > 1 on GPUs: the sequence-parallel collectives of every layer run inside the GEMM kernels over NVLink
        peer memory (``GCORE_FUSED_TP=0`` keeps the NCCL twins)."""
        from ..models import gpt as gpt_mod
        if (self.model.tp_size == 1 or not self.model.sequence_parallel or self.device.type != "cuda"
                or self.backend != "native" or os.environ.get("GCORE_FUSED_TP", "1") == "0"
                or self.policy_cfg.lora.enabled or getattr(self, "lowp_modules", None)):
            return
        from ..parallel.symm import get_fused_tp
        tp = self.model.tp_size
        mb_tokens = self.policy_cfg.dynamic_mbs_target_seqlen or self.train_cfg.seq_length * self.train_cfg.train_mbs
        rows = ((mb_tokens + 2 * self.train_cfg.seq_length) // tp + 127) // 128 * 128
        gpt_mod.FUSED_TP["ftp"] = get_fused_tp(ps.get_tensor_model_parallel_group(), rows, self.model_cfg.hidden_size)
        self.fused_tp_rows = rows

    def _apply_freeze(self):
        import re
        t = self.train_cfg
        named = {"freeze_moe_router": r"\.router\.", "freeze_moe_shared_experts": r"\.shared_expert(s|_gate)\.",
                 "freeze_vit": r"^vision\.(?!merge_fc)", "freeze_projector": r"^vision\.merge_fc",
                 "freeze_llm": r"^(?!vision\.)"}
        flags = [pat for k, pat in named.items() if getattr(t, k, False)]
        for pat in flags + list(self.policy_cfg.freeze_patterns):
            for n, p in self.model.named_parameters():
                if re.search(pat, n):
                    p.requires_grad_(False)
        for pat in self.policy_cfg.unfreeze_patterns:
            for n, p in self.model.named_parameters():
                if re.search(pat, n):
                    p.requires_grad_(True)

    def set_model_train(self):
        self.model.train()

    def set_model_eval(self):
        self.model.eval()

    # ------------------------------------------------------------------ forward helpers
    def _hidden(self, model: GPTModel, mb: PackedBatch):
        kw = {"vision": mb.vision} if (mb.vision is not None and hasattr(model, "vision")) else {}
        return model(mb.tokens, mb.position_ids, mb.cp_ctx if mb.cp_ctx is not None else mb.cu_seqlens, mb.max_seqlen,
                     **kw)

    def _cp_group(self):
        return ps.get_context_parallel_group() if ps.get_context_parallel_world_size() > 1 else None

    def _gather_cp(self, x: torch.Tensor) -> torch.Tensor:
        """Token-axis tensors of a context-parallel shard -> the whole packed micro-batch (forward-only results)."""
        g = self._cur_cpg if self._dcp is not None else self._cp_group()
        if g is None:
            return x
        parts = [torch.empty_like(x) for _ in range(dist.get_world_size(g))]
        dist.all_gather(parts, x.contiguous(), group=g)
        return torch.cat(parts, dim=0)

    def _for_each_microbatch(self, model: GPTModel, samples, batches, keys, step_fn, forward_only: bool = False):
        """Drives ``step_fn(mb, hidden, aux)`` over the micro-batches ``batches`` (lists of sample indices).  In
        training mode ``step_fn`` returns the micro-batch loss, which is back-propagated here; in forward-only mode
        its return values are collected.  With pipeline parallelism the micro-batches run through the 1F1B schedule
        and ``step_fn`` executes on the last stage only (other stages get an empty result list)."""
        pp = ps.get_pipeline_model_parallel_world_size()
        if pp == 1:
            out = []
            for idx in batches:
                mb = self._pack(samples, idx, keys)
                hidden, aux = self._hidden(model, mb)
                r = step_fn(mb, hidden, aux)
                if forward_only:
                    out.append(r)
                else:
                    r.backward()
            return out
        from ..parallel.pp import PipelineComm, forward_backward_1f1b, forward_backward_interleaved
        comm = PipelineComm(ps.get_pipeline_model_parallel_group(), ps.get_pipeline_backward_group(),
                            *ps.get_pipeline_wrap_groups())
        n_chunks = len(getattr(model, "chunk_bounds", [0]))
        packed: Dict[int, PackedBatch] = {}

        def get(i):
            if i not in packed:
                packed[i] = self._pack(samples, batches[i], keys)
            return packed[i]

        aux_scale = self._aux_scale(len(batches))

        def forward_step(i, hidden_in, chunk=None):
            mb = get(i)
            out, aux = model(mb.tokens, mb.position_ids, mb.cp_ctx if mb.cp_ctx is not None else mb.cu_seqlens,
                             mb.max_seqlen, hidden_in=hidden_in, chunk=chunk)
            ends_here = ps.is_pipeline_last_stage() and (chunk is None or chunk == n_chunks - 1)
            if aux is not None and not ends_here:
                # a stage (or model chunk) that does not evaluate the loss back-propagates its own auxiliary loss with
                # a unit gradient: give it the weight the loss-side adds it with
                aux = aux * aux_scale
            return out, aux

        def loss_step(i, hidden, aux):
            r = step_fn(get(i), hidden, aux)
            if forward_only:
                packed.pop(i, None)
            return r

        def act_shape(i):
            mb = get(i)
            t_local = mb.tokens.numel() // (ps.get_tensor_model_parallel_world_size() if model.sequence_parallel else 1)
            dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[self.model_cfg.dtype]
            return (t_local, self.model_cfg.hidden_size), dt, self.device

        if n_chunks > 1:
            return forward_backward_interleaved(comm, len(batches), n_chunks,
                                                lambda i, v, x: forward_step(i, x, v), loss_step, act_shape,
                                                forward_only)
        return forward_backward_1f1b(comm, len(batches), forward_step, loss_step, act_shape, forward_only)

    def _from_last_stage(self, t, shape, dtype):
        """Results computed at the end of the pipeline, made available on every stage."""
        if ps.get_pipeline_model_parallel_world_size() == 1:
            return t
        from ..parallel.pp import broadcast_from_last_stage
        return broadcast_from_last_stage(t, shape, dtype, self.device, ps.get_pipeline_model_parallel_group())

    def _logprob_entropy(self, model: GPTModel, hidden, targets, want_entropy=True, mask=None):
        """Log-prob of ``targets`` (and entropy) per position.  With ``mask`` (and ``policy.ce_token_compaction``) only
        the positions inside the loss mask go through the vocabulary projection - prompt and padding positions never
        contribute to a loss or a metric - and the other positions read 0 (the reference's CE token compaction)."""
        w = model.output_weight()
        tp_group = ps.get_tensor_model_parallel_group() if model.tp_size > 1 else None
        mg = getattr(w, "main_grad", None) if (w.requires_grad and torch.is_grad_enabled()) else None
        T = hidden.shape[0]
        if mask is not None and getattr(self.policy_cfg, "ce_token_compaction", False) and mask.numel() == T:
            idx = torch.nonzero(mask > 0).flatten()
            n = int(idx.numel())
            if 0 < n <= (T * 7) // 8:   # a sparse enough mask pays for the gather
                lp_c, ent_c = linear_logprob_entropy(hidden.index_select(0, idx), w, targets.index_select(0, idx),
                                                     self.temperature, tp_group, model.vocab_start(), mg, want_entropy)
                lp = torch.zeros(T, dtype=lp_c.dtype, device=lp_c.device).index_copy(0, idx, lp_c)
                ent = None
                if ent_c is not None:
                    ent = torch.zeros(T, dtype=ent_c.dtype, device=ent_c.device).index_copy(0, idx, ent_c)
                return lp, ent
            # dense mask: full projection, same convention (zeros outside the mask) so results do not depend on
            # how a batch happens to be sharded or packed
            lp, ent = linear_logprob_entropy(hidden, w, targets, self.temperature, tp_group, model.vocab_start(), mg,
                                             want_entropy)
            keep = (mask > 0).to(lp.dtype)
            return lp * keep, (ent * keep if ent is not None else None)
        return linear_logprob_entropy(hidden, w, targets, self.temperature, tp_group, model.vocab_start(), mg,
                                      want_entropy)

    def _mtp_loss(self, model: GPTModel, mb: PackedBatch, hidden, per_token: bool, denom, detach_trunk: bool):
        """Scaled cross-entropy of the multi-token-prediction blocks on one micro-batch: depth k reads the trunk's
        hidden state at t and the embedding of token t + k and is scored on token t + k + 1 under the loss mask of
        that position; positions whose k-step look-ahead leaves their sequence are dropped.  Weighted like the main
        loss (same normaliser), averaged over depths and scaled by ``mtp_loss_scaling_factor``.  Returns
        ``(loss, [sum of masked nll, mask count])`` (Megatron's multi-token-prediction loss; label / mask shifting as in
        gpatch_v4/extended_model/mtp_mixin.py:44-80)."""
        cfg = self.model_cfg
        seq_ids = mb.seq_ids.long()
        halo = mb.halo if mb.cp_ctx is not None else None
        assert mb.cp_ctx is None or halo is not None, "context-parallel shard without its look-ahead positions"
        outs, aux = model.mtp_hidden(hidden.detach() if detach_trunk else hidden, mb.tokens, mb.position_ids,
                                     mb.cp_ctx if mb.cp_ctx is not None else mb.cu_seqlens, mb.max_seqlen, seq_ids,
                                     halo=halo)
        T = mb.tokens.shape[0]
        ar = torch.arange(T, device=mb.tokens.device)
        # under context parallelism the look-ahead of the last positions lives on the next rank: read it from the halo
        loss_mask = mb.loss_mask if halo is None else torch.cat([mb.loss_mask, halo["loss_mask"]])
        all_targets = mb.targets if halo is None else torch.cat([mb.targets, halo["targets"]])
        total, stat = None, torch.zeros(2, device=hidden.device)
        for k, (h, valid) in enumerate(outs, start=1):
            src = (ar + k).clamp_max(loss_mask.shape[0] - 1)
            mask = loss_mask[src] * valid.to(loss_mask.dtype)
            targets = all_targets[src]
            lp, _ = self._logprob_entropy(model, h, targets, False, mask)
            w = PL.aggregation_weights(mask, mb.seq_ids, mb.num_seqs + 1, per_token, denom)
            term = -(lp * w).sum()
            total = term if total is None else total + term
            with torch.no_grad():
                stat += torch.stack([-(lp.detach() * mask).sum(), mask.sum()])
        loss = total * (cfg.mtp_loss_scaling_factor / len(outs))
        if aux is not None:
            loss = loss + aux * self._aux_scale(1)
        return loss, stat

    def _tp_pad(self):
        return ps.get_tensor_model_parallel_world_size() if (self.model is not None and self.model.sequence_parallel) \
            else 1

    def _pad_multiple(self, cpg="static") -> int:
        pad = max(self._tp_pad(), 1)
        if self.device.type == "cuda":
            from ..models import gpt as gpt_mod
            pad = pad * (128 if gpt_mod.FUSED_TP["ftp"] is not None else 8) if pad > 1 else 8
        if isinstance(cpg, str):
            cpg = self._cp_group()
        if cpg is not None:
            pad *= dist.get_world_size(cpg)
        return pad

    def _pack(self, samples, idx, keys=()):
        cpg = idx.cp_group if isinstance(idx, CPBatch) else self._cp_group()
        pad = self._pad_multiple(cpg)
        if self._dcp is not None:
            self._cur_cpg = cpg
            PL.set_context_parallel_group(cpg)
        mb = pack_samples(samples, idx, keys, pad_to_multiple=pad, pin=self.device.type == "cuda")
        if isinstance(idx, FillerBatch):
            mb.loss_mask.zero_()
        if cpg is not None:
            from ..parallel.cp import shard_packed_batch
            PL.set_context_parallel_group(cpg)
            mb = shard_packed_batch(mb, cpg, self.device, halo=int(getattr(self.model_cfg, "mtp_num_layers", 0) or 0))
        io_counters.add_h2d(io_counters.tensor_bytes(mb.tokens, mb.position_ids, mb.cu_seqlens, mb.targets, mb.loss_mask,
                                                     mb.seq_ids, *mb.fields.values()))
        return mb.to(self.device)

    def _microbatches(self, samples, forward_only=False):
        lens = [len(s["tokens"]) for s in samples]
        pc = self.policy_cfg
        max_tok = pc.dynamic_mbs_target_seqlen
        mbs = pc.forward_only_mbs if forward_only else self.train_cfg.train_mbs
        if forward_only and getattr(pc, "dynamic_mbs_target_seqlen_fwd_only", None):
            max_tok = pc.dynamic_mbs_target_seqlen_fwd_only
        smart = pc.smart_pad_infer if forward_only else pc.smart_pad_train
        if smart and not max_tok:
            # samples of similar length share a micro-batch (gpatch_v4/core/smart_pad_helper.py:300-1044): with a fixed
            # number of samples per micro-batch this evens out the work of a micro-batch's sequences and, under
            # pipeline parallelism, the per-micro-batch activation shapes
            from ..core.dp_balancing import smart_pad_buckets
            batches, _ = smart_pad_buckets(lens, mbs or 1)
        else:
            batches = make_microbatches(lens, mbs=mbs, max_tokens=max_tok)
        return self._equalize_microbatch_count(batches, lens)

    def _equalize_microbatch_count(self, batches, lens):
        """Expert-parallel ranks are data-parallel ranks with their own samples, and every MoE layer runs one
        all-to-all per micro-batch: all of them must run the same number of micro-batches, whatever their local
        lengths pack into (the reference derives one micro-batch size from the group-max sequence length,
        gpatch_v4/training_backend/megatron_backend/mixin.py:2743-2765).  Ranks with fewer micro-batches first split
        their largest ones, then append filler micro-batches (see ``FillerBatch``)."""
        if ps.get_expert_model_parallel_world_size() <= 1 or not dist.is_initialized():
            return batches
        g = ps.get_data_parallel_group(with_context_parallel=True)
        if g is None or dist.get_world_size(g) <= 1:
            return batches
        t = torch.tensor([len(batches)], dtype=torch.int64,
                         device=self.device if dist.get_backend(g) == "nccl" else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=g)
        want = int(t.item())
        batches = [list(b) for b in batches]
        while len(batches) < want:
            k = max(range(len(batches)), key=lambda i: len(batches[i])) if batches else -1
            if k >= 0 and len(batches[k]) > 1:
                b = batches.pop(k)
                batches += [b[:len(b) // 2], b[len(b) // 2:]]
            else:
                shortest = min(range(len(lens)), key=lambda i: lens[i])
                batches.append(FillerBatch([shortest]))
        return batches

    # ------------------------------------------------------------------ log-probs (forward only)
    @torch.no_grad()
    def compute_log_probs(self, samples: Sequence[dict], use_ref: bool = False, with_entropy: bool = True,
                          out_key: Optional[str] = None):
        """Writes ``logprobs`` (or ``ref_logprobs``) and ``prev_per_token_entropies`` (fp32 CPU tensors of length
        S-1... stored at length S with a trailing 0) into every sample."""
        model = self.ref_model if use_ref else self.model
        assert model is not None
        was_training = model.training
        model.eval()
        key = out_key or ("ref_logprobs" if use_ref else "logprobs")
        originals = None
        if self._dcp is not None:
            originals = samples
            samples, dcp_batches = self._dynamic_cp_plan(samples, forward_only=True)
        with backend_scope(self.backend):
            batches = dcp_batches if originals is not None else self._microbatches(samples, forward_only=True)

            def step(mb, hidden, aux):
                lp, ent = self._logprob_entropy(model, hidden, mb.targets, with_entropy, mb.loss_mask)
                return self._gather_cp(lp.float()), self._gather_cp(ent.float()) if ent is not None else None

            results = self._for_each_microbatch(model, samples, batches, (), step, forward_only=True)
            for bi, idx in enumerate(batches):
                if isinstance(idx, FillerBatch):
                    continue
                lens = [len(samples[i]["tokens"]) for i in idx]
                total = sum(lens)
                pad_mult = self._pad_multiple(idx.cp_group if isinstance(idx, CPBatch) else "static")
                total_padded = (total + pad_mult - 1) // pad_mult * pad_mult
                lp, ent = results[bi] if results else (None, None)
                lp = self._from_last_stage(lp, (total_padded,), torch.float32)
                if with_entropy and not use_ref:
                    ent = self._from_last_stage(ent, (total_padded,), torch.float32)
                lp_c = lp.cpu()
                ent_c = ent.cpu() if (with_entropy and not use_ref and ent is not None) else None
                io_counters.add_d2h(io_counters.tensor_bytes(lp_c) + (io_counters.tensor_bytes(ent_c) if ent_c is not None
                                                                      else 0))
                o = 0
                for i, ln in zip(idx, lens):
                    samples[i][key] = lp_c[o:o + ln].clone()
                    if ent_c is not None:
                        samples[i]["prev_per_token_entropies"] = ent_c[o:o + ln].clone()
                    o += ln
        if originals is not None:
            from ..parallel.dynamic_cp import reverse_reroute
            back = reverse_reroute(samples, len(originals), self._dcp["pool"], keys=(key, "prev_per_token_entropies"))
            for smp, res in zip(originals, back):
                smp.update(res)
            samples = originals
        if was_training:
            model.train()
        return samples

    @torch.no_grad()
    def compute_values(self, samples: Sequence[dict]):
        assert self.value_head
        self.model.eval()
        with backend_scope(self.backend):
            batches = self._microbatches(samples, forward_only=True)
            results = self._for_each_microbatch(self.model, samples, batches, (),
                                                lambda mb, v, aux: self._gather_cp(v.float()), forward_only=True)
            for bi, idx in enumerate(batches):
                if isinstance(idx, FillerBatch):
                    continue
                lens = [len(samples[i]["tokens"]) for i in idx]
                pad_mult = self._pad_multiple("static")
                total_padded = (sum(lens) + pad_mult - 1) // pad_mult * pad_mult
                # with pipeline stages the last one holds the values: every stage receives them
                v = self._from_last_stage(results[bi] if results else None, (total_padded,), torch.float32)
                vc = v.cpu()
                o = 0
                for i, ln in zip(idx, lens):
                    samples[i]["values"] = vc[o:o + ln].clone()
                    o += ln
        return samples

    # ------------------------------------------------------------------ shared step machinery
    def _global_counts(self, samples, per_token: bool, sqrt_lengths: bool = False) -> float:
        if sqrt_lengths:   # square-averaging normaliser: sum over sequences of sqrt(answer tokens)
            n = sum(float(torch.as_tensor(s["mask"] if "mask" in s else s["loss_mask"]).sum()) ** 0.5 for s in samples)
        elif per_token:
            n = sum(float(torch.as_tensor(s["mask"] if "mask" in s else s["loss_mask"]).sum()) for s in samples)
        else:
            n = float(len(samples))
        n /= ps.get_context_parallel_world_size()  # context-parallel ranks hold the same samples
        t = torch.tensor([n], dtype=torch.float64)
        g = ps.get_data_parallel_group(with_context_parallel=True)
        if g is not None and dist.get_world_size(g) > 1:
            tt = t.float().to(self.device) if dist.get_backend(g) == "nccl" else t.float()
            dist.all_reduce(tt, group=g)
            n = float(tt.item())
        return max(n, 1.0)

    def _aux_scale(self, n_microbatches: int) -> float:
        """Weight of one micro-batch's MoE auxiliary (load-balance / z) loss.  Gradients are *summed* over the
        micro-batches and over data-parallel ranks (``_finish_step``), so the auxiliary term is divided by both counts:
        the effective ``moe_aux_loss_coef`` is then the configured one whatever the parallel layout or the packing
        (Megatron scales by 1 / num_microbatches and averages over data parallel)."""
        dp = ps.get_data_parallel_world_size(with_context_parallel=True)
        # under sequence parallelism every TP rank evaluates the term on its own token shard and the router gradients
        # of the ranks are summed: each rank's term is one of TP equal shares
        return 1.0 / (max(n_microbatches, 1) * max(dp, 1) * max(self._tp_pad(), 1))

    def _finish_step(self, lr=None):
        dp = ps.get_data_parallel_world_size(with_context_parallel=True)
        # micro-batch losses are already normalised by global counts: sum (not average) over data parallel ranks
        self.ddp.finish_grad_sync(extra_scale=float(dp))
        lr = self.optimizer.step(lr)
        self.step += 1
        self.router_bias_violation = None
        t = self.train_cfg
        if not getattr(t, "freeze_router_correction_bias", True) and getattr(self.model_cfg, "moe_router_bias", False):
            from ..models.moe import update_router_bias
            groups = [ps.get_data_parallel_group(with_context_parallel=True)]
            if ps.get_tensor_model_parallel_world_size() > 1:
                groups.append(ps.get_tensor_model_parallel_group())
            self.router_bias_violation = update_router_bias(self.model, t.router_correction_bias_update_speed,
                                                            t.router_correction_bias_use_abs_update, groups)
        return lr, float(self.optimizer.last_grad_norm.item())

    def _reduce_metrics(self, acc: Dict[str, torch.Tensor]) -> Dict[str, float]:
        """``[sum, count]`` pairs become ratios after a sum over DP; scalars are averaged."""
        pp = ps.get_pipeline_model_parallel_world_size()
        if pp > 1:
            # only the last stage evaluated the loss: it tells the others which metrics exist
            box = [sorted(acc) if ps.is_pipeline_last_stage() else None]
            g_pp = ps.get_pipeline_model_parallel_group()
            dist.broadcast_object_list(box, src=dist.get_process_group_ranks(g_pp)[-1], group=g_pp)
            for k in box[0]:
                if k not in acc:
                    acc[k] = torch.zeros(2, device=self.device)
        if not acc:
            return {}
        keys = sorted(acc)
        flat = torch.stack([acc[k].reshape(-1)[:2] if acc[k].numel() >= 2 else
                            torch.stack([acc[k].reshape(()), acc[k].new_tensor(1.0)]) for k in keys]).float()
        g = ps.get_data_parallel_group(with_context_parallel=True)
        if g is not None and dist.get_world_size(g) > 1:
            dist.all_reduce(flat, group=g)
        if ps.get_pipeline_model_parallel_world_size() > 1:
            if not ps.is_pipeline_last_stage():
                flat.zero_()  # only the last stage evaluates the loss
            dist.all_reduce(flat, group=ps.get_pipeline_model_parallel_group())
        flat = flat.cpu()
        io_counters.add_d2h(io_counters.tensor_bytes(flat))
        return {k: float(flat[i, 0] / flat[i, 1].clamp_min(1e-12)) for i, k in enumerate(keys)}

    # ------------------------------------------------------------------ SFT
    def finetune_step(self, samples: Sequence[dict]) -> Dict[str, float]:
        """One optimizer step of masked next-token cross-entropy over ``samples`` (this rank's share of the global
        batch).  Loss = sum(mask * nll) / global mask count (gpatch_v4/training_backend/loss_factory.py:2250-2309)."""
        per_token = self.train_cfg.per_token_loss
        self.model.train()
        self.ddp.zero_grad_buffer()
        for s in samples:
            if "mask" not in s and "loss_mask" not in s:
                from ..core.packing import response_mask
                s["mask"] = response_mask(int(s.get("prompt_length", 0)), len(s["tokens"]))
        square_avg = getattr(self.train_cfg, "loss_func", "cross_entropy") == "square_averaging_cross_entropy"
        denom = self._global_counts(samples, per_token, sqrt_lengths=square_avg)
        acc = {"lm_loss": torch.zeros(2, device=self.device)}
        with backend_scope(self.backend):
            if self._dcp is not None:
                assert not square_avg, "square-averaging weights need whole sequences on a rank (no dynamic CP)"
                samples, batches = self._dynamic_cp_plan(samples, forward_only=False)
            else:
                batches = self._microbatches(samples)
            aux_scale = self._aux_scale(len(batches))

            def step(mb, hidden, aux):
                lp, _ = self._logprob_entropy(self.model, hidden, mb.targets, False, mb.loss_mask)
                if square_avg:
                    assert mb.cp_ctx is None, "square-averaging weights need whole sequences on a rank"
                    w = PL.square_averaging_weights(mb.loss_mask, mb.seq_ids, mb.num_seqs + 1, denom)
                else:
                    w = PL.aggregation_weights(mb.loss_mask, mb.seq_ids, mb.num_seqs + 1, per_token, denom)
                loss = -(lp * w).sum()
                if aux is not None:
                    loss = loss + aux * aux_scale
                with torch.no_grad():
                    acc["lm_loss"] += torch.stack([-(lp.detach() * mb.loss_mask).sum(), mb.loss_mask.sum()])
                if hasattr(self.model, "mtp"):
                    ml, st = self._mtp_loss(self.model, mb, hidden, per_token, denom, detach_trunk=False)
                    loss = loss + ml
                    acc.setdefault("mtp_loss", torch.zeros(2, device=self.device)).add_(st)
                return loss

            self._for_each_microbatch(self.model, samples, batches, (), step)
            lr, gn = self._finish_step()
        out = self._reduce_metrics(acc)
        out.update(lr=lr, grad_norm=gn)
        if self.router_bias_violation is not None:
            out["moe/max_violation"], out["moe/mean_violation"] = self.router_bias_violation
        return out

    pretrain_step = finetune_step

    # ------------------------------------------------------------------ RL actor
    def rl_train_actor(self, samples: Sequence[dict]) -> Dict[str, float]:
        """One policy update over ``samples`` (each holds tokens, mask, advantages, logprobs, ref_logprobs and
        optionally rollout_log_probs).  Mirrors ``_update_policy`` (megatron_backend/mixin.py:2689-2912)."""
        cfg = self.ppo_cfg
        per_token = cfg.per_token_loss
        self.model.train()
        self.ddp.zero_grad_buffer()
        denom = self._global_counts(samples, per_token)
        keys = ["advantages"]
        has_old = not cfg.skip_prev_logps and all("logprobs" in s for s in samples)
        has_ref = cfg.grpo_kl_loss_beta != 0 and all("ref_logprobs" in s for s in samples)
        has_roll = cfg.offpolicy_correction != "none" and all("rollout_log_probs" in s for s in samples)
        if has_old:
            keys.append("logprobs")
        if has_ref:
            keys.append("ref_logprobs")
        if has_roll or cfg.loss_func == "vespo":
            keys.append("rollout_log_probs")
        want_ent = cfg.ppo_entropy_bonus != 0 or cfg.loss_func == "steer"
        has_old_ent = False
        if cfg.loss_func == "steer":
            # STEER weights tokens by the entropy of the policy that generated the batch, not the current one
            # (gpatch_v4/training_backend/loss/ppo_loss.py:387,409-416)
            assert not cfg.skip_prev_logps, "the steer loss needs the previous-policy pass (skip_prev_logps must be off)"
            has_old_ent = all("prev_per_token_entropies" in s for s in samples)
            if has_old_ent:
                keys.append("prev_per_token_entropies")
        fast = (cfg.loss_func == "grpo" and not has_roll and not want_ent and cfg.kl_estimator == "k3"
                and cfg.loss_func_py_path is None and not cfg.entropy_regularization_type)
        loss_fn = None if fast else self._resolve_loss()
        acc: Dict[str, torch.Tensor] = {}
        online_mtp = bool(getattr(self.train_cfg, "online_mtp_sft", False)) and hasattr(self.model, "mtp")

        def add(k, v):
            acc[k] = acc[k] + v if k in acc else v.clone()

        for s in samples:
            s.setdefault("loss_mask", s["mask"])
        with backend_scope(self.backend):
            def step(mb, hidden, aux):
                lp, ent = self._logprob_entropy(self.model, hidden, mb.targets, want_ent, mb.loss_mask)
                f = mb.fields
                w = PL.aggregation_weights(mb.loss_mask, mb.seq_ids, mb.num_seqs + 1, per_token, denom)
                old = f.get("logprobs") if has_old else None
                ref = f.get("ref_logprobs") if has_ref else None
                if fast:
                    loss, st = fused_grpo_loss(lp, old, ref, f["advantages"], w, clip_low=cfg.clip_low,
                                               clip_high=cfg.clip_high, dual_clip_c=cfg.ppo_dual_clip_ratio_c or 0.0,
                                               kl_beta=cfg.grpo_kl_loss_beta if has_ref else 0.0,
                                               ratio_clamp=cfg.ppo_logps_ratio_clamp or 0.0,
                                               kl_clamp=cfg.ppo_clamp_kl_val or 0.0)
                    cnt = mb.loss_mask.sum() / max(denom, 1.0) if per_token else st[2]
                    add("ppo-metrics/pg_loss", torch.stack([st[0], st[2]]))
                    add("ppo-metrics/kl_to_ref", torch.stack([st[1], st[2]]))
                    add("ppo-metrics/clipfrac", torch.stack([st[3], st[2]]))
                    add("ppo-metrics/ratio", torch.stack([st[4], st[2]]))
                    add("ppo-metrics/approx_kl", torch.stack([st[5], st[2]]))
                else:
                    li = PL.LossInput(lp, old, ref, f.get("rollout_log_probs"), f["advantages"], mb.loss_mask,
                                      mb.seq_ids, mb.num_seqs + 1, ent,
                                      f.get("prev_per_token_entropies") if has_old_ent else None)
                    lo = loss_fn(cfg, li)
                    tl = lo.token_loss
                    if has_roll and cfg.loss_func != "vespo":
                        cw, cm = PL.offpolicy_correction(cfg, old if old is not None else lp.detach(),
                                                         f["rollout_log_probs"], mb.loss_mask, mb.seq_ids,
                                                         mb.num_seqs + 1)
                        tl = tl * cw
                        for k, v in cm.items():
                            add(k, v)
                    if has_ref:
                        kl = PL.kl_penalty(lp, ref, cfg.kl_estimator, cfg.ppo_clamp_kl_val)
                        tl = tl + cfg.grpo_kl_loss_beta * kl
                        add("ppo-metrics/kl_to_ref", torch.stack([(kl.detach() * w).sum(), w.sum()]))
                    if want_ent:
                        tl = tl - cfg.ppo_entropy_bonus * ent
                    loss = (tl * w).sum()
                    add("ppo-metrics/pg_loss", torch.stack([(lo.token_loss.detach() * w).sum(), w.sum()]))
                    add("ppo-metrics/ratio", torch.stack([(lo.ratios * w).sum(), w.sum()]))
                    for k, v in lo.metrics.items():
                        add("ppo-metrics/" + k, v)
                if want_ent or not fast:
                    if ent is not None:
                        add("policy/entropy", torch.stack([(ent.detach() * mb.loss_mask).sum(), mb.loss_mask.sum()]))
                if aux is not None:
                    loss = loss + aux * aux_scale
                if online_mtp:
                    ml, st = self._mtp_loss(self.model, mb, hidden, per_token, denom, detach_trunk=True)
                    loss = loss + ml
                    add("ppo-metrics/mtp_loss", st)
                return loss

            if self._dcp is not None:
                samples, batches = self._dynamic_cp_plan(samples, forward_only=False)
            else:
                batches = self._microbatches(samples)
            aux_scale = self._aux_scale(len(batches))
            self._for_each_microbatch(self.model, samples, batches, keys, step)
            lr, gn = self._finish_step()
        out = self._reduce_metrics(acc)
        out.update({"policy/lr": lr, "policy/grad_norm": gn})
        if self.router_bias_violation is not None:
            out["moe/max_violation"], out["moe/mean_violation"] = self.router_bias_violation
        return out

    def _resolve_loss(self):
        cfg = self.ppo_cfg
        if cfg.loss_func_py_path:
            from ..configs.base import import_from_path
            return import_from_path(cfg.loss_func_py_path, cfg.loss_func_fn_name or "loss_func")
        if cfg.entropy_regularization_type:
            return PL.get_loss(cfg.entropy_regularization_type.replace("-", "_"))
        return PL.get_loss(cfg.loss_func)

    # ------------------------------------------------------------------ critic
    def rl_train_value(self, samples: Sequence[dict]) -> Dict[str, float]:
        assert self.value_head
        cfg = self.ppo_cfg
        self.model.train()
        self.ddp.zero_grad_buffer()
        denom = self._global_counts(samples, True)
        acc = {"value/loss": torch.zeros(2, device=self.device)}
        for s in samples:
            s.setdefault("loss_mask", s["mask"])
        with backend_scope(self.backend):
            def step(mb, v, aux):
                w = mb.loss_mask / denom
                loss = PL.value_loss(v, mb.fields["values"], mb.fields["returns"], w, cfg.ppo_value_clip)
                acc["value/loss"] += torch.stack([loss.detach() * denom, mb.loss_mask.sum()])
                return loss

            # through the micro-batch driver, so that a critic split over pipeline stages runs the same schedule as
            # the policy
            self._for_each_microbatch(self.model, samples, self._microbatches(samples), ["returns", "values"], step)
            lr, gn = self._finish_step()
        out = self._reduce_metrics(acc)
        out.update({"value/lr": lr, "value/grad_norm": gn})
        return out

    # ------------------------------------------------------------------ memory time-sharing
    def _ref_swap(self):
        if self.ref_model is None:
            return None
        if getattr(self, "_ref_swapper", None) is None:
            from .swap import ModuleSwap
            self._ref_swapper = ModuleSwap(self.ref_model, frozen=True)
        return self._ref_swapper

    def offload_ref_model(self):
        """Frees the frozen reference policy's device memory (its pinned host image is written once)."""
        sw = self._ref_swap()
        if sw is not None:
            sw.offload()

    def prefetch_ref_model(self):
        """Starts bringing the reference policy back on a side stream (hidden under whatever runs next)."""
        sw = self._ref_swap()
        if sw is not None:
            sw.prefetch()

    def onload_ref_model(self):
        sw = self._ref_swap()
        if sw is not None:
            sw.onload()

    def offload_model(self):
        """Moves the trainable model's flat parameter buffers to pinned host memory (buffers that are mapped on
        data-parallel peers stay: their addresses are part of the peers' kernels' arguments)."""
        from .swap import BufferSwap
        if getattr(self, "_model_swaps", None) is None:
            self._model_swaps = []
            for buf in (self.ddp.buffers if self.ddp is not None else []):
                if buf.peer:
                    continue

                shapes = {id(p): (tuple(p.shape), p.numel()) for p in buf.params}

                def rebind(t, buf=buf, shapes=shapes):
                    for p in buf.params:
                        o = buf.offsets[id(p)]
                        shp, n = shapes[id(p)]
                        p.data = t[o:o + n].view(shp) if t is not None else \
                            torch.empty(0, dtype=p.dtype, device=p.device)

                def set_buffer(t, buf=buf):
                    buf.param_data = t

                self._model_swaps.append(BufferSwap(lambda buf=buf: buf.param_data, set_buffer, rebind))
        for sw in self._model_swaps:
            sw.offload()

    def onload_model(self):
        for sw in getattr(self, "_model_swaps", None) or []:
            sw.onload()

    def offload_process_groups(self):
        """Releases the model-parallel communicators for the duration of a rollout (not with peer-memory buffers: those
        are rendezvoused over their group once and stay mapped on the peers)."""
        assert not any(b.peer for b in (self.ddp.buffers if self.ddp is not None else [])), \
            "communicators that back peer-memory buffers cannot be released: set GCORE_FUSED_DP=0"
        return ps.offload_process_groups()

    def reload_process_groups(self):
        n = ps.reload_process_groups(self.policy_cfg.dist_config.torch_dist_timeout_minutes)
        if n and self.ddp is not None:
            dense = ps.get_data_parallel_group(with_context_parallel=True)
            expert = ps.get_expert_data_parallel_group()
            for buf in self.ddp.buffers:   # reduction domains fetch their new communicators
                buf.group = expert if any(getattr(p, "is_expert", False) for p in buf.params) else dense
        if self._dcp is not None:
            from ..parallel.dynamic_cp import build_block_groups
            self._dcp = {"pool": ps.get_data_parallel_group(with_context_parallel=True),
                         "groups": build_block_groups(ps.get_data_parallel_group(with_context_parallel=True))}
        return n

    def offload_optimizer(self):
        if self.optimizer is not None:
            self.optimizer.offload()

    def onload_optimizer(self):
        if self.optimizer is not None:
            self.optimizer.onload()

    def release_grad_buffers(self):
        if self.ddp is not None:
            self.ddp.release_grads()
            if torch.cuda.is_available():
                torch.cuda.empty_cache()

    def allocate_grad_buffers(self):
        if self.ddp is not None:
            self.ddp.allocate_grads()

    # ------------------------------------------------------------------ weights
    def named_local_weights(self, merged_lora: bool = True):
        """(name, tensor) of this rank's parameter shards; LoRA deltas are folded into their base on the fly."""
        from ..models.gpt import ParallelLinear
        lora_of = {}
        if merged_lora:
            for n, m in self.model.named_modules():
                if (isinstance(m, ParallelLinear) or type(m).__name__ == "Router") and getattr(m, "lora", None) is not None:
                    lora_of[n + ".weight"] = m.lora
                elif type(m).__name__ == "Experts":
                    for leaf in ("fc1", "fc2"):
                        if getattr(m, "lora_" + leaf, None) is not None:
                            lora_of[f"{n}.linear_{leaf}.weight"] = getattr(m, "lora_" + leaf)
        for n, p in self.model.named_parameters():
            if getattr(p, "is_lora", False):
                continue
            if n in lora_of:
                yield n, (p.detach().float() + lora_of[n].delta_weight()).to(p.dtype)
            else:
                yield n, p.detach()

    def export_weights(self, to_hf: bool = True):
        """Generator of full (TP / EP gathered) tensors under HF names, the contract of mbridge ``export_weights``
        used for resync and safetensors export (gpatch_v4/training_backend/megatron_backend/mcore_engine.py:366-370)."""
        from ..checkpoint.layout import export_full_weights
        yield from export_full_weights(self, to_hf=to_hf)
