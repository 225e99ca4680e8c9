"""Decoder-only transformer (Llama / Qwen2 / Qwen3 / Qwen3-MoE / DeepSeek-V3 families) over packed (THD) tokens with
tensor + sequence parallelism.  Parameter names follow Megatron-Core's GPTModel (``embedding.word_embeddings``,
``decoder.layers.N.self_attention.linear_qkv`` ..., see tools/px_ckpt_conv/moe_hf_to_mlm.py:26-244 in the reference)
so torch_dist checkpoints and the HF converters address the same tensors.

Internal weight layouts differ from mcore where the kernels want it and are converted at checkpoint / resync time
(``gcore_b200/checkpoint/layout.py``):
  * ``linear_qkv.weight`` rows are ``[Q heads | K heads | V heads]`` of this TP rank (mcore interleaves per KV group);
  * ``linear_fc1.weight`` rows are ``[gate | up]`` of this TP rank.

The forward returns the final hidden states; the vocabulary projection is fused into the loss / log-prob op
(``ops.vocab.linear_logprob_entropy``) so ``[T, V]`` logits are never materialised.
"""
from __future__ import annotations

import math
import os
import re
from typing import Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..core import parallel_state as ps
from ..ops import fused
from ..ops.attention import flash_attn_qkvpacked, flash_attn_varlen
from ..ops.gemm import linear
from ..parallel import tp_ops
from ..parallel.cp import CPContext, cp_attention
from .config import ModelConfig
from .lora import LoRAAdapter


# Fused tensor-parallel communication (parallel/symm.py).  "ftp" is installed by the training engine when TP > 1 on a
# GPU; "active" is switched on per layer call when the token count fits the fused kernels.
FUSED_TP = {"ftp": None, "active": False}


def _dtype(cfg: ModelConfig):
    return {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[cfg.dtype]


class ParallelLinear(nn.Module):
    """Weight ``[out_local, in_local]``.  ``mode``: 'column' shards the output dim over TP, 'row' the input dim,
    'none' replicates.  ``main_grad`` (fp32, set by the DDP wrapper) receives the weight gradient directly from the
    wgrad GEMM epilogue."""

    def __init__(self, in_features, out_features, mode, cfg: ModelConfig, bias=False, tp_size=1, init_std=None,
                 device=None):
        super().__init__()
        self.mode = mode
        self.tp_size = tp_size
        self.in_features, self.out_features = in_features, out_features
        self.in_local = in_features // tp_size if mode == "row" else in_features
        self.out_local = out_features // tp_size if mode == "column" else out_features
        dt = _dtype(cfg)
        self.weight = nn.Parameter(torch.empty(self.out_local, self.in_local, dtype=dt, device=device))
        self.bias = nn.Parameter(torch.zeros(self.out_local, dtype=dt, device=device)) if bias else None
        self.init_std = init_std if init_std is not None else cfg.init_std
        self.weight.tp_mode = mode
        if self.bias is not None:
            self.bias.tp_mode = "column" if mode == "column" else "none"
        self.lora: Optional[LoRAAdapter] = None
        self.precision: Optional[str] = None   # None (bf16) | "fp8" | "fp8_qat" | "fp4_qat" (ops/lowp_linear.py)
        self._fp8_cache: dict = {}

    def forward(self, x):
        w = self.weight
        if self.precision is not None:
            from ..ops import lowp_linear
            mg = getattr(w, "main_grad", None) if w.requires_grad else None
            if self.precision == "fp8":
                y = lowp_linear.fp8_linear(x, w, self.bias, mg, self._fp8_cache)
            else:
                y = lowp_linear.qat_linear(x, w, self.bias, mg, self.precision)
            return y + self.lora(x) if self.lora is not None else y
        ftp = FUSED_TP["ftp"] if FUSED_TP["active"] else None
        if ftp is not None and self.lora is None and self.tp_size > 1 and self.mode in ("column", "row"):
            # sequence-parallel layer with its collective fused into the GEMM (x is the local token shard for a
            # column-parallel layer, the full token set for a row-parallel one)
            mg = getattr(w, "main_grad", None) if w.requires_grad else None
            if self.mode == "column":
                return ftp.ag_linear(x, w, self.bias, mg)
            return ftp.linear_rs(x, w, mg)
        y = linear(x, w, self.bias, getattr(w, "main_grad", None) if w.requires_grad else None)
        if self.lora is not None:
            y = y + self.lora(x)
        return y


class RMSNormWeight(nn.Module):
    def __init__(self, dim, cfg, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=_dtype(cfg), device=device))
        self.weight.tp_mode = "none"
        self.weight.sequence_parallel = True


class SelfAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, tp_size: int, device=None):
        super().__init__()
        self.cfg, self.layer_idx, self.tp = cfg, layer_idx, tp_size
        D = cfg.head_dim
        self.hq, self.hk = cfg.num_attention_heads // tp_size, max(cfg.num_kv_heads // tp_size, 1)
        assert cfg.num_attention_heads % tp_size == 0
        assert cfg.num_kv_heads % tp_size == 0, "replicated KV heads (tp > num_kv_heads) are not supported"
        self.linear_qkv = ParallelLinear(cfg.hidden_size, (cfg.num_attention_heads + 2 * cfg.num_kv_heads) * D,
                                         "column", cfg, bias=cfg.qkv_bias, tp_size=tp_size, device=device)
        self.linear_proj = ParallelLinear(cfg.num_attention_heads * D, cfg.hidden_size, "row", cfg, tp_size=tp_size,
                                          init_std=cfg.init_std / math.sqrt(2 * cfg.num_layers), device=device)
        if cfg.qk_layernorm:
            self.q_layernorm = RMSNormWeight(D, cfg, device)
            self.k_layernorm = RMSNormWeight(D, cfg, device)
            if tp_size > 1:   # one gain for all heads, but every TP rank sees only its own heads
                self.q_layernorm.weight.tp_partial_grad = True
                self.k_layernorm.weight.tp_partial_grad = True
        self.window = cfg.layer_window(layer_idx)
        if cfg.attention_sinks:
            self.sinks = nn.Parameter(torch.zeros(self.hq, dtype=torch.float32, device=device))
            self.sinks.tp_mode = "column"
        else:
            self.sinks = None

    def forward(self, x, pos, cu_seqlens, max_seqlen):
        cfg = self.cfg
        D, hq, hk = cfg.head_dim, self.hq, self.hk
        qkv = self.linear_qkv(x)  # [T, (hq + 2 hk) * D]; with fused TP comm x is the local shard and T the full count
        T = qkv.shape[0]
        scale = 1.0 / math.sqrt(D)
        if not cfg.qk_layernorm:
            qkv = fused_rope_qk(qkv.view(T, hq + 2 * hk, D), pos, hq + hk, cfg.rope_theta, cfg.rotary_dim,
                                cfg.rope_interleaved)
            if isinstance(cu_seqlens, CPContext):
                q3 = qkv.view(T, hq + 2 * hk, D)
                o = cp_attention(q3[:, :hq], q3[:, hq:hq + hk], q3[:, hq + hk:], cu_seqlens, self.window, self.sinks,
                                 scale)
            else:
                o = flash_attn_qkvpacked(qkv, hq, hk, cu_seqlens, max_seqlen, causal=True, window=self.window,
                                         sinks=self.sinks, scale=scale)
        elif isinstance(cu_seqlens, CPContext):
            q, k, v = qkv.view(T, hq + 2 * hk, D).split([hq, hk, hk], dim=1)
            q = fused.rmsnorm(q.reshape(-1, D), self.q_layernorm.weight, cfg.rms_norm_eps)[0].view(T, hq, D)
            k = fused.rmsnorm(k.reshape(-1, D), self.k_layernorm.weight, cfg.rms_norm_eps)[0].view(T, hk, D)
            q = fused.rope(q, pos, cfg.rope_theta, cfg.rotary_dim, cfg.rope_interleaved)
            k = fused.rope(k, pos, cfg.rope_theta, cfg.rotary_dim, cfg.rope_interleaved)
            o = cp_attention(q, k, v, cu_seqlens, self.window, self.sinks, scale)
        else:
            q, k, v = qkv.view(T, hq + 2 * hk, D).split([hq, hk, hk], dim=1)
            q = fused.rmsnorm(q.reshape(-1, D), self.q_layernorm.weight, cfg.rms_norm_eps)[0].view(T, hq, D)
            k = fused.rmsnorm(k.reshape(-1, D), self.k_layernorm.weight, cfg.rms_norm_eps)[0].view(T, hk, D)
            q = fused.rope(q, pos, cfg.rope_theta, cfg.rotary_dim, cfg.rope_interleaved)
            k = fused.rope(k, pos, cfg.rope_theta, cfg.rotary_dim, cfg.rope_interleaved)
            o = flash_attn_varlen(q, k, v.contiguous(), cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, causal=True,
                                  window=self.window, sinks=self.sinks, scale=scale)
        return self.linear_proj(o.reshape(T, hq * D))


class _RopeQKInplace(torch.autograd.Function):
    """Rotates the first ``nrot_heads`` heads of a packed ``[T, heads, D]`` buffer in place (the producing GEMM does
    not need its output for backward, so overwriting it is safe); backward rotates the gradient back."""

    @staticmethod
    def forward(ctx, qkv, pos, nrot_heads, theta, rot, interleaved):
        ctx.pos = pos   # position ids or (cos, sin) tables: never differentiated
        ctx.args = (nrot_heads, theta, rot, interleaved)
        fused.rope_inplace(qkv[:, :nrot_heads], pos, theta, rot, interleaved, False)
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, g):
        pos = ctx.pos
        n, theta, rot, interleaved = ctx.args
        g = g.contiguous() if not g.is_contiguous() else g
        fused.rope_inplace(g[:, :n], pos, theta, rot, interleaved, True)
        return g, None, None, None, None, None


def fused_rope_qk(qkv, pos, nrot_heads, theta, rot, interleaved):
    if qkv.requires_grad and torch.is_grad_enabled():
        return _RopeQKInplace.apply(qkv, pos, nrot_heads, theta, rot, interleaved)
    fused.rope_inplace(qkv[:, :nrot_heads], pos, theta, rot, interleaved, False)
    return qkv


class MLAttention(nn.Module):
    """Multi-head latent attention (DeepSeek-V3): low-rank q and joint kv compression, decoupled RoPE key shared by
    all heads.  Projections run on the tcgen05 GEMM; the (192 / 128)-dim attention core uses the reference path
    until the kernel grows mixed qk / v head dims."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, tp_size: int, device=None):
        super().__init__()
        self.cfg, self.tp = cfg, tp_size
        self.h = cfg.num_attention_heads // tp_size
        dq, dn, dr, dv = cfg.qk_head_dim, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        H = cfg.hidden_size
        if cfg.q_lora_rank:
            self.linear_q_down_proj = ParallelLinear(H, cfg.q_lora_rank, "none", cfg, device=device)
            self.q_layernorm = RMSNormWeight(cfg.q_lora_rank, cfg, device)
            self.linear_q_up_proj = ParallelLinear(cfg.q_lora_rank, cfg.num_attention_heads * dq, "column", cfg,
                                                   tp_size=tp_size, device=device)
        else:
            self.linear_q_proj = ParallelLinear(H, cfg.num_attention_heads * dq, "column", cfg, tp_size=tp_size,
                                                device=device)
        self.linear_kv_down_proj = ParallelLinear(H, cfg.kv_lora_rank + dr, "none", cfg, device=device)
        self.kv_layernorm = RMSNormWeight(cfg.kv_lora_rank, cfg, device)
        self.linear_kv_up_proj = ParallelLinear(cfg.kv_lora_rank, cfg.num_attention_heads * (dn + dv), "column", cfg,
                                                tp_size=tp_size, device=device)
        if tp_size > 1:
            # the down-projections (and the shared rotary key inside the kv one) are replicated while the heads behind
            # them are sharded: every TP rank sends back the part of their gradient that flows through its heads, and
            # the parts are summed over the TP group with the gradient reduction (their norm gains already are)
            for lin in (getattr(self, "linear_q_down_proj", None), self.linear_kv_down_proj):
                if lin is not None:
                    lin.weight.tp_partial_grad = True
            for nm in (getattr(self, "q_layernorm", None), self.kv_layernorm):
                if nm is not None:
                    nm.weight.tp_partial_grad = True
        self.linear_proj = ParallelLinear(cfg.num_attention_heads * dv, H, "row", cfg, tp_size=tp_size,
                                          init_std=cfg.init_std / math.sqrt(2 * cfg.num_layers), device=device)

    def project(self, x, pos):
        """Per-token projections: ``q_nope [T, h, dn]``, rotated ``q_rope [T, h, dr]``, the normalised latent
        ``c_kv [T, kv_lora]`` and the rotated shared key ``k_rope [T, dr]`` (the last two are what a decoder caches)."""
        cfg = self.cfg
        T, h = x.shape[0], self.h
        dn, dr = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim
        if cfg.q_lora_rank:
            ql = fused.rmsnorm(self.linear_q_down_proj(x), self.q_layernorm.weight, cfg.rms_norm_eps)[0]
            q = self.linear_q_up_proj(ql).view(T, h, dn + dr)
        else:
            q = self.linear_q_proj(x).view(T, h, dn + dr)
        kv = self.linear_kv_down_proj(x)
        c_kv, k_rope = kv.split([cfg.kv_lora_rank, dr], dim=-1)
        c_kv = fused.rmsnorm(c_kv.contiguous(), self.kv_layernorm.weight, cfg.rms_norm_eps)[0]
        q_nope, q_rope = q.split([dn, dr], dim=-1)
        q_rope = fused.rope(q_rope.contiguous(), pos, cfg.rope_theta, dr, cfg.rope_interleaved)
        k_rope = fused.rope(k_rope.reshape(T, 1, dr).contiguous(), pos, cfg.rope_theta, dr, cfg.rope_interleaved)
        return q_nope, q_rope, c_kv, k_rope.reshape(T, dr)

    def attend(self, q_nope, q_rope, c_kv, k_rope, cu_seqlens, max_seqlen=None):
        """Causal attention over packed sequences with the latent expanded to per-head keys and values."""
        cfg = self.cfg
        T, h = q_nope.shape[0], self.h
        dn, dr, dv = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        cu_q = cu_k = cu_seqlens
        max_q = max_k = max_seqlen
        cp_on = isinstance(cu_seqlens, CPContext)
        if cp_on:
            # context parallel: what crosses the ranks is the compressed latent and the shared rotary key
            # (kv_lora + dr numbers a token, not heads x (dn + dr + dv)); each rank expands the document prefixes its
            # queries need.  The gather's backward sums the ranks' gradient parts back onto the owning rows.
            from ..parallel.cp import gather_from_cp
            cpx = cu_seqlens
            plan = cpx.plan(0)
            cu_q, cu_k = cpx.cu_tensors(0)
            max_q, max_k = plan.max_q, plan.max_k
            lat = gather_from_cp(torch.cat([c_kv, k_rope], -1).contiguous(), cpx.group)[plan.k0:plan.k0 + plan.rows]
            c_kv, k_rope = lat[:, :cfg.kv_lora_rank].contiguous(), lat[:, cfg.kv_lora_rank:]
        Tk = c_kv.shape[0]
        kvu = self.linear_kv_up_proj(c_kv).view(Tk, h, dn + dv)
        k_nope, v = kvu.split([dn, dv], dim=-1)
        qf = torch.cat([q_nope, q_rope], -1)
        kf = torch.cat([k_nope, k_rope.reshape(Tk, 1, dr).expand(Tk, h, dr)], -1)
        from ..ops import _lib
        if (dn + dr, dv) == (192, 128) and qf.is_cuda and qf.dtype == torch.bfloat16 and not _lib.force_eager() \
                and os.environ.get("GCORE_MLA_FLASH", "1") != "0":
            # 192-wide keys / 128-wide values: the tcgen05 flash kernels' wide-key instances (forward and backward)
            # over the whole packed batch
            from ..ops.attention import flash_attn_varlen
            if max_q is None:
                max_q = max_k = int((cu_seqlens[1:] - cu_seqlens[:-1]).max())
            o = flash_attn_varlen(qf, kf, v.contiguous(), cu_q, cu_k, max_q, max_k, causal=True,
                                  scale=1.0 / math.sqrt(dn + dr))
            return o.reshape(T, h * dv)
        # pad v to the qk head dim so one attention call serves both (extra columns are zero and sliced away)
        vpad = torch.nn.functional.pad(v, (0, dn + dr - dv))
        scale = 1.0 / math.sqrt(dn + dr)
        if qf.is_cuda and qf.dtype in (torch.bfloat16, torch.float16) and not _lib.force_eager() and not cp_on:
            # other latent geometries: the library's fused attention, one sequence at a time (memory linear in the
            # sequence length)
            bounds = cu_seqlens.tolist()
            outs = []
            for a, b in zip(bounds[:-1], bounds[1:]):
                if b > a:
                    outs.append(torch.nn.functional.scaled_dot_product_attention(
                        qf[a:b].transpose(0, 1)[None], kf[a:b].transpose(0, 1)[None], vpad[a:b].transpose(0, 1)[None],
                        is_causal=True, scale=scale)[0].transpose(0, 1))
            if bounds[-1] < T:   # padding rows behind the last sequence
                outs.append(qf.new_zeros(T - bounds[-1], h, dn + dr))
            o = torch.cat(outs, 0)
        else:
            from ..ops.attention import attn_varlen_ref
            o = attn_varlen_ref(qf, kf, vpad, cu_q, cu_k, True, 0, None, scale)
        return o[..., :dv].reshape(T, h * dv)

    def forward(self, x, pos, cu_seqlens, max_seqlen):
        return self.linear_proj(self.attend(*self.project(x, pos), cu_seqlens, max_seqlen))


class MLP(nn.Module):
    def __init__(self, cfg: ModelConfig, ffn: int, tp_size: int, device=None):
        super().__init__()
        self.linear_fc1 = ParallelLinear(cfg.hidden_size, 2 * ffn, "column", cfg, tp_size=tp_size, device=device)
        self.linear_fc2 = ParallelLinear(ffn, cfg.hidden_size, "row", cfg, tp_size=tp_size,
                                         init_std=cfg.init_std / math.sqrt(2 * cfg.num_layers), device=device)

    def forward(self, x):
        return self.linear_fc2(fused.swiglu(self.linear_fc1(x)))


class TransformerLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, tp_size: int, ep_size: int, device=None):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.input_layernorm = RMSNormWeight(cfg.hidden_size, cfg, device)
        self.self_attention = (MLAttention if cfg.use_mla else SelfAttention)(cfg, layer_idx, tp_size, device)
        self.pre_mlp_layernorm = RMSNormWeight(cfg.hidden_size, cfg, device)
        if cfg.layer_is_moe(layer_idx):
            from .moe import MoELayer
            self.mlp = MoELayer(cfg, layer_idx, tp_size, ep_size, device)
        else:
            self.mlp = MLP(cfg, cfg.ffn_hidden_size, tp_size, device)
        self.is_moe = cfg.layer_is_moe(layer_idx)

    def forward(self, x, residual, pos, cu_seqlens, max_seqlen, tp_group, sp):
        cfg = self.cfg
        ftp = FUSED_TP["ftp"]
        fused_comm = (sp and ftp is not None and x.is_cuda and x.dtype == torch.bfloat16 and not cfg.use_mla
                      and x.shape[0] % 128 == 0 and x.shape[0] <= ftp.max_rows)
        if fused_comm:
            return self._forward_fused(x, residual, pos, cu_seqlens, max_seqlen)
        h, residual = fused.rmsnorm(x, self.input_layernorm.weight, cfg.rms_norm_eps, residual)
        if sp:
            h = tp_ops.gather_from_sequence_parallel(h, tp_group)
        else:
            h = tp_ops.copy_to_tensor_parallel(h, tp_group)
        a = self.self_attention(h, pos, cu_seqlens, max_seqlen)
        a = tp_ops.reduce_scatter_to_sequence_parallel(a, tp_group) if sp else \
            tp_ops.reduce_from_tensor_parallel(a, tp_group)
        h, residual = fused.rmsnorm(a, self.pre_mlp_layernorm.weight, cfg.rms_norm_eps, residual)
        aux = None
        if self.is_moe:
            # experts see the sequence-parallel token shard: every TP rank routes its own tokens (ETP = 1)
            m, aux = self.mlp(h)
            return m, residual, aux
        if sp:
            h = tp_ops.gather_from_sequence_parallel(h, tp_group)
        else:
            h = tp_ops.copy_to_tensor_parallel(h, tp_group)
        m = self.mlp(h)
        m = tp_ops.reduce_scatter_to_sequence_parallel(m, tp_group) if sp else \
            tp_ops.reduce_from_tensor_parallel(m, tp_group)
        return m, residual, aux


def _layer_forward_fused(self, x, residual, pos, cu_seqlens, max_seqlen):
    """Sequence-parallel layer whose four TP collectives run inside the GEMM kernels: the column-parallel layers
    (QKV, FC1) are all-gather -> GEMM, the row-parallel ones (proj, FC2) GEMM -> reduce-scatter."""
    cfg = self.cfg
    FUSED_TP["active"] = True
    try:
        h, residual = fused.rmsnorm(x, self.input_layernorm.weight, cfg.rms_norm_eps, residual)
        a = self.self_attention(h, pos, cu_seqlens, max_seqlen)
        h, residual = fused.rmsnorm(a, self.pre_mlp_layernorm.weight, cfg.rms_norm_eps, residual)
        if self.is_moe:
            FUSED_TP["active"] = False
            m, aux = self.mlp(h)
            return m, residual, aux
        m = self.mlp(h)
        return m, residual, None
    finally:
        FUSED_TP["active"] = False


TransformerLayer._forward_fused = _layer_forward_fused


class MTPBlock(nn.Module):
    """One depth of multi-token prediction: ``h' = layer(W [norm_e(emb(token t+k)) ; norm_h(h_t)])`` followed by its
    own final norm; the vocabulary projection is the trunk's (the multi-token-prediction layers the reference trains
    through Megatron and its online-MTP data preparation, gpatch_v4/extended_model/mtp_mixin.py:11-80)."""

    def __init__(self, cfg: ModelConfig, depth: int, tp_size: int, ep_size: int, device=None):
        super().__init__()
        self.enorm = RMSNormWeight(cfg.hidden_size, cfg, device)
        self.hnorm = RMSNormWeight(cfg.hidden_size, cfg, device)
        # replicated, applied to the sequence-parallel token shard: its gradient is summed over the TP group
        self.eh_proj = ParallelLinear(2 * cfg.hidden_size, cfg.hidden_size, "none", cfg, device=device)
        self.eh_proj.weight.sequence_parallel = True
        self.transformer_layer = TransformerLayer(cfg, cfg.num_layers + depth, tp_size, ep_size, device)
        self.final_layernorm = RMSNormWeight(cfg.hidden_size, cfg, device)


class GPTModel(nn.Module):
    """One pipeline stage worth of layers (all of them when PP = 1)."""

    def __init__(self, cfg: ModelConfig, tp_size: int = 1, ep_size: int = 1, sequence_parallel: bool = True,
                 pre_process: bool = True, post_process: bool = True, layer_range=None, recompute: str = "none",
                 device=None, value_head: bool = False):
        super().__init__()
        self.cfg = cfg
        self.tp_size, self.ep_size = tp_size, ep_size
        self.sequence_parallel = sequence_parallel and tp_size > 1
        if tp_size > 1 and not self.sequence_parallel and cfg.num_experts:
            # without the token shard every TP rank would route (and back-propagate) the same tokens through the same
            # unsplit experts (Megatron-LM makes the same demand of MoE models under tensor parallelism)
            raise ValueError("mixture-of-experts layers under tensor parallelism need sequence_parallel=True")
        self.pre_process, self.post_process = pre_process, post_process
        self.recompute = recompute
        dt = _dtype(cfg)
        self.vocab_local = _padded_vocab(cfg.vocab_size, tp_size) // tp_size
        if pre_process:
            self.embedding = nn.Module()
            self.embedding.word_embeddings = nn.Module()
            self.embedding.word_embeddings.weight = nn.Parameter(
                torch.empty(self.vocab_local, cfg.hidden_size, dtype=dt, device=device))
            self.embedding.word_embeddings.weight.tp_mode = "column"
        # one (lo, hi) range of global layer indices, or a list of them: the model chunks of an interleaved
        # (virtual) pipeline stage, run one at a time with ``forward(chunk=v)``
        if layer_range is None:
            ranges = [(0, cfg.num_layers)]
        elif isinstance(layer_range[0], (tuple, list)):
            ranges = [tuple(r) for r in layer_range]
        else:
            ranges = [tuple(layer_range)]
        self.layer_ranges = ranges
        self.layer_offset = ranges[0][0]
        self.global_layer_ids = [i for lo, hi in ranges for i in range(lo, hi)]
        self.chunk_bounds, n0 = [], 0
        for lo, hi in ranges:
            self.chunk_bounds.append((n0, n0 + hi - lo))
            n0 += hi - lo
        self.decoder = nn.Module()
        self.decoder.layers = nn.ModuleList(
            [TransformerLayer(cfg, i, tp_size, ep_size, device) for i in self.global_layer_ids])
        self.value_head = value_head
        if post_process:
            self.decoder.final_layernorm = RMSNormWeight(cfg.hidden_size, cfg, device)
            if value_head:
                # critic: hidden -> 1 (gpatch_v4/training_backend/megatron_backend/megatron_bridge.py:77-138)
                self.output_layer = ParallelLinear(cfg.hidden_size, 1, "none", cfg, device=device)
            elif not (cfg.tie_word_embeddings and pre_process):
                self.output_layer = nn.Module()
                self.output_layer.weight = nn.Parameter(
                    torch.empty(self.vocab_local, cfg.hidden_size, dtype=dt, device=device))
                self.output_layer.weight.tp_mode = "column"
        if cfg.mtp_num_layers > 0 and not value_head:
            assert pre_process and post_process and len(ranges) == 1, \
                "multi-token prediction needs the embedding and the head on one stage (pipeline size 1)"
            self.mtp = nn.Module()
            self.mtp.layers = nn.ModuleList([MTPBlock(cfg, k, tp_size, ep_size, device)
                                             for k in range(cfg.mtp_num_layers)])
        self.reset_parameters()

    # ------------------------------------------------------------------ init
    def reset_parameters(self, seed: Optional[int] = None):
        """Each parameter is drawn from its own generator keyed by (seed, parameter name, TP shard) so the values do
        not depend on construction order.  TP-sharded tensors of small models are drawn at full size and sliced, which
        makes a TP>1 model bit-identical to the TP=1 model (the CPU oracle tests rely on it)."""
        import zlib
        seed = 1234 if seed is None else seed
        tp_rank = ps.get_tensor_model_parallel_rank() if self.tp_size > 1 else 0
        for name, p in self.named_parameters():
            mod_std = self.cfg.init_std
            owner = self._owner(name)
            if isinstance(owner, ParallelLinear):
                mod_std = owner.init_std
            if name.endswith("bias") or "sinks" in name:
                with torch.no_grad():
                    p.zero_()
                continue
            if p.dim() == 1:
                with torch.no_grad():
                    p.fill_(1.0)
                continue
            mode = getattr(p, "tp_mode", "none")
            # keyed by the parameter's name in the unpartitioned model, so a pipeline stage draws the same values
            canon = self.canonical_name(name)
            key = zlib.crc32(f"0:{canon}".encode()) ^ seed
            full_numel = p.numel() * (self.tp_size if mode in ("column", "row") else 1)
            with torch.no_grad():
                if mode == "expert" and self.ep_size > 1:
                    # experts are drawn as one [E_total, ...] tensor and sliced, so EP > 1 equals the EP = 1 model
                    ep_rank = ps.get_expert_model_parallel_rank()
                    if p.numel() * self.ep_size <= (1 << 26):
                        g = torch.Generator(device="cpu").manual_seed(key & 0x7FFFFFFF)
                        full = torch.randn(p.shape[0] * self.ep_size, *p.shape[1:], generator=g) * mod_std
                        p.copy_(full[ep_rank * p.shape[0]:(ep_rank + 1) * p.shape[0]])
                    else:
                        g = torch.Generator(device=p.device).manual_seed((key + 104729 * ep_rank) & 0x7FFFFFFF)
                        p.copy_(torch.randn(p.shape, generator=g, device=p.device, dtype=torch.float32) * mod_std)
                elif self.tp_size > 1 and mode in ("column", "row") and full_numel <= (1 << 26) and p.dim() == 2:
                    g = torch.Generator(device="cpu").manual_seed(key & 0x7FFFFFFF)
                    if mode == "column":
                        full = torch.randn(p.shape[0] * self.tp_size, p.shape[1], generator=g) * mod_std
                        p.copy_(_column_shard(full, name, self, tp_rank))
                    else:
                        full = torch.randn(p.shape[0], p.shape[1] * self.tp_size, generator=g) * mod_std
                        p.copy_(full.chunk(self.tp_size, 1)[tp_rank])
                elif p.is_cuda and p.numel() > (1 << 22):
                    g = torch.Generator(device=p.device).manual_seed(
                        (key + (7919 * tp_rank if mode in ("column", "row") else 0)) & 0x7FFFFFFF)
                    p.copy_(torch.randn(p.shape, generator=g, device=p.device, dtype=torch.float32) * mod_std)
                else:
                    g = torch.Generator(device="cpu").manual_seed(
                        (key + (7919 * tp_rank if mode in ("column", "row") else 0)) & 0x7FFFFFFF)
                    p.copy_(torch.randn(p.shape, generator=g) * mod_std)

    def canonical_name(self, name: str) -> str:
        """Parameter name in the unpartitioned model (local layer position -> global layer index)."""
        ids = self.global_layer_ids
        return re.sub(r"decoder\.layers\.(\d+)\.", lambda m: f"decoder.layers.{ids[int(m.group(1))]}.", name, count=1)

    def _owner(self, pname: str):
        mod = self
        for part in pname.split(".")[:-1]:
            mod = getattr(mod, part)
        return mod

    # ------------------------------------------------------------------ forward
    def output_weight(self):
        if hasattr(self, "output_layer") and not self.value_head:
            return self.output_layer.weight
        return self.embedding.word_embeddings.weight

    def vocab_start(self):
        return self.vocab_local * (ps.get_tensor_model_parallel_rank() if self.tp_size > 1 else 0)

    def forward(self, input_ids=None, position_ids=None, cu_seqlens=None, max_seqlen=None, hidden_in=None,
                inputs_embeds=None, chunk=None, deepstack=None):
        """``input_ids`` [T] packed tokens (first stage) or ``hidden_in`` (later pipeline stages, sequence-parallel
        shard).  Returns ``(hidden, aux_loss)``: on the last stage ``hidden`` is the final-normed ``[T, H]`` (gathered
        over SP), otherwise the stage output to send downstream.  ``chunk`` selects one model chunk of an interleaved
        pipeline stage (embedding only in front of the first, final norm only behind the last); None runs them all."""
        tp_group = ps.get_tensor_model_parallel_group() if self.tp_size > 1 else None
        sp = self.sequence_parallel
        n_chunks = len(self.chunk_bounds)
        first = self.pre_process and (chunk is None or chunk == 0)
        last = self.post_process and (chunk is None or chunk == n_chunks - 1)
        l0, l1 = (0, len(self.decoder.layers)) if chunk is None else self.chunk_bounds[chunk]
        if first:
            if inputs_embeds is None:
                x = tp_ops.vocab_parallel_embedding(input_ids, self.embedding.word_embeddings.weight,
                                                    self.vocab_start(), tp_group)
            else:
                x = inputs_embeds
            if sp:
                x = tp_ops.scatter_to_sequence_parallel(x, tp_group)
        else:
            x = hidden_in
        residual = None
        aux_total = None
        if position_ids.dim() == 2:
            # [T, 3] (temporal, height, width) ids of a vision-language stream: rotary tables replace the ids
            cfg = self.cfg
            assert cfg.mrope_sections is not None, "multi-axis position ids need model_config.mrope_sections"
            pos32 = fused.mrope_tables(position_ids, cfg.rope_theta, cfg.rotary_dim or cfg.head_dim,
                                       tuple(cfg.mrope_sections), cfg.mrope_interleaved)
        else:
            pos32 = position_ids.to(torch.int32) if position_ids.dtype != torch.int32 else position_ids
        n_ckpt = getattr(self, "recompute_num_layers", None)
        for li in range(l0, l1):
            layer = self.decoder.layers[li]
            if (self.recompute == "full" and torch.is_grad_enabled() and x.requires_grad
                    and (n_ckpt is None or li < n_ckpt)):
                x, residual, aux = checkpoint(layer, x, residual, pos32, cu_seqlens, max_seqlen, tp_group, sp,
                                              use_reentrant=False)
            else:
                x, residual, aux = layer(x, residual, pos32, cu_seqlens, max_seqlen, tp_group, sp)
            if aux is not None:
                aux_total = aux if aux_total is None else aux_total + aux
            if deepstack is not None and li < len(deepstack[1]):
                # intermediate vision-tower features join the hidden state of the visual tokens behind each of the
                # first decoder layers (Qwen3-VL "deepstack")
                x = x.index_add(0, deepstack[0], deepstack[1][li].to(x.dtype))
        if not last:
            # carry the un-added residual forward as one tensor
            return (x + residual if residual is not None else x), aux_total
        h, _ = fused.rmsnorm(x, self.decoder.final_layernorm.weight, self.cfg.rms_norm_eps, residual)
        if sp:
            h = tp_ops.gather_from_sequence_parallel(h, tp_group)
        elif tp_group is not None and not self.value_head:
            # every TP rank holds the whole hidden state; the vocabulary-parallel head behind it sends back only the
            # part of the gradient that flows through its own vocabulary shard
            h = tp_ops.copy_to_tensor_parallel(h, tp_group)
        if self.value_head:
            if sp:   # the scalar head is replicated: every TP rank back-propagates the whole value loss
                h = tp_ops.replicated_consumer_of_gathered(h, tp_group)
            return self.output_layer(h).squeeze(-1).float(), aux_total
        return h, aux_total

    def mtp_hidden(self, hidden, input_ids, position_ids, cu_seqlens, max_seqlen, seq_ids, halo=None):
        """Final-normed hidden states of every prediction depth, ``[(h_k, valid_k)]``: ``h_k[t]`` predicts token
        ``t + k + 1`` (k = 1 .. depth) and ``valid_k[t]`` says whether tokens ``t + 1 .. t + k`` belong to the same
        packed sequence as ``t``.  ``hidden`` is the trunk's final-normed output (gathered over sequence parallel),
        ``seq_ids`` [T] the sequence index of every position.  On a context-parallel shard ``halo`` carries the
        ``tokens`` / ``seq_ids`` of the positions behind this rank's chunk (the look-ahead of its last positions) and
        ``cu_seqlens`` is the shard's ``CPContext``.  Returns ``([...], aux_loss)``."""
        tp_group = ps.get_tensor_model_parallel_group() if self.tp_size > 1 else None
        sp, cfg = self.sequence_parallel, self.cfg
        T = input_ids.shape[0]
        pos32 = position_ids.to(torch.int32) if position_ids.dtype != torch.int32 else position_ids
        outs, aux_total, h_prev = [], None, hidden
        ar = torch.arange(T, device=input_ids.device)
        ids_ext, seq_ext = input_ids, seq_ids
        if halo is not None:
            ids_ext = torch.cat([input_ids, halo["tokens"].to(input_ids.dtype)])
            seq_ext = torch.cat([seq_ids, halo["seq_ids"].to(seq_ids.dtype)])
        Te = ids_ext.shape[0]
        for k, blk in enumerate(self.mtp.layers, start=1):
            src = (ar + k).clamp_max(Te - 1)
            valid = (ar + k < Te) & (seq_ext[src] == seq_ids)
            e = tp_ops.vocab_parallel_embedding(ids_ext[src], self.embedding.word_embeddings.weight,
                                                self.vocab_start(), tp_group)
            hp = h_prev
            if sp:
                # the embedding rows were computed in full on every rank; the hidden state came out of a
                # sequence-parallel gather, whose backward sums the ranks' gradients: hand back this rank's share only
                e = tp_ops.scatter_to_sequence_parallel(e, tp_group)
                hp = tp_ops.slice_of_gathered(hp, tp_group)
            elif tp_group is not None and k == 1:
                # without sequence parallelism the trunk's output sums the gradients of all TP ranks, and this
                # (replicated) branch computes the same full gradient on every one of them
                hp = tp_ops.replicated_consumer_of_gathered(hp, tp_group)
            e = fused.rmsnorm(e, blk.enorm.weight, cfg.rms_norm_eps)[0]
            hp = fused.rmsnorm(hp, blk.hnorm.weight, cfg.rms_norm_eps)[0]
            x = blk.eh_proj(torch.cat([e, hp], dim=-1))
            x, residual, aux = blk.transformer_layer(x, None, pos32, cu_seqlens, max_seqlen, tp_group, sp)
            if aux is not None:
                aux_total = aux if aux_total is None else aux_total + aux
            h, _ = fused.rmsnorm(x, blk.final_layernorm.weight, cfg.rms_norm_eps, residual)
            if sp:
                h = tp_ops.gather_from_sequence_parallel(h, tp_group)
            h_prev = h
            if not sp and tp_group is not None:
                h = tp_ops.copy_to_tensor_parallel(h, tp_group)   # in front of the vocabulary-parallel head
            outs.append((h, valid))
        return outs, aux_total

    def logits(self, hidden):
        """Materialised (local-vocab) logits; only for small debugging / generation on CPU."""
        return torch.nn.functional.linear(hidden, self.output_weight())


def _padded_vocab(v: int, tp: int, multiple: int = 128) -> int:
    m = multiple * tp
    return (v + m - 1) // m * m


def padded_vocab_size(cfg: ModelConfig, tp: int) -> int:
    return _padded_vocab(cfg.vocab_size, tp)


def _column_shard(full: torch.Tensor, name: str, model: "GPTModel", tp_rank: int) -> torch.Tensor:
    """Slices this rank's rows out of a full column-parallel weight, honouring the fused layouts: QKV is
    [Q | K | V] per rank and fc1 is [gate | up] per rank."""
    tp = model.tp_size
    cfg = model.cfg
    if name.endswith("linear_qkv.weight") or name.endswith("linear_qkv.bias"):
        D = cfg.head_dim
        q, k, v = full.split([cfg.num_attention_heads * D, cfg.num_kv_heads * D, cfg.num_kv_heads * D], 0)
        return torch.cat([q.chunk(tp, 0)[tp_rank], k.chunk(tp, 0)[tp_rank], v.chunk(tp, 0)[tp_rank]], 0)
    if name.endswith("linear_fc1.weight") and "experts" not in name:
        g, u = full.chunk(2, 0)
        return torch.cat([g.chunk(tp, 0)[tp_rank], u.chunk(tp, 0)[tp_rank]], 0)
    return full.chunk(tp, 0)[tp_rank]
