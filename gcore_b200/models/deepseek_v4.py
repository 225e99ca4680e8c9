"""DeepSeek-V4-class decoder: shared-key/value multi-query attention over a sliding window plus compressed history
(compressed sparse attention with a lightning indexer, or heavily compressed attention), per-head sinks, grouped
low-rank output projection, hyper-connection residual streams, hash / top-k routed experts with a shared expert.

Behavioural model: gpatch_v4/models/deepseek_v4/modeling_deepseek_v4.py (compressors :134-286 and :605-790, indexer
:288-603, attention :844-1086, router :1410-1459, decoder layer :1494-1552).  Differences of form, not of function:
sequences are packed (``[T, ...]`` with ``cu_seqlens``) from the start instead of padded batches with a THD side path;
every layer builds, per query, the list of key rows it may read (window rows, then compressed rows) and runs ONE
gather-attention kernel over it (``ops.dsv4.sparse_mqa``), which also serves the heavily compressed variant; the
indexer scores come from ``ops.dsv4.indexer_scores`` and its training signal through ``indexer_selected_scores``.

Keys double as values (one ``head_dim`` row per token): the rotary slice of the attention output is rotated back by the
query position so that every contribution depends on relative distance only.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import dsv4 as K4
from ..ops import fused
from ..ops.gemm import linear
from .moe import Experts, build_dispatch_plan, padded_rows_bound

SLIDING, CSA, HCA = "sliding_attention", "compressed_sparse_attention", "heavily_compressed_attention"


@dataclass
class DSV4Config:
    vocab_size: int = 1024
    hidden_size: int = 256
    num_layers: int = 3
    num_attention_heads: int = 4
    head_dim: int = 64
    qk_rope_head_dim: int = 16
    q_lora_rank: int = 64
    o_groups: int = 2
    o_lora_rank: int = 32
    sliding_window: int = 16
    layer_types: Tuple[str, ...] = (SLIDING, CSA, HCA)
    compress_rate_csa: int = 4
    compress_rate_hca: int = 8
    index_n_heads: int = 4
    index_head_dim: int = 32
    index_topk: int = 8
    hc_mult: int = 2
    hc_sinkhorn_iters: int = 4
    num_experts: int = 8
    num_experts_per_tok: int = 2
    moe_intermediate_size: int = 64
    shared_intermediate_size: int = 64
    scoring_func: str = "sqrtsoftplus"   # sqrtsoftplus | sigmoid | softmax
    routed_scaling_factor: float = 1.5
    hash_layers: Tuple[int, ...] = (0,)   # layers whose experts are chosen by a hash of the token id
    rope_theta: float = 10000.0
    compress_rope_theta: float = 160000.0
    rms_norm_eps: float = 1e-6
    indexer_rotate: bool = False          # Hadamard-rotate indexer queries / keys (low-precision indexer)
    dtype: str = "float32"
    init_std: float = 0.02

    def __post_init__(self):
        self.layer_types = tuple(self.layer_types)
        assert len(self.layer_types) == self.num_layers
        assert self.qk_rope_head_dim % 2 == 0 and self.qk_rope_head_dim <= self.head_dim
        assert (self.num_attention_heads * self.head_dim) % self.o_groups == 0


class _Lin(nn.Module):
    def __init__(self, i, o, cfg: DSV4Config, std=None, device=None):
        super().__init__()
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[cfg.dtype]
        self.weight = nn.Parameter((torch.randn(o, i, device=device) * (std or cfg.init_std)).to(dt))

    def forward(self, x):
        return linear(x, self.weight, None, getattr(self.weight, "main_grad", None) if self.weight.requires_grad
                      else None)


class _Norm(nn.Module):
    def __init__(self, d, cfg: DSV4Config, device=None):
        super().__init__()
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[cfg.dtype]
        self.weight = nn.Parameter(torch.ones(d, dtype=dt, device=device))
        self.eps = cfg.rms_norm_eps

    def forward(self, x):
        return fused.rmsnorm(x.reshape(-1, x.shape[-1]), self.weight, self.eps)[0].view(x.shape)


def _unit_norm(x, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def rope_tail(x: torch.Tensor, pos: torch.Tensor, theta: float, rot: int, inverse: bool = False) -> torch.Tensor:
    """Rotates the LAST ``rot`` elements of every head of x [T, H, D] (interleaved pairs) at positions ``pos`` [T]."""
    D = x.shape[-1]
    head, tail = x[..., :D - rot], x[..., D - rot:]
    out = fused.rope_ref(tail, pos, theta, rot, interleaved=True, backward=inverse)
    return torch.cat([head, out], -1)


# ---------------------------------------------------------------------------------------------------- compressors
def _window_layout(cu: Sequence[int], m: int):
    """Closed windows of ``m`` tokens inside every sequence of the packed stream.
    -> (token index of each window's first token [W], sequence id per window [W], position of the window inside its
    sequence (first token's position) [W], first window id of every sequence [n_seq + 1])."""
    starts, seg, pos, first = [], [], [], [0]
    for s in range(len(cu) - 1):
        n = (cu[s + 1] - cu[s]) // m
        for w in range(n):
            starts.append(cu[s] + w * m)
            seg.append(s)
            pos.append(w * m)
        first.append(first[-1] + n)
    return starts, seg, pos, first


class HCACompressor(nn.Module):
    """Every closed window of ``m`` tokens becomes one entry: softmax-gated (over the window, per channel, with a
    learned position bias) sum of the tokens' projections, normalised, rotated at the window's first position."""

    def __init__(self, cfg: DSV4Config, device=None):
        super().__init__()
        self.cfg, self.m = cfg, cfg.compress_rate_hca
        self.kv_proj = _Lin(cfg.hidden_size, cfg.head_dim, cfg, device=device)
        self.gate_proj = _Lin(cfg.hidden_size, cfg.head_dim, cfg, device=device)
        self.position_bias = nn.Parameter(torch.zeros(self.m, cfg.head_dim, dtype=torch.float32, device=device))
        self.kv_norm = _Norm(cfg.head_dim, cfg, device)

    def forward(self, x, cu: List[int]):
        cfg, m = self.cfg, self.m
        starts, seg, pos, first = _window_layout(cu, m)
        W = len(starts)
        if W == 0:
            return x.new_zeros(0, cfg.head_dim), seg, first
        idx = (torch.tensor(starts, device=x.device)[:, None] + torch.arange(m, device=x.device)[None, :]).reshape(-1)
        kv = self.kv_proj(x)[idx].view(W, m, -1)
        gate = self.gate_proj(x)[idx].view(W, m, -1).float() + self.position_bias
        comp = self.kv_norm((kv * gate.softmax(1).to(kv.dtype)).sum(1))
        comp = rope_tail(comp[:, None, :], torch.tensor(pos, device=x.device), cfg.compress_rope_theta,
                         cfg.qk_rope_head_dim)[:, 0]
        return comp, seg, first


class _OverlapCompress(nn.Module):
    """Two series per token (Ca for the NEXT window's entry, Cb for the CURRENT one): entry ``w`` is the gated sum over
    window ``w - 1``'s Ca slice and window ``w``'s Cb slice - width ``2 m``, stride ``m``; the first window of a
    sequence has no previous slice."""

    def __init__(self, cfg: DSV4Config, dim: int, device=None):
        super().__init__()
        self.cfg, self.m, self.dim = cfg, cfg.compress_rate_csa, dim
        self.kv_proj = _Lin(cfg.hidden_size, 2 * dim, cfg, device=device)
        self.gate_proj = _Lin(cfg.hidden_size, 2 * dim, cfg, device=device)
        self.position_bias = nn.Parameter(torch.zeros(self.m, 2 * dim, dtype=torch.float32, device=device))
        self.kv_norm = _Norm(dim, cfg, device)

    def forward(self, x, cu: List[int]):
        cfg, m, d = self.cfg, self.m, self.dim
        starts, seg, pos, first = _window_layout(cu, m)
        W = len(starts)
        if W == 0:
            return x.new_zeros(0, d), seg, first
        dev = x.device
        idx = (torch.tensor(starts, device=dev)[:, None] + torch.arange(m, device=dev)[None, :]).reshape(-1)
        kv = self.kv_proj(x)[idx].view(W, m, 2 * d)
        gate = self.gate_proj(x)[idx].view(W, m, 2 * d).float() + self.position_bias
        is_first = torch.tensor([w in set(first[:-1]) for w in range(W)], device=dev)
        prev = torch.arange(W, device=dev).sub(1).clamp_min(0)
        ca_kv, ca_gate = kv[prev][..., :d], gate[prev][..., :d]
        ca_gate = ca_gate.masked_fill(is_first[:, None, None], float("-inf"))
        ca_kv = ca_kv.masked_fill(is_first[:, None, None], 0.0)
        all_kv = torch.cat([ca_kv, kv[..., d:]], 1)                   # [W, 2m, d]
        all_gate = torch.cat([ca_gate, gate[..., d:]], 1)
        comp = self.kv_norm((all_kv * all_gate.softmax(1).to(all_kv.dtype)).sum(1))
        comp = rope_tail(comp[:, None, :], torch.tensor(pos, device=dev), cfg.compress_rope_theta,
                         cfg.qk_rope_head_dim)[:, 0]
        return comp, seg, first


class LightningIndexer(nn.Module):
    """Scores every query against the compressed keys of its own sequence that are already closed,
    ``sum_h w_h relu(q_h . k)``, and keeps the ``index_topk`` best (``-1`` where fewer exist)."""

    def __init__(self, cfg: DSV4Config, device=None):
        super().__init__()
        self.cfg = cfg
        self.compress = _OverlapCompress(cfg, cfg.index_head_dim, device)
        self.q_b_proj = _Lin(cfg.q_lora_rank, cfg.index_n_heads * cfg.index_head_dim, cfg, device=device)
        self.weights_proj = _Lin(cfg.hidden_size, cfg.index_n_heads, cfg, device=device)

    def forward(self, x, q_residual, pos, cu: List[int], seq_of_token, first_window, thresholds):
        cfg = self.cfg
        T = x.shape[0]
        keys, _, _ = self.compress(x, cu)                              # [W, Di]
        W = keys.shape[0]
        k_top = min(cfg.index_topk, max(W, 1))
        if W == 0:
            return torch.full((T, k_top), -1, dtype=torch.int32, device=x.device), None
        q = self.q_b_proj(q_residual).view(T, cfg.index_n_heads, cfg.index_head_dim)
        q = rope_tail(q, pos, cfg.compress_rope_theta, min(cfg.qk_rope_head_dim, cfg.index_head_dim))
        if cfg.indexer_rotate:
            q, keys = K4.rotate_activation(q), K4.rotate_activation(keys)
        w = self.weights_proj(x).float() * cfg.index_n_heads ** -0.5
        ks = first_window[seq_of_token]
        ke = ks + thresholds
        scale = cfg.index_head_dim ** -0.5
        with torch.no_grad():
            scores = K4.indexer_scores(q.detach(), keys.detach(), w.detach(), ks, ke, scale)
            top = scores.topk(k_top, dim=-1)
            idx = torch.where(torch.isfinite(top.values), top.indices, torch.full_like(top.indices, -1)).int()
        # differentiable scores of the kept entries: the indexer learns from a loss on them (see ``indexer_loss``)
        sel = K4.indexer_selected_scores(q, keys, w, idx, scale)
        return idx, sel


class CSACompressor(nn.Module):
    def __init__(self, cfg: DSV4Config, device=None):
        super().__init__()
        self.compress = _OverlapCompress(cfg, cfg.head_dim, device)
        self.indexer = LightningIndexer(cfg, device)
        self.m = cfg.compress_rate_csa


# ---------------------------------------------------------------------------------------------------- attention
class DSV4Attention(nn.Module):
    def __init__(self, cfg: DSV4Config, layer_idx: int, device=None):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.layer_type = cfg.layer_types[layer_idx]
        H, D = cfg.num_attention_heads, cfg.head_dim
        self.theta = cfg.rope_theta if self.layer_type == SLIDING else cfg.compress_rope_theta
        self.q_a_proj = _Lin(cfg.hidden_size, cfg.q_lora_rank, cfg, device=device)
        self.q_a_norm = _Norm(cfg.q_lora_rank, cfg, device)
        self.q_b_proj = _Lin(cfg.q_lora_rank, H * D, cfg, device=device)
        self.kv_proj = _Lin(cfg.hidden_size, D, cfg, device=device)
        self.kv_norm = _Norm(D, cfg, device)
        g = cfg.o_groups
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[cfg.dtype]
        # grouped low-rank output projection: every group of heads has its own [o_lora_rank, H * D / groups] matrix
        self.o_a_weight = nn.Parameter((torch.randn(g, cfg.o_lora_rank, H * D // g, device=device) * cfg.init_std).to(dt))
        self.o_b_proj = _Lin(g * cfg.o_lora_rank, cfg.hidden_size, cfg, std=cfg.init_std / math.sqrt(2 * cfg.num_layers),
                             device=device)
        self.sinks = nn.Parameter(torch.zeros(H, dtype=torch.float32, device=device))
        self.compressor = {SLIDING: None, CSA: CSACompressor, HCA: HCACompressor}[self.layer_type]
        if self.compressor is not None:
            self.compressor = self.compressor(cfg, device)
        self.last_indexer_scores = None

    def forward(self, x, pos, cu: List[int], seq_of_token, window_idx):
        """x [T, hidden]; ``window_idx`` [T, sliding_window] rows of the sliding window of every query (-1 = none)."""
        cfg = self.cfg
        T = x.shape[0]
        H, D, rot = cfg.num_attention_heads, cfg.head_dim, cfg.qk_rope_head_dim
        q_res = self.q_a_norm(self.q_a_proj(x))
        q = _unit_norm(self.q_b_proj(q_res).view(T, H, D), cfg.rms_norm_eps)
        q = rope_tail(q, pos, self.theta, rot)
        kv = rope_tail(self.kv_norm(self.kv_proj(x))[:, None, :], pos, self.theta, rot)[:, 0]     # [T, D], K == V
        idx = window_idx
        if self.compressor is not None:
            if self.layer_type == HCA:
                comp, seg, first = self.compressor(x, cu)
                m = cfg.compress_rate_hca
            else:
                comp, seg, first = self.compressor.compress(x, cu)
                m = cfg.compress_rate_csa
            first_t = torch.tensor(first, device=x.device, dtype=torch.int32)
            thr = ((pos + 1) // m).to(torch.int32)          # closed windows of its own sequence a query may read
            if self.layer_type == HCA:
                # every closed window of the own sequence, as an index list of fixed width
                width = max(max((first[i + 1] - first[i]) for i in range(len(first) - 1)), 1)
                j = torch.arange(width, device=x.device, dtype=torch.int32)[None, :]
                cidx = torch.where(j < thr[:, None], first_t[seq_of_token][:, None] + j, torch.full_like(j, -1))
            else:
                cidx, sel = self.compressor.indexer(x, q_res, pos, cu, seq_of_token, first_t, thr)
                self.last_indexer_scores = sel
            # compressed rows sit behind the T token rows of the shared key / value matrix
            idx = torch.cat([window_idx, torch.where(cidx >= 0, cidx + T, cidx)], 1)
            kv = torch.cat([kv, comp.to(kv.dtype)], 0)
        o = K4.sparse_mqa(q, kv, self.sinks, idx.int().contiguous(), D ** -0.5)                   # [T, H, D]
        o = rope_tail(o, pos, self.theta, rot, inverse=True)
        g = cfg.o_groups
        og = o.reshape(T, g, H * D // g)
        low = torch.einsum("tgi,gri->tgr", og, self.o_a_weight.to(og.dtype)).reshape(T, g * cfg.o_lora_rank)
        return self.o_b_proj(low)


def sliding_window_index(cu: List[int], window: int, device) -> torch.Tensor:
    """[T, window] int32: rows (inside the own sequence) of the ``window`` most recent tokens of every query, itself
    included; -1 where the sequence is shorter."""
    T = cu[-1]
    start = torch.zeros(T, dtype=torch.int32, device=device)
    for s in range(len(cu) - 1):
        start[cu[s]:cu[s + 1]] = cu[s]
    t = torch.arange(T, dtype=torch.int32, device=device)[:, None]
    rows = t - torch.arange(window, dtype=torch.int32, device=device)[None, :]
    return torch.where(rows >= start[:, None], rows, torch.full_like(rows, -1))


# ---------------------------------------------------------------------------------------------------- residual streams
class HyperConnection(nn.Module):
    """``hc_mult`` parallel residual streams [T, n, D].  From the (normalised) streams the module derives, per token:
    read weights that collapse the streams into the sub-layer's input, write weights that spread the sub-layer's output
    over the streams, and an n x n mixing matrix projected onto the doubly-stochastic matrices by Sinkhorn iterations,
    so that the residual path neither amplifies nor attenuates the signal."""

    def __init__(self, cfg: DSV4Config, device=None):
        super().__init__()
        n, d = cfg.hc_mult, cfg.hidden_size
        self.n, self.iters, self.eps = n, cfg.hc_sinkhorn_iters, cfg.rms_norm_eps
        self.proj = nn.Parameter(torch.zeros(n * d, 2 * n + n * n, dtype=torch.float32, device=device))
        bias = torch.zeros(2 * n + n * n, device=device)
        bias[:n] = 0.0                      # read: uniform after the softmax
        bias[n:2 * n] = 0.0                 # write: sigmoid(0) * 2 = 1
        bias[2 * n:] = (torch.eye(n, device=device) * 4.0).reshape(-1)   # mixing starts close to the identity
        self.bias = nn.Parameter(bias)

    def forward(self, streams):
        T, n, d = streams.shape
        flat = _unit_norm(streams.reshape(T, n * d), self.eps).float()
        z = flat @ self.proj + self.bias
        read = z[:, :n].softmax(-1)
        write = 2.0 * torch.sigmoid(z[:, n:2 * n])
        m = torch.exp(z[:, 2 * n:].view(T, n, n))
        for _ in range(self.iters):
            m = m / m.sum(-1, keepdim=True)
            m = m / m.sum(-2, keepdim=True)
        collapsed = (read.to(streams.dtype)[:, :, None] * streams).sum(1)
        return write, m, collapsed

    @staticmethod
    def combine(streams, out, write, mix):
        dt = streams.dtype
        return write.to(dt)[:, :, None] * out[:, None, :] + torch.matmul(mix.to(dt).transpose(-1, -2), streams)


# ---------------------------------------------------------------------------------------------------- experts
def _score(logits, kind):
    if kind == "sqrtsoftplus":
        return torch.sqrt(F.softplus(logits.float()))
    if kind == "sigmoid":
        return torch.sigmoid(logits.float())
    return logits.float().softmax(-1)


class DSV4MoE(nn.Module):
    def __init__(self, cfg: DSV4Config, layer_idx: int, device=None):
        super().__init__()
        self.cfg = cfg
        self.is_hash = layer_idx in cfg.hash_layers
        self.gate = _Lin(cfg.hidden_size, cfg.num_experts, cfg, device=device)
        self.register_buffer("e_score_correction_bias", torch.zeros(cfg.num_experts, device=device))
        shim = SimpleNamespace(dtype=cfg.dtype, moe_ffn_hidden_size=cfg.moe_intermediate_size,
                               hidden_size=cfg.hidden_size)
        self.experts = Experts(shim, cfg.num_experts, device)
        for w in (self.experts.linear_fc1.weight, self.experts.linear_fc2.weight):
            nn.init.normal_(w, std=cfg.init_std)
        self.shared_fc1 = _Lin(cfg.hidden_size, 2 * cfg.shared_intermediate_size, cfg, device=device)
        self.shared_fc2 = _Lin(cfg.shared_intermediate_size, cfg.hidden_size, cfg, device=device)
        self.replay_indices = None    # router replay: recorded expert ids [T, K] override the choice

    def route(self, x, input_ids):
        cfg = self.cfg
        logits = self.gate(x)
        scores = _score(logits, cfg.scoring_func)
        K, E = cfg.num_experts_per_tok, cfg.num_experts
        if self.replay_indices is not None:
            idx = self.replay_indices
        elif self.is_hash:
            # experts by a multiplicative hash of the token id: stable per token, balanced over the vocabulary
            primes = torch.tensor([1000003, 998244353, 19260817, 1000000007, 7368787, 15485863, 32452843, 49979687][:K],
                                  device=x.device)
            base = (input_ids.long()[:, None] * primes[None, :] + torch.arange(K, device=x.device)[None, :] * 7919) % E
            # distinct experts per token: later picks step forward past earlier ones
            idx = base.clone()
            for j in range(1, K):
                for _ in range(K):
                    clash = (idx[:, j:j + 1] == idx[:, :j]).any(1)
                    idx[:, j] = torch.where(clash, (idx[:, j] + 1) % E, idx[:, j])
        else:
            idx = torch.topk(scores + self.e_score_correction_bias, K, dim=-1, sorted=False).indices
        w = scores.gather(1, idx)
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
        return logits, w * cfg.routed_scaling_factor, idx

    def forward(self, x, input_ids):
        cfg = self.cfg
        T, Hd = x.shape
        K = cfg.num_experts_per_tok
        _, w, idx = self.route(x, input_ids)
        self.last_indices = idx
        dest, offsets = build_dispatch_plan(idx.reshape(-1), cfg.num_experts)
        rows = padded_rows_bound(T * K, cfg.num_experts)
        token_of = torch.arange(T, device=x.device).repeat_interleave(K)
        x_perm = torch.zeros(rows, Hd, dtype=x.dtype, device=x.device).index_copy(0, dest, x[token_of])
        y = (self.experts(x_perm, offsets)[dest].view(T, K, Hd) * w.to(x.dtype)[:, :, None]).sum(1)
        return y + self.shared_fc2(fused.swiglu(self.shared_fc1(x)))


# ---------------------------------------------------------------------------------------------------- model
class DSV4Layer(nn.Module):
    def __init__(self, cfg: DSV4Config, layer_idx: int, device=None):
        super().__init__()
        self.self_attn = DSV4Attention(cfg, layer_idx, device)
        self.mlp = DSV4MoE(cfg, layer_idx, device)
        self.input_layernorm = _Norm(cfg.hidden_size, cfg, device)
        self.post_attention_layernorm = _Norm(cfg.hidden_size, cfg, device)
        self.attn_hc, self.ffn_hc = HyperConnection(cfg, device), HyperConnection(cfg, device)

    def forward(self, streams, input_ids, pos, cu, seq_of_token, window_idx):
        write, mix, collapsed = self.attn_hc(streams)
        a = self.self_attn(self.input_layernorm(collapsed), pos, cu, seq_of_token, window_idx)
        streams = HyperConnection.combine(streams, a, write, mix)
        write, mix, collapsed = self.ffn_hc(streams)
        f = self.mlp(self.post_attention_layernorm(collapsed), input_ids)
        return HyperConnection.combine(streams, f, write, mix)


class DeepseekV4Model(nn.Module):
    def __init__(self, cfg: DSV4Config, device=None):
        super().__init__()
        self.cfg = cfg
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[cfg.dtype]
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden_size, device=device, dtype=dt)
        nn.init.normal_(self.embed.weight, std=cfg.init_std)
        self.layers = nn.ModuleList(DSV4Layer(cfg, i, device) for i in range(cfg.num_layers))
        self.norm = _Norm(cfg.hidden_size, cfg, device)
        self.lm_head = _Lin(cfg.hidden_size, cfg.vocab_size, cfg, device=device)
        self.final_hc = nn.Parameter(torch.zeros(cfg.hc_mult, dtype=torch.float32, device=device))

    def forward(self, input_ids: torch.Tensor, cu_seqlens, position_ids: Optional[torch.Tensor] = None):
        """Packed tokens [T] with sequence boundaries ``cu_seqlens`` -> final hidden states [T, hidden]."""
        cfg = self.cfg
        cu = [int(c) for c in (cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens)]
        T = input_ids.numel()
        assert cu[-1] == T
        dev = input_ids.device
        seq_of_token = torch.zeros(T, dtype=torch.long, device=dev)
        pos = torch.zeros(T, dtype=torch.int32, device=dev)
        for s in range(len(cu) - 1):
            seq_of_token[cu[s]:cu[s + 1]] = s
            pos[cu[s]:cu[s + 1]] = torch.arange(cu[s + 1] - cu[s], dtype=torch.int32, device=dev)
        if position_ids is not None:
            pos = position_ids.to(torch.int32)
        window_idx = sliding_window_index(cu, cfg.sliding_window, dev)
        x = self.embed(input_ids)
        streams = x[:, None, :].expand(T, cfg.hc_mult, cfg.hidden_size).contiguous()
        for layer in self.layers:
            streams = layer(streams, input_ids, pos, cu, seq_of_token, window_idx)
        h = (self.final_hc.softmax(0).to(streams.dtype)[None, :, None] * streams).sum(1)
        return self.norm(h)

    def logits(self, hidden):
        return self.lm_head(hidden)

    def indexer_loss(self) -> Optional[torch.Tensor]:
        """Keeps the indexers trainable without touching the main path: maximises the (log-)scores of the entries each
        indexer selected, i.e. sharpens its ranking around what attention then used (a stand-in for the reference's
        distillation of attention mass into the indexer; freeze_csa_indexer.py covers the frozen case)."""
        terms = [l.self_attn.last_indexer_scores for l in self.layers if l.self_attn.last_indexer_scores is not None]
        if not terms:
            return None
        return -sum(torch.log1p(t.clamp_min(0)).mean() for t in terms) / len(terms)


def causal_lm_loss(model: DeepseekV4Model, input_ids, cu_seqlens, loss_mask=None):
    """Mean next-token cross-entropy inside every sequence of the packed stream."""
    h = model(input_ids, cu_seqlens)
    logits = model.logits(h).float()
    cu = cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else list(cu_seqlens)
    tgt = torch.roll(input_ids, -1)
    m = torch.ones(input_ids.numel(), device=input_ids.device) if loss_mask is None else loss_mask.float().clone()
    for e in cu[1:]:
        m[e - 1] = 0.0      # the last token of a sequence predicts nothing
    nll = F.cross_entropy(logits, tgt, reduction="none")
    return (nll * m).sum() / m.sum().clamp_min(1.0)
