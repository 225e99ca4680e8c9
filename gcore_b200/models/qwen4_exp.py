"""Qwen4-exp-class hybrid decoder: gated delta-net (linear attention) layers, block-sparse grouped-query attention
layers whose key set is chosen by an indexer (QSA), hashed n-gram ("engram") embeddings injected into the residual
streams, gated hyper-connection residuals and routed experts.

Behavioural model: gpatch_v4/models/qwen4_exp/modeling_qwen4_exp.py (gated delta rule :278-413, delta-net layer
:415-671, QSA indexer :718-825 with its batched form qsa.py:75-170, attention :864-946, gated residual :1048-1083,
n-gram embedding :1125-1221, PLE layer :1224-1300, decoder layer :1389-1467).  Sequences are packed (``[T, ...]`` plus
``cu_seqlens``); every per-sequence recurrence (delta rule state, causal convolutions, n-gram history) restarts at a
sequence boundary.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from types import SimpleNamespace
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import fused
from ..ops.gemm import linear
from .moe import Experts, build_dispatch_plan, padded_rows_bound

LINEAR, FULL = "linear_attention", "full_attention"


@dataclass
class Qwen4ExpConfig:
    vocab_size: int = 1024
    hidden_size: int = 128
    num_layers: int = 4
    layer_types: Tuple[str, ...] = (LINEAR, LINEAR, LINEAR, FULL)
    num_attention_heads: int = 4
    num_key_value_heads: int = 2
    head_dim: int = 32
    rope_theta: float = 1e6
    partial_rotary_factor: float = 0.5
    # delta net
    linear_num_value_heads: int = 4
    linear_num_key_heads: int = 2
    linear_key_head_dim: int = 16
    linear_value_head_dim: int = 16
    linear_conv_kernel_dim: int = 4
    # QSA indexer
    indexer_n_heads: int = 2
    indexer_head_dim: int = 16
    indexer_budget: int = 16
    indexer_compress_ratio: int = 4
    # hyper-connections / engram
    hc_count: int = 2
    hc_lowrank: int = 16
    ngram_size: int = 3
    heads_per_ngram: int = 2
    ngram_vocab_size_base: int = 499
    ple_embed_dim: int = 32
    ple_conv_kernel_size: int = 2
    ple_layer_ids: Tuple[int, ...] = (1, 3)        # 1-based layer numbers that inject n-gram features
    eos_token_id: int = 2
    seed: int = 0
    # experts
    num_experts: int = 4
    num_experts_per_tok: int = 2
    moe_intermediate_size: int = 64
    shared_expert_intermediate_size: int = 64
    norm_topk_prob: bool = True
    rms_norm_eps: float = 1e-6
    dtype: str = "float32"
    init_std: float = 0.02

    def __post_init__(self):
        self.layer_types = tuple(self.layer_types)
        assert len(self.layer_types) == self.num_layers


class _Lin(nn.Module):
    def __init__(self, i, o, cfg, device=None, std=None):
        super().__init__()
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[cfg.dtype]
        self.weight = nn.Parameter((torch.randn(o, i, device=device) * (std or cfg.init_std)).to(dt))

    def forward(self, x):
        return linear(x, self.weight, None, getattr(self.weight, "main_grad", None) if self.weight.requires_grad
                      else None)


class _Norm(nn.Module):
    """RMS norm over the last ``group`` elements (``group < width``: every residual stream on its own)."""

    def __init__(self, width, cfg, device=None, group: Optional[int] = None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width, device=device))
        self.eps, self.group = cfg.rms_norm_eps, group or width

    def forward(self, x):
        xf = x.float().unflatten(-1, (-1, self.group))
        y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).flatten(-2)
        return (y * self.weight.float()).to(x.dtype)


def _segments(cu: Sequence[int]):
    return list(zip(cu[:-1], cu[1:]))


def _causal_conv(x: torch.Tensor, weight: torch.Tensor, cu, dilation: int = 1) -> torch.Tensor:
    """Depthwise causal convolution along the token axis, restarted at every sequence start.  x [T, C], weight
    [C, 1, k]."""
    k = weight.shape[-1]
    out = torch.empty_like(x)
    for a, b in _segments(cu):
        seg = F.pad(x[a:b].t()[None], ((k - 1) * dilation, 0))
        out[a:b] = F.conv1d(seg, weight.to(x.dtype), groups=x.shape[1], dilation=dilation)[0].t()
    return out


# ---------------------------------------------------------------------------------------------------- delta net
def gated_delta_rule(q, k, v, g, beta, cu):
    """Recurrent gated delta rule per sequence: state S [Dk, Dv] per head;
    ``S <- S * exp(g_t);  S <- S + k_t (beta_t (v_t - S^T k_t))^T;  o_t = S^T q_t`` with l2-normalised q / k and q
    scaled by ``Dk ** -0.5``.  q, k [T, H, Dk]; v [T, H, Dv]; g, beta [T, H]."""
    T, H, Dk = q.shape
    qf = F.normalize(q.float(), dim=-1) * Dk ** -0.5
    kf = F.normalize(k.float(), dim=-1)
    vf, gf, bf = v.float(), g.float(), beta.float()
    out = torch.empty(T, H, v.shape[-1], dtype=torch.float32, device=q.device)
    for a, b in _segments(cu):
        S = torch.zeros(H, Dk, v.shape[-1], dtype=torch.float32, device=q.device)
        for t in range(a, b):
            S = S * gf[t].exp()[:, None, None]
            mem = torch.einsum("hkv,hk->hv", S, kf[t])
            delta = (vf[t] - mem) * bf[t][:, None]
            S = S + kf[t][:, :, None] * delta[:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, qf[t])
    return out.to(q.dtype)


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: Qwen4ExpConfig, device=None):
        super().__init__()
        self.cfg = cfg
        self.hv, self.hk = cfg.linear_num_value_heads, cfg.linear_num_key_heads
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        kd, vd = self.hk * self.dk, self.hv * self.dv
        self.in_proj_qkv = _Lin(cfg.hidden_size, 2 * kd + vd, cfg, device)
        self.in_proj_z = _Lin(cfg.hidden_size, vd, cfg, device)
        self.in_proj_b = _Lin(cfg.hidden_size, self.hv, cfg, device)
        self.in_proj_a = _Lin(cfg.hidden_size, self.hv, cfg, device)
        self.conv_weight = nn.Parameter(torch.randn(2 * kd + vd, 1, cfg.linear_conv_kernel_dim, device=device) * 0.2)
        self.dt_bias = nn.Parameter(torch.ones(self.hv, device=device))
        self.A_log = nn.Parameter(torch.log(torch.empty(self.hv, device=device).uniform_(0.5, 8)))
        self.norm_weight = nn.Parameter(torch.ones(self.dv, device=device))
        self.out_proj = _Lin(vd, cfg.hidden_size, cfg, device, std=cfg.init_std / math.sqrt(2 * cfg.num_layers))

    def forward(self, x, cu):
        T = x.shape[0]
        kd, vd = self.hk * self.dk, self.hv * self.dv
        qkv = F.silu(_causal_conv(self.in_proj_qkv(x), self.conv_weight, cu))
        q, k, v = qkv.split([kd, kd, vd], -1)
        rep = self.hv // self.hk
        q = q.view(T, self.hk, self.dk).repeat_interleave(rep, 1)
        k = k.view(T, self.hk, self.dk).repeat_interleave(rep, 1)
        v = v.view(T, self.hv, self.dv)
        beta = torch.sigmoid(self.in_proj_b(x).float())
        g = -self.A_log.float().exp() * F.softplus(self.in_proj_a(x).float() + self.dt_bias)
        o = gated_delta_rule(q, k, v, g, beta, cu)
        z = self.in_proj_z(x).view(T, self.hv, self.dv)
        of = o.float()
        o = (of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps) * self.norm_weight.float()
             * F.silu(z.float())).to(x.dtype)
        return self.out_proj(o.reshape(T, vd))


# ---------------------------------------------------------------------------------------------------- QSA attention
def _rope(x, pos, theta, rot):
    return fused.rope_ref(x, pos, theta, rot, interleaved=False) if rot else x


@torch.no_grad()
def select_qsa_membership(iq, raw_keys, pos, cu, k_norm, theta, rot, ratio: int, block_topk: int):
    """Key set of every query of a packed stream: the ``block_topk`` best complete blocks of ``ratio`` keys inside its
    causal prefix (score = sum over index heads of relu(q . pooled key), pooled = mean of the block's raw keys,
    normalised and rotated at the block's first position) plus the incomplete tail behind the last complete block.
    Returns bool [T, T] (rows = queries, columns = keys of the same packed stream)."""
    T = iq.shape[0]
    member = torch.zeros(T, T, dtype=torch.bool, device=iq.device)
    for a, b in _segments(cu):
        n = b - a
        nb = n // ratio
        p = torch.arange(n, device=iq.device)
        prefix = p + 1                                            # visible keys of query p: [0, p]
        vis_blocks = prefix // ratio
        key_ids = torch.arange(n, device=iq.device)
        tail = (key_ids[None, :] >= (vis_blocks * ratio)[:, None]) & (key_ids[None, :] < prefix[:, None])
        m = tail
        if nb > 0:
            pooled = raw_keys[a:a + nb * ratio].view(nb, ratio, -1).float().mean(1).to(raw_keys.dtype)
            pooled = _rope(k_norm(pooled)[:, None, :], torch.arange(nb, device=iq.device) * ratio, theta, rot)[:, 0]
            sc = torch.relu(torch.einsum("qhd,nd->qhn", iq[a:b].float(), pooled.float())).sum(1) / math.sqrt(iq.shape[-1])
            blk_vis = torch.arange(nb, device=iq.device)[None, :] < vis_blocks[:, None]
            sc = sc.masked_fill(~blk_vis, float("-inf"))
            kmax = min(block_topk, nb)
            top = torch.topk(sc, kmax, dim=-1, sorted=False).indices
            bm = torch.zeros(n, nb, dtype=torch.bool, device=iq.device).scatter_(-1, top, blk_vis.gather(-1, top))
            bm = bm.repeat_interleave(ratio, -1)
            m = tail | F.pad(bm, (0, n - bm.shape[-1]))
        member[a:b, a:b] = m
    return member


class QSAAttention(nn.Module):
    def __init__(self, cfg: Qwen4ExpConfig, device=None):
        super().__init__()
        self.cfg = cfg
        H, Hk, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.q_proj = _Lin(cfg.hidden_size, 2 * H * D, cfg, device)     # queries and the output gate
        self.k_proj = _Lin(cfg.hidden_size, Hk * D, cfg, device)
        self.v_proj = _Lin(cfg.hidden_size, Hk * D, cfg, device)
        self.o_proj = _Lin(H * D, cfg.hidden_size, cfg, device, std=cfg.init_std / math.sqrt(2 * cfg.num_layers))
        self.q_norm, self.k_norm = _Norm(D, cfg, device), _Norm(D, cfg, device)
        Di = cfg.indexer_head_dim
        self.index_qk_proj = _Lin(cfg.hidden_size, (cfg.indexer_n_heads + 1) * Di, cfg, device)
        self.iq_norm, self.ik_norm = _Norm(Di, cfg, device), _Norm(Di, cfg, device)
        self.rot = int(D * cfg.partial_rotary_factor) // 2 * 2
        self.irot = int(Di * cfg.partial_rotary_factor) // 2 * 2

    def forward(self, x, pos, cu):
        cfg = self.cfg
        T = x.shape[0]
        H, Hk, D, Di = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.indexer_head_dim
        iqk = self.index_qk_proj(x)
        iq = _rope(self.iq_norm(iqk[:, :cfg.indexer_n_heads * Di].view(T, cfg.indexer_n_heads, Di)), pos,
                   cfg.rope_theta, self.irot)
        member = select_qsa_membership(iq, iqk[:, cfg.indexer_n_heads * Di:], pos, cu, self.ik_norm, cfg.rope_theta,
                                       self.irot, cfg.indexer_compress_ratio,
                                       cfg.indexer_budget // cfg.indexer_compress_ratio)
        qg = self.q_proj(x).view(T, H, 2 * D)
        q, gate = qg[..., :D], qg[..., D:].reshape(T, H * D)
        q = _rope(self.q_norm(q), pos, cfg.rope_theta, self.rot)
        k = _rope(self.k_norm(self.k_proj(x).view(T, Hk, D)), pos, cfg.rope_theta, self.rot)
        v = self.v_proj(x).view(T, Hk, D)
        o = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
                                           attn_mask=member[None, None], enable_gqa=True)[0].transpose(0, 1)
        return self.o_proj(o.reshape(T, H * D) * torch.sigmoid(gate))


# ---------------------------------------------------------------------------------------------------- engram / PLE
_MASK64 = (1 << 64) - 1
_GAMMA, _M1, _M2 = 0x9E3779B97F4A7C15, 0xBF58476D1CE4E5B9, 0x94D049BB133111EB


def _splitmix64(v: int) -> int:
    v = (v + _GAMMA) & _MASK64
    v = ((v ^ (v >> 30)) * _M1) & _MASK64
    v = ((v ^ (v >> 27)) * _M2) & _MASK64
    return (v ^ (v >> 31)) & _MASK64


def _is_prime(n: int) -> bool:
    if n < 2:
        return False
    if n % 2 == 0:
        return n == 2
    return all(n % d for d in range(3, math.isqrt(n) + 1, 2))


def _nth_prime_after(start: int, count: int) -> int:
    p = start
    for _ in range(count):
        p += 1
        while not _is_prime(p):
            p += 1
    return p


class NGramEmbedding(nn.Module):
    """Hashed n-gram features: for n = 2 .. ngram_size, ``heads_per_ngram`` hash heads map the last n token ids (odd
    64-bit multipliers from a seeded splitmix, XOR-combined, reduced modulo a distinct prime per head) into one shared
    embedding table; an n-gram never reaches across a sequence start or an end-of-sequence token."""

    def __init__(self, cfg: Qwen4ExpConfig, dim: int, ple_index: int, device=None):
        super().__init__()
        self.cfg = cfg
        self.n, self.hpn = cfg.ngram_size, cfg.heads_per_ngram
        heads = (self.n - 1) * self.hpn
        sizes, offs, tot = [], [], 0
        for h in range(heads):
            s = _nth_prime_after(cfg.ngram_vocab_size_base - 1, ple_index * heads + h + 1)
            sizes.append(s)
            offs.append(tot)
            tot += s
        bound = max(1, ((1 << 63) - 1) // max(cfg.vocab_size, 1) // 2)
        base = cfg.seed + 10007 * ple_index
        mult = [2 * (_splitmix64((base + _GAMMA * (i + 1)) & _MASK64) % bound) + 1 for i in range(self.n)]
        self.register_buffer("mult", torch.tensor(mult, dtype=torch.long, device=device))
        self.register_buffer("sizes", torch.tensor(sizes, dtype=torch.long, device=device))
        self.register_buffer("offs", torch.tensor(offs, dtype=torch.long, device=device))
        self.table = nn.Embedding(tot, dim // heads, device=device)
        nn.init.normal_(self.table.weight, std=cfg.init_std)

    def _shifted(self, ids, cu, shift):
        if shift == 0:
            return ids
        eos = self.cfg.eos_token_id
        out = torch.full_like(ids, eos)
        T = ids.numel()
        p = torch.arange(T, device=ids.device)
        start = torch.zeros(T, dtype=torch.long, device=ids.device)
        for a, b in _segments(cu):
            start[a:b] = a
        # an end-of-sequence token also starts a new n-gram segment behind it
        eos_pos = torch.where(ids == eos, p, torch.full_like(p, -1))
        prev_eos = torch.cat([eos_pos.new_full((1,), -1), torch.cummax(eos_pos, 0).values[:-1]])
        seg_start = torch.maximum(start, prev_eos + 1)
        ok = (p - shift) >= seg_start
        out[ok] = ids[(p - shift)[ok]]
        return out

    def forward(self, ids, cu):
        ids = ids.long()
        sh = [self._shifted(ids, cu, s) for s in range(self.n)]
        blocks = []
        for n in range(2, self.n + 1):
            mixed = sh[0] * self.mult[0]
            for j in range(1, n):
                mixed = torch.bitwise_xor(mixed, sh[j] * self.mult[j])
            a = (n - 2) * self.hpn
            blocks.append(torch.remainder(mixed[:, None], self.sizes[a:a + self.hpn][None]) + self.offs[a:a + self.hpn][None])
        return self.table(torch.cat(blocks, -1)).flatten(-2)


class PLELayer(nn.Module):
    """N-gram features enter every residual stream: a shared value and one key per stream; the normalised stream gates
    the value (signed square root of the scaled dot product through a sigmoid); a dilated depthwise causal
    convolution adds local context."""

    def __init__(self, cfg: Qwen4ExpConfig, ple_index: int, device=None):
        super().__init__()
        self.cfg = cfg
        hc = cfg.hc_count * cfg.hidden_size
        self.emb = NGramEmbedding(cfg, cfg.ple_embed_dim, ple_index, device)
        self.key_proj = _Lin(cfg.ple_embed_dim, hc, cfg, device)
        self.value_proj = _Lin(cfg.ple_embed_dim, cfg.hidden_size, cfg, device)
        self.norm_key = _Norm(hc, cfg, device, cfg.hidden_size)
        self.norm_query = _Norm(hc, cfg, device, cfg.hidden_size)
        self.norm_conv = _Norm(hc, cfg, device, cfg.hidden_size)
        self.conv_weight = nn.Parameter(torch.randn(hc, 1, cfg.ple_conv_kernel_size, device=device) * 0.1)

    def forward(self, streams, ids, cu):
        cfg = self.cfg
        e = self.emb(ids, cu).to(streams.dtype)
        key = self.norm_key(self.key_proj(e)).unflatten(-1, (cfg.hc_count, cfg.hidden_size))
        val = self.value_proj(e)
        qry = self.norm_query(streams).unflatten(-1, (cfg.hc_count, cfg.hidden_size))
        gate = (key * qry).sum(-1, keepdim=True) / math.sqrt(cfg.hidden_size)
        gate = gate.abs().clamp_min(1e-6).sqrt() * gate.sign()
        gv = (torch.sigmoid(gate) * val[:, None, :]).flatten(-2)
        return gv + F.silu(_causal_conv(self.norm_conv(gv), self.conv_weight, cu, dilation=cfg.ngram_size))


class GatedResidual(nn.Module):
    """``hc_count`` residual streams kept flat ([T, hc * hidden]): a low-rank gate mixes the normalised streams into
    the sub-layer's input; per-stream injection weights (2 * sigmoid) spread its output back."""

    def __init__(self, cfg: Qwen4ExpConfig, device=None, combine: bool = True):
        super().__init__()
        self.cfg = cfg
        hc = cfg.hc_count * cfg.hidden_size
        self.norm = _Norm(hc, cfg, device, cfg.hidden_size)
        self.down, self.up = _Lin(hc, cfg.hc_lowrank, cfg, device), _Lin(cfg.hc_lowrank, hc, cfg, device)
        self.inject = _Lin(hc, cfg.hc_count, cfg, device) if combine else None   # the final mixer only reads

    def forward(self, streams):
        cfg = self.cfg
        n = self.norm(streams)
        w = torch.sigmoid(self.up(F.silu(self.down(n) / cfg.hc_count))).unflatten(-1, (cfg.hc_count, cfg.hidden_size))
        mixed = (w * n.unflatten(-1, (cfg.hc_count, cfg.hidden_size))).mean(-2)
        return mixed, (2 * torch.sigmoid(self.inject(n) / cfg.hc_count) if self.inject is not None else None)

    @staticmethod
    def inject_back(streams, out, weights):
        return streams + (out[:, None, :] * weights[:, :, None]).flatten(-2)


# ---------------------------------------------------------------------------------------------------- experts / model
class Qwen4MoE(nn.Module):
    def __init__(self, cfg: Qwen4ExpConfig, device=None):
        super().__init__()
        self.cfg = cfg
        self.gate = _Lin(cfg.hidden_size, cfg.num_experts, cfg, device)
        self.experts = Experts(SimpleNamespace(dtype=cfg.dtype, moe_ffn_hidden_size=cfg.moe_intermediate_size,
                                               hidden_size=cfg.hidden_size), cfg.num_experts, device)
        for w in (self.experts.linear_fc1.weight, self.experts.linear_fc2.weight):
            nn.init.normal_(w, std=cfg.init_std)
        self.shared_fc1 = _Lin(cfg.hidden_size, 2 * cfg.shared_expert_intermediate_size, cfg, device)
        self.shared_fc2 = _Lin(cfg.shared_expert_intermediate_size, cfg.hidden_size, cfg, device)
        self.shared_gate = _Lin(cfg.hidden_size, 1, cfg, device)

    def forward(self, x):
        cfg = self.cfg
        T, Hd = x.shape
        K = cfg.num_experts_per_tok
        probs = self.gate(x).float().softmax(-1)
        w, idx = probs.topk(K, -1)
        if cfg.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        self.last_probs, self.last_indices = probs, idx
        dest, offsets = build_dispatch_plan(idx.reshape(-1), cfg.num_experts)
        rows = padded_rows_bound(T * K, cfg.num_experts)
        token_of = torch.arange(T, device=x.device).repeat_interleave(K)
        xp = torch.zeros(rows, Hd, dtype=x.dtype, device=x.device).index_copy(0, dest, x[token_of])
        y = (self.experts(xp, offsets)[dest].view(T, K, Hd) * w.to(x.dtype)[:, :, None]).sum(1)
        return y + torch.sigmoid(self.shared_gate(x)) * self.shared_fc2(fused.swiglu(self.shared_fc1(x)))


class Qwen4ExpLayer(nn.Module):
    def __init__(self, cfg: Qwen4ExpConfig, idx: int, device=None):
        super().__init__()
        self.kind = cfg.layer_types[idx]
        self.mixer = GatedDeltaNet(cfg, device) if self.kind == LINEAR else QSAAttention(cfg, device)
        self.mlp = Qwen4MoE(cfg, device)
        self.ple = PLELayer(cfg, cfg.ple_layer_ids.index(idx + 1), device) if (idx + 1) in cfg.ple_layer_ids else None
        self.attn_hc, self.mlp_hc = GatedResidual(cfg, device), GatedResidual(cfg, device)

    def forward(self, streams, ids, pos, cu):
        if self.ple is not None:
            streams = streams + self.ple(streams, ids, cu)
        x, w = self.attn_hc(streams)
        y = self.mixer(x, cu) if self.kind == LINEAR else self.mixer(x, pos, cu)
        streams = GatedResidual.inject_back(streams, y, w)
        x, w = self.mlp_hc(streams)
        return GatedResidual.inject_back(streams, self.mlp(x), w)


class Qwen4ExpModel(nn.Module):
    def __init__(self, cfg: Qwen4ExpConfig, device=None):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden_size, device=device)
        nn.init.normal_(self.embed.weight, std=cfg.init_std)
        self.layers = nn.ModuleList(Qwen4ExpLayer(cfg, i, device) for i in range(cfg.num_layers))
        self.out_hc = GatedResidual(cfg, device, combine=False)
        self.norm = _Norm(cfg.hidden_size, cfg, device)
        self.lm_head = _Lin(cfg.hidden_size, cfg.vocab_size, cfg, device)

    def forward(self, input_ids, cu_seqlens):
        cfg = self.cfg
        cu = [int(c) for c in (cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens)]
        T = input_ids.numel()
        pos = torch.zeros(T, dtype=torch.int32, device=input_ids.device)
        for a, b in _segments(cu):
            pos[a:b] = torch.arange(b - a, dtype=torch.int32, device=input_ids.device)
        x = self.embed(input_ids)
        streams = x.repeat(1, cfg.hc_count)
        for layer in self.layers:
            streams = layer(streams, input_ids, pos, cu)
        h, _ = self.out_hc(streams)
        return self.norm(h)

    def logits(self, h):
        return self.lm_head(h)

    def load_balancing_loss(self):
        """Switch-style auxiliary loss over all layers: experts x (fraction of routed tokens) x (mean router prob)."""
        E, K = self.cfg.num_experts, self.cfg.num_experts_per_tok
        tot = 0.0
        for l in self.layers:
            p, idx = l.mlp.last_probs, l.mlp.last_indices
            frac = torch.zeros(E, device=p.device).scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), device=p.device))
            tot = tot + E * ((frac / idx.numel()) * p.mean(0)).sum() * K
        return tot / len(self.layers)
