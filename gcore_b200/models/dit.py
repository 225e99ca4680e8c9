"""Image-generation model family: a rectified-flow multimodal diffusion transformer (double-stream + single-stream
blocks over text and latent-patch tokens, adaLN modulation from timestep / pooled text / guidance, 3-axis rotary
position ids), a text encoder, and a latent autoencoder.

These are the networks the reference drives through diffusers inside its text-to-image pipelines (Flux,
Qwen-Image-Edit; gpatch_v4/extended_pipeline/pipeline_flux.py:52-110, pipeline_qwen_image_edit.py) - here they are
ordinary modules of this package, random-initialised or loaded from a state dict, whose linear layers run on the
package's GEMM (``ops.gemm.linear``) and whose joint attention runs on the package's non-causal flash attention when
the head size allows it.

Call contract of ``MMDiT.forward`` (names of the diffusers transformer the reference calls, pipeline_flux.py:288-300):
``hidden_states [B, N, C]`` packed latent patches, ``encoder_hidden_states [B, Nt, Dt]``, ``timestep [B]`` in [0, 1],
``pooled_projections [B, Dp]``, ``img_ids [N, 3]``, ``txt_ids [Nt, 3]``, ``guidance [B] | None`` -> velocity
``[B, N, C]``.  Extra conditioning tokens (an edit's source image) are appended to ``hidden_states`` by the caller
with their own ids; the caller keeps the first N outputs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class DiTConfig:
    in_channels: int = 64            # latent channels x patch area (16 x 2 x 2)
    hidden_size: int = 256
    num_heads: int = 4
    depth_double: int = 2
    depth_single: int = 2
    text_dim: int = 128
    pooled_dim: int = 64
    mlp_ratio: float = 4.0
    guidance_embeds: bool = False
    axes_dims_rope: Tuple[int, int, int] = (16, 24, 24)   # sums to the head size
    rope_theta: float = 10000.0
    dtype: str = "float32"

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    def __post_init__(self):
        self.axes_dims_rope = tuple(self.axes_dims_rope)
        assert sum(self.axes_dims_rope) == self.head_dim, "rotary axes must sum to the head size"
        assert all(d % 2 == 0 for d in self.axes_dims_rope)


def _linear(x, w, b=None):
    from ..ops.gemm import linear
    return linear(x, w, b)


class Linear(nn.Module):
    """``y = x W^T + b`` on the package GEMM (tcgen05 on a GPU in bf16, ``F.linear`` elsewhere)."""

    def __init__(self, din, dout, bias=True, zero=False):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(dout, din))
        self.bias = nn.Parameter(torch.zeros(dout)) if bias else None
        if zero:
            nn.init.zeros_(self.weight)
        else:
            nn.init.normal_(self.weight, std=0.02)

    def forward(self, x):
        return _linear(x, self.weight, self.bias)


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0, scale: float = 1000.0):
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    args = (t.float() * scale)[:, None] * freqs[None]
    return torch.cat([args.cos(), args.sin()], -1)


def rope_tables(ids: torch.Tensor, axes: Tuple[int, ...], theta: float):
    """ids [N, len(axes)] -> (cos, sin) [N, head_dim / 2]."""
    cos, sin = [], []
    for a, d in enumerate(axes):
        inv = theta ** (-torch.arange(0, d, 2, device=ids.device, dtype=torch.float32) / d)
        ang = ids[:, a].float()[:, None] * inv[None]
        cos.append(ang.cos())
        sin.append(ang.sin())
    return torch.cat(cos, -1), torch.cat(sin, -1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """x [B, N, H, D] with interleaved pairs; tables [N, D/2]."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    a, b = xf[..., 0], xf[..., 1]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.stack([a * c - b * s, a * s + b * c], -1).reshape(x.shape).to(x.dtype)


def joint_attention(q, k, v):
    """Full (non-causal) attention, q / k / v [B, N, H, D] -> [B, N, H * D]."""
    B, N, H, D = q.shape
    if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128):
        from ..ops.attention import flash_attn_varlen
        cu = torch.arange(0, (B + 1) * N, N, device=q.device, dtype=torch.int32)
        o = flash_attn_varlen(q.reshape(B * N, H, D), k.reshape(B * N, H, D), v.reshape(B * N, H, D), cu, cu, N, N,
                              causal=False)
        return o.reshape(B, N, H * D)
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    return o.transpose(1, 2).reshape(B, N, H * D)


class RMSNorm(nn.Module):
    def __init__(self, d, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)


class Modulation(nn.Module):
    def __init__(self, d, n):
        super().__init__()
        self.n = n
        self.lin = Linear(d, n * d, zero=True)

    def forward(self, vec):
        return self.lin(F.silu(vec))[:, None, :].chunk(self.n, -1)


def _ln(x):
    return F.layer_norm(x.float(), x.shape[-1:]).to(x.dtype)


class StreamParams(nn.Module):
    """One stream (image or text) of a double block."""

    def __init__(self, cfg: DiTConfig):
        super().__init__()
        d, h = cfg.hidden_size, int(cfg.hidden_size * cfg.mlp_ratio)
        self.mod = Modulation(d, 6)
        self.qkv = Linear(d, 3 * d)
        self.q_norm, self.k_norm = RMSNorm(cfg.head_dim), RMSNorm(cfg.head_dim)
        self.proj = Linear(d, d)
        self.fc1, self.fc2 = Linear(d, h), Linear(h, d)


class DoubleStreamBlock(nn.Module):
    def __init__(self, cfg: DiTConfig):
        super().__init__()
        self.cfg = cfg
        self.img, self.txt = StreamParams(cfg), StreamParams(cfg)

    def _pre(self, sp: StreamParams, x, vec):
        m = sp.mod(vec)
        B, N, _ = x.shape
        H, D = self.cfg.num_heads, self.cfg.head_dim
        q, k, v = sp.qkv(_ln(x) * (1 + m[1]) + m[0]).view(B, N, 3, H, D).unbind(2)
        return sp.q_norm(q), sp.k_norm(k), v, m

    def forward(self, img, txt, vec, rope):
        qi, ki, vi, mi = self._pre(self.img, img, vec)
        qt, kt, vt, mt = self._pre(self.txt, txt, vec)
        q, k, v = torch.cat([qt, qi], 1), torch.cat([kt, ki], 1), torch.cat([vt, vi], 1)
        q, k = apply_rope(q, *rope), apply_rope(k, *rope)
        a = joint_attention(q, k, v)
        nt = txt.shape[1]
        at, ai = a[:, :nt], a[:, nt:]
        img = img + mi[2] * self.img.proj(ai)
        img = img + mi[5] * self.img.fc2(F.gelu(self.img.fc1(_ln(img) * (1 + mi[4]) + mi[3]), approximate="tanh"))
        txt = txt + mt[2] * self.txt.proj(at)
        txt = txt + mt[5] * self.txt.fc2(F.gelu(self.txt.fc1(_ln(txt) * (1 + mt[4]) + mt[3]), approximate="tanh"))
        return img, txt


class SingleStreamBlock(nn.Module):
    def __init__(self, cfg: DiTConfig):
        super().__init__()
        self.cfg = cfg
        d, h = cfg.hidden_size, int(cfg.hidden_size * cfg.mlp_ratio)
        self.h = h
        self.mod = Modulation(d, 3)
        self.lin1 = Linear(d, 3 * d + h)
        self.lin2 = Linear(d + h, d)
        self.q_norm, self.k_norm = RMSNorm(cfg.head_dim), RMSNorm(cfg.head_dim)

    def forward(self, x, vec, rope):
        B, N, d = x.shape
        H, D = self.cfg.num_heads, self.cfg.head_dim
        shift, scale, gate = self.mod(vec)
        y = self.lin1(_ln(x) * (1 + scale) + shift)
        qkv, mlp = y[..., :3 * d], y[..., 3 * d:]
        q, k, v = qkv.reshape(B, N, 3, H, D).unbind(2)
        q, k = apply_rope(self.q_norm(q), *rope), apply_rope(self.k_norm(k), *rope)
        a = joint_attention(q, k, v)
        return x + gate * self.lin2(torch.cat([a, F.gelu(mlp, approximate="tanh")], -1))


class MMDiT(nn.Module):
    def __init__(self, cfg: DiTConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.hidden_size
        self.img_in = Linear(cfg.in_channels, d)
        self.txt_in = Linear(cfg.text_dim, d)
        self.time_in = nn.Sequential(Linear(256, d), nn.SiLU(), Linear(d, d))
        self.pooled_in = nn.Sequential(Linear(cfg.pooled_dim, d), nn.SiLU(), Linear(d, d))
        self.guidance_in = nn.Sequential(Linear(256, d), nn.SiLU(), Linear(d, d)) if cfg.guidance_embeds else None
        self.double_blocks = nn.ModuleList(DoubleStreamBlock(cfg) for _ in range(cfg.depth_double))
        self.single_blocks = nn.ModuleList(SingleStreamBlock(cfg) for _ in range(cfg.depth_single))
        self.final_mod = Modulation(d, 2)
        self.final = Linear(d, cfg.in_channels, zero=True)
        self.gradient_checkpointing = False

    @property
    def hf_model_config(self):
        return self.cfg

    def forward(self, hidden_states, encoder_hidden_states, timestep, pooled_projections, img_ids, txt_ids,
                guidance=None):
        cfg = self.cfg
        dt = hidden_states.dtype
        img = self.img_in(hidden_states)
        txt = self.txt_in(encoder_hidden_states.to(dt))
        vec = self.time_in(timestep_embedding(timestep, 256).to(dt)) + self.pooled_in(pooled_projections.to(dt))
        if self.guidance_in is not None:
            g = guidance if guidance is not None else torch.ones_like(timestep)
            vec = vec + self.guidance_in(timestep_embedding(g, 256).to(dt))
        ids = torch.cat([txt_ids, img_ids], 0)
        rope = rope_tables(ids, cfg.axes_dims_rope, cfg.rope_theta)
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.double_blocks:
            if ckpt:
                img, txt = torch.utils.checkpoint.checkpoint(blk, img, txt, vec, rope, use_reentrant=False)
            else:
                img, txt = blk(img, txt, vec, rope)
        x = torch.cat([txt, img], 1)
        for blk in self.single_blocks:
            x = torch.utils.checkpoint.checkpoint(blk, x, vec, rope, use_reentrant=False) if ckpt else blk(x, vec, rope)
        img = x[:, txt.shape[1]:]
        shift, scale = self.final_mod(vec)
        return self.final(_ln(img) * (1 + scale) + shift)


# ---------------------------------------------------------------------------------------------------- text side
class ByteTokenizer:
    """UTF-8 bytes + pad (256) / eos (257): prompts need no vocabulary file."""
    pad_id, eos_id, vocab_size = 256, 257, 258

    def __call__(self, texts: List[str], max_length: int = 64):
        ids = torch.full((len(texts), max_length), self.pad_id, dtype=torch.long)
        mask = torch.zeros(len(texts), max_length, dtype=torch.bool)
        for i, t in enumerate(texts):
            b = list(t.encode("utf-8"))[:max_length - 1] + [self.eos_id]
            ids[i, :len(b)] = torch.tensor(b)
            mask[i, :len(b)] = True
        return ids, mask


class TextEncoder(nn.Module):
    """Bidirectional transformer encoder: per-token embeddings (the T5 role) and a pooled vector (the CLIP role)."""

    def __init__(self, text_dim=128, pooled_dim=64, layers=2, heads=4, vocab=ByteTokenizer.vocab_size, max_len=256):
        super().__init__()
        self.emb = nn.Embedding(vocab, text_dim)
        self.pos = nn.Embedding(max_len, text_dim)
        self.layers = nn.ModuleList(nn.TransformerEncoderLayer(text_dim, heads, 4 * text_dim, dropout=0.0,
                                                               batch_first=True, norm_first=True) for _ in range(layers))
        self.norm = nn.LayerNorm(text_dim)
        self.pool = nn.Linear(text_dim, pooled_dim)

    def forward(self, ids, mask):
        x = self.emb(ids) + self.pos(torch.arange(ids.shape[1], device=ids.device))[None]
        for l in self.layers:
            x = l(x, src_key_padding_mask=~mask)
        x = self.norm(x) * mask[..., None]
        pooled = self.pool(x.sum(1) / mask.sum(1, keepdim=True).clamp_min(1))
        return x, pooled


# ---------------------------------------------------------------------------------------------------- latent side
class LatentAutoencoder(nn.Module):
    """Convolutional autoencoder, images [B, 3, H, W] in [-1, 1] <-> latents [B, C, H / f, W / f]."""

    def __init__(self, latent_channels=16, base=32, factor=8, scaling_factor=0.3611, shift_factor=0.1159):
        super().__init__()
        n = int(math.log2(factor))
        enc, ch = [nn.Conv2d(3, base, 3, padding=1)], base
        for _ in range(n):
            enc += [nn.SiLU(), nn.Conv2d(ch, ch * 2, 3, stride=2, padding=1)]
            ch *= 2
        enc += [nn.SiLU(), nn.Conv2d(ch, latent_channels, 3, padding=1)]
        dec = [nn.Conv2d(latent_channels, ch, 3, padding=1)]
        for _ in range(n):
            dec += [nn.SiLU(), nn.Upsample(scale_factor=2, mode="nearest"), nn.Conv2d(ch, ch // 2, 3, padding=1)]
            ch //= 2
        dec += [nn.SiLU(), nn.Conv2d(ch, 3, 3, padding=1)]
        self.encoder, self.decoder = nn.Sequential(*enc), nn.Sequential(*dec)
        self.factor, self.latent_channels = factor, latent_channels
        self.scaling_factor, self.shift_factor = scaling_factor, shift_factor

    def encode(self, images):
        return (self.encoder(images) - self.shift_factor) * self.scaling_factor

    def decode(self, latents):
        return self.decoder(latents / self.scaling_factor + self.shift_factor).clamp(-1, 1)


# ---------------------------------------------------------------------------------------------------- packing
def pack_latents(lat: torch.Tensor) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H/2)(W/2), 4C]: 2 x 2 latent patches become tokens (pipeline mixin ``pack_latents``,
    gpatch_v4/extended_pipeline/mixin.py:199-221)."""
    B, C, H, W = lat.shape
    x = lat.view(B, C, H // 2, 2, W // 2, 2).permute(0, 2, 4, 1, 3, 5)
    return x.reshape(B, (H // 2) * (W // 2), C * 4)


def unpack_latents(tok: torch.Tensor, H: int, W: int) -> torch.Tensor:
    B, N, C4 = tok.shape
    x = tok.view(B, H // 2, W // 2, C4 // 4, 2, 2).permute(0, 3, 1, 4, 2, 5)
    return x.reshape(B, C4 // 4, H, W)


def latent_image_ids(H: int, W: int, device, index: int = 0) -> torch.Tensor:
    """[(H/2)(W/2), 3]: (image index, row, column) of every packed token."""
    ids = torch.zeros(H // 2, W // 2, 3, device=device)
    ids[..., 0] = index
    ids[..., 1] = torch.arange(H // 2, device=device)[:, None]
    ids[..., 2] = torch.arange(W // 2, device=device)[None, :]
    return ids.reshape(-1, 3)
