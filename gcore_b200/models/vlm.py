"""Vision-language model: a ViT-style vision tower with a 2x2 spatial merger in front of the text decoder
(Qwen2-VL / Qwen3-VL layout, the family the reference adapts in gpatch_v4/extended_model/qwen3_vl.py).

Images arrive as flattened patches ``[num_patches, 3 * patch * patch]`` with one ``(h, w)`` patch grid per image
(h and w even).  The tower runs full (non-causal) varlen attention over each image's patches with the same
flash-attention, RMSNorm, SwiGLU and GEMM kernels as the decoder; the merger concatenates every 2x2 patch block and
projects it to the decoder width; the resulting vectors replace the embeddings of the ``image_token_id`` placeholders
in the packed token stream, in order, and the decoder runs on ``inputs_embeds``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..ops import fused
from ..ops.attention import flash_attn_varlen
from ..ops.gemm import linear
from .config import ModelConfig
from .gpt import GPTModel


@dataclass
class VisionConfig:
    patch_size: int = 14
    in_channels: int = 3
    hidden_size: int = 256
    num_layers: int = 2
    num_heads: int = 4
    ffn_hidden_size: int = 512
    max_grid: int = 64            # learned 2-D position table covers grids up to max_grid x max_grid patches
    spatial_merge: int = 2
    rms_norm_eps: float = 1e-6
    init_std: float = 0.02

    @property
    def patch_dim(self):
        return self.in_channels * self.patch_size * self.patch_size

    @property
    def head_dim(self):
        return self.hidden_size // self.num_heads


class _Lin(nn.Module):
    def __init__(self, i, o, dtype, device, bias=True, std=0.02):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(o, i, dtype=torch.float32, device=device).mul_(std).to(dtype))
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype, device=device)) if bias else None

    def forward(self, x):
        return linear(x, self.weight, self.bias, getattr(self.weight, "main_grad", None) if self.weight.requires_grad
                      else None)


class VisionBlock(nn.Module):
    def __init__(self, vc: VisionConfig, dtype, device):
        super().__init__()
        self.vc = vc
        H = vc.hidden_size
        self.ln1 = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.ln2 = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.qkv = _Lin(H, 3 * H, dtype, device, std=vc.init_std)
        self.proj = _Lin(H, H, dtype, device, std=vc.init_std / math.sqrt(2 * vc.num_layers))
        self.fc1 = _Lin(H, 2 * vc.ffn_hidden_size, dtype, device, bias=False, std=vc.init_std)
        self.fc2 = _Lin(vc.ffn_hidden_size, H, dtype, device, bias=False, std=vc.init_std / math.sqrt(2 * vc.num_layers))

    def forward(self, x, cu, max_len):
        vc = self.vc
        T = x.shape[0]
        h = fused.rmsnorm(x, self.ln1, vc.rms_norm_eps)[0]
        qkv = self.qkv(h).view(T, 3, vc.num_heads, vc.head_dim)
        o = flash_attn_varlen(qkv[:, 0].contiguous(), qkv[:, 1].contiguous(), qkv[:, 2].contiguous(), cu, cu, max_len,
                              max_len, causal=False)
        x = x + self.proj(o.reshape(T, vc.hidden_size))
        h = fused.rmsnorm(x, self.ln2, vc.rms_norm_eps)[0]
        return x + self.fc2(fused.swiglu(self.fc1(h)))


class VisionTower(nn.Module):
    def __init__(self, vc: VisionConfig, out_hidden: int, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.vc = vc
        H = vc.hidden_size
        self.patch_embed = _Lin(vc.patch_dim, H, dtype, device, std=vc.init_std)
        self.pos_h = nn.Parameter(torch.randn(vc.max_grid, H // 2, device=device).mul_(vc.init_std).to(dtype))
        self.pos_w = nn.Parameter(torch.randn(vc.max_grid, H - H // 2, device=device).mul_(vc.init_std).to(dtype))
        self.blocks = nn.ModuleList([VisionBlock(vc, dtype, device) for _ in range(vc.num_layers)])
        self.ln_out = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        m = vc.spatial_merge ** 2
        self.merge_fc1 = _Lin(H * m, H * m, dtype, device, std=vc.init_std)
        self.merge_fc2 = _Lin(H * m, out_hidden, dtype, device, std=vc.init_std)

    def forward(self, patches: torch.Tensor, grids: Sequence[Tuple[int, int]]) -> torch.Tensor:
        """patches [sum(h*w), patch_dim] in row-major patch order per image -> [sum(h*w / 4), out_hidden]."""
        vc = self.vc
        dev = patches.device
        x = self.patch_embed(patches.to(self.patch_embed.weight.dtype))
        pos, cu, mx = [], [0], 0
        for (h, w) in grids:
            assert h % vc.spatial_merge == 0 and w % vc.spatial_merge == 0 and max(h, w) <= vc.max_grid
            ph = self.pos_h[:h][:, None, :].expand(h, w, -1)
            pw = self.pos_w[:w][None, :, :].expand(h, w, -1)
            pos.append(torch.cat([ph, pw], dim=-1).reshape(h * w, -1))
            cu.append(cu[-1] + h * w)
            mx = max(mx, h * w)
        x = x + torch.cat(pos, 0)
        cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
        for blk in self.blocks:
            x = blk(x, cu_t, mx)
        x = fused.rmsnorm(x, self.ln_out, vc.rms_norm_eps)[0]
        # 2x2 merge: gather the four patches of every block next to each other
        s = vc.spatial_merge
        merged = []
        for i, (h, w) in enumerate(grids):
            xi = x[cu[i]:cu[i + 1]].view(h // s, s, w // s, s, -1).permute(0, 2, 1, 3, 4).reshape((h // s) * (w // s), -1)
            merged.append(xi)
        y = torch.cat(merged, 0)
        return self.merge_fc2(torch.nn.functional.gelu(self.merge_fc1(y)))


class VLModel(nn.Module):
    """Text decoder + vision tower.  ``forward`` has the decoder's signature plus ``vision=(patches, grids)``."""

    def __init__(self, cfg: ModelConfig, vc: VisionConfig, image_token_id: int, device=None, **gpt_kw):
        super().__init__()
        assert gpt_kw.get("tp_size", 1) == 1, "the vision-language wrapper runs with tensor parallel size 1"
        self.cfg, self.vc, self.image_token_id = cfg, vc, image_token_id
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[cfg.dtype]
        self.language_model = GPTModel(cfg, device=device, **gpt_kw)
        self.vision = VisionTower(vc, cfg.hidden_size, dt, device)

    # the training engine talks to these
    def output_weight(self):
        return self.language_model.output_weight()

    def vocab_start(self):
        return 0

    @property
    def tp_size(self):
        return 1

    @property
    def sequence_parallel(self):
        return False

    @property
    def decoder(self):
        return self.language_model.decoder

    def reset_parameters(self, seed: Optional[int] = None):
        self.language_model.reset_parameters(seed)

    def num_image_tokens(self, grids) -> List[int]:
        s = self.vc.spatial_merge ** 2
        return [h * w // s for h, w in grids]

    def forward(self, input_ids, position_ids, cu_seqlens, max_seqlen, vision=None, **kw):
        emb = torch.nn.functional.embedding(input_ids, self.language_model.embedding.word_embeddings.weight)
        if vision is not None and vision[0] is not None and vision[0].numel():
            feats = self.vision(vision[0], vision[1]).to(emb.dtype)
            where = (input_ids == self.image_token_id).nonzero().flatten()
            assert where.numel() == feats.shape[0], (f"{where.numel()} image placeholder tokens for "
                                                     f"{feats.shape[0]} merged vision patches")
            emb = emb.index_copy(0, where, feats)
        return self.language_model(None, position_ids, cu_seqlens, max_seqlen, inputs_embeds=emb, **kw)
