"""Qwen3-VL-style vision-language adapter: images and videos, multi-axis rotary position ids, intermediate
vision-tower features injected into the first decoder layers.

What the reference's adapter does around the Megatron decoder (gpatch_v4/extended_model/qwen3_vl.py:50 data
preparation, :823-847 rope index, :1383 dynamic-CP reroute of vision inputs) and what this module provides:

* ``get_rope_index``  - (temporal, height, width) position ids of a token stream with image / video placeholders: text
  tokens advance all three axes together; the merged tokens of a visual block share the block's start on the
  temporal axis (plus the frame index) and spread over rows and columns; the text behind a block continues after
  the largest index used (so a decoded token at cache position ``p`` rotates at ``p + delta``; ``rope_delta``).
* ``Qwen3VLModel``    - vision tower over image patches ``(h, w)`` and video patch volumes ``(t, h, w)`` (attention
  inside every frame), 2x2 spatial merge, features written over the placeholder embeddings, features of selected
  tower layers added to the visual tokens' hidden states behind the first decoder layers, decoder run with
  multi-axis rotary tables.
* vision inputs travel inside the samples (``pixel_patches`` / ``image_grid`` / ``video_patches`` / ``video_grid``),
  so DP balancing and the dynamic context-parallel reroute move them with their sequence.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..ops import fused
from .config import ModelConfig
from .vlm import VisionConfig, VisionTower, VLModel, _Lin


def get_rope_index(tokens: Sequence[int], blocks: Sequence[Tuple[int, int, int]], image_token_id: int,
                   video_token_id: Optional[int] = None, spatial_merge: int = 2,
                   video_blocks: Sequence[Tuple[int, int, int]] = ()):
    """-> (pos3 [T, 3] long, rope_delta).  ``blocks``: (t, h, w) patch grid of every image block in order of
    appearance (t = 1), ``video_blocks`` the same for runs of the video placeholder; a block occupies
    ``t * (h / merge) * (w / merge)`` consecutive placeholder tokens."""
    toks = torch.as_tensor(tokens).tolist()
    T = len(toks)
    pos = torch.zeros(T, 3, dtype=torch.long)
    nxt, i = 0, 0
    queues = {image_token_id: list(blocks)}
    if video_token_id is not None:
        queues[video_token_id] = list(video_blocks)
    while i < T:
        q = queues.get(toks[i])
        if q is None:
            pos[i] = nxt
            nxt += 1
            i += 1
            continue
        assert q, "more visual placeholder runs than grids"
        t, h, w = q.pop(0)
        hh, ww = h // spatial_merge, w // spatial_merge
        n = t * hh * ww
        assert i + n <= T and all(x == toks[i] for x in toks[i:i + n]), \
            "a visual block does not match its placeholder run"
        ti = torch.arange(t).view(t, 1, 1).expand(t, hh, ww).reshape(-1)
        hi = torch.arange(hh).view(1, hh, 1).expand(t, hh, ww).reshape(-1)
        wi = torch.arange(ww).view(1, 1, ww).expand(t, hh, ww).reshape(-1)
        pos[i:i + n] = torch.stack([ti, hi, wi], 1) + nxt
        nxt = int(pos[i:i + n].max()) + 1
        i += n
    assert not any(queues.values()), "fewer visual placeholder runs than grids"
    return pos, nxt - T


class DeepStackTower(VisionTower):
    """Vision tower that also returns the merged features of chosen intermediate layers."""

    def __init__(self, vc: VisionConfig, out_hidden: int, dtype, device, deepstack_layers: Sequence[int] = (),
                 temporal_patch: int = 1):
        super().__init__(vc, out_hidden, dtype, device)
        self.deepstack_layers = tuple(deepstack_layers)
        m = vc.spatial_merge ** 2
        H = vc.hidden_size
        self.deep_fc1 = nn.ModuleList([_Lin(H * m, H * m, dtype, device, std=vc.init_std) for _ in self.deepstack_layers])
        self.deep_fc2 = nn.ModuleList([_Lin(H * m, out_hidden, dtype, device, std=vc.init_std)
                                       for _ in self.deepstack_layers])
        self.temporal_patch = temporal_patch
        if temporal_patch > 1:   # video volumes stack `temporal_patch` frames per patch
            self.video_embed = _Lin(vc.patch_dim * temporal_patch, H, dtype, device, std=vc.init_std)

    def _merge(self, x, cu, grids):
        s = self.vc.spatial_merge
        out = []
        for i, (h, w) in enumerate(grids):
            out.append(x[cu[i]:cu[i + 1]].view(h // s, s, w // s, s, -1).permute(0, 2, 1, 3, 4)
                       .reshape((h // s) * (w // s), -1))
        return torch.cat(out, 0)

    def forward(self, patches: torch.Tensor, grids: Sequence[Tuple[int, ...]], video: bool = False):
        """``grids``: (h, w) per image or (t, h, w) per video; attention runs inside every frame.  Returns
        ``(features [N, out], [deepstack features [N, out], ...])``."""
        vc = self.vc
        frames: List[Tuple[int, int]] = []
        for g in grids:
            if len(g) == 3:
                frames += [(g[1], g[2])] * g[0]
            else:
                frames.append(tuple(g))
        embed = self.video_embed if (video and self.temporal_patch > 1) else self.patch_embed
        x = embed(patches.to(embed.weight.dtype))
        pos, cu, mx = [], [0], 0
        for (h, w) in frames:
            assert h % vc.spatial_merge == 0 and w % vc.spatial_merge == 0 and max(h, w) <= vc.max_grid
            pos.append(torch.cat([self.pos_h[:h][:, None, :].expand(h, w, -1),
                                  self.pos_w[:w][None, :, :].expand(h, w, -1)], -1).reshape(h * w, -1))
            cu.append(cu[-1] + h * w)
            mx = max(mx, h * w)
        x = x + torch.cat(pos, 0)
        cu_t = torch.tensor(cu, dtype=torch.int32, device=patches.device)
        deep = []
        for li, blk in enumerate(self.blocks):
            x = blk(x, cu_t, mx)
            if li in self.deepstack_layers:
                k = self.deepstack_layers.index(li)
                y = self._merge(fused.rmsnorm(x, self.ln_out, vc.rms_norm_eps)[0], cu, frames)
                deep.append(self.deep_fc2[k](torch.nn.functional.gelu(self.deep_fc1[k](y))))
        y = self._merge(fused.rmsnorm(x, self.ln_out, vc.rms_norm_eps)[0], cu, frames)
        return self.merge_fc2(torch.nn.functional.gelu(self.merge_fc1(y))), deep


class Qwen3VLModel(VLModel):
    def __init__(self, cfg: ModelConfig, vc: VisionConfig, image_token_id: int, video_token_id: Optional[int] = None,
                 deepstack_layers: Sequence[int] = (0,), temporal_patch: int = 2, device=None, **gpt_kw):
        super().__init__(cfg, vc, image_token_id, device=device, **gpt_kw)
        assert cfg.mrope_sections is not None, "Qwen3-VL decoders rotate with multi-axis position ids"
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[cfg.dtype]
        self.video_token_id = video_token_id
        self.vision = DeepStackTower(vc, cfg.hidden_size, dt, device, deepstack_layers, temporal_patch)

    @staticmethod
    def _as_blocks(grids):
        return [(1, g[0], g[1]) if len(g) == 2 else tuple(g) for g in (grids or [])]

    def position_ids(self, input_ids: torch.Tensor, cu_seqlens: torch.Tensor, per_seq_blocks):
        """Multi-axis ids of a packed batch: every sequence of the batch is indexed on its own.
        ``per_seq_blocks[i] = (image blocks, video blocks)`` of sequence i."""
        cu = cu_seqlens.tolist()
        toks = input_ids.tolist()
        out = []
        for i in range(len(cu) - 1):
            img, vid = per_seq_blocks[i] if i < len(per_seq_blocks) else ([], [])
            p, _ = get_rope_index(toks[cu[i]:cu[i + 1]], img, self.image_token_id, self.video_token_id,
                                  self.vc.spatial_merge, vid)
            out.append(p)
        pos = torch.cat(out, 0) if out else torch.zeros(0, 3, dtype=torch.long)
        if pos.shape[0] < input_ids.numel():   # padding pseudo-tokens behind the last sequence
            pad = torch.arange(input_ids.numel() - pos.shape[0])[:, None].expand(-1, 3)
            pos = torch.cat([pos, pad], 0)
        return pos.to(input_ids.device)

    def forward(self, input_ids, position_ids, cu_seqlens, max_seqlen, vision=None, **kw):
        """``vision``: the engine's ``(patches, grids)`` pair for images, or a dict with ``image_patches`` /
        ``image_grid`` / ``video_patches`` / ``video_grid`` and ``blocks_per_sequence`` (grids of every sequence of
        the packed batch, in order of appearance)."""
        emb = torch.nn.functional.embedding(input_ids, self.language_model.embedding.word_embeddings.weight)
        if vision is not None and not isinstance(vision, dict):
            grids = list(vision[1])
            vision = {"image_patches": vision[0], "image_grid": grids}
        deep = None
        per_seq = []
        if vision is not None:
            feats, deep_parts, where_parts = [], [], []
            for kind, tok in (("image", self.image_token_id), ("video", self.video_token_id)):
                p = vision.get(kind + "_patches")
                if p is None or not p.numel():
                    continue
                f, d = self.vision(p.to(emb.device), vision[kind + "_grid"], video=kind == "video")
                w = (input_ids == tok).nonzero().flatten()
                assert w.numel() == f.shape[0], f"{w.numel()} {kind} placeholder tokens for {f.shape[0]} features"
                feats.append(f)
                deep_parts.append(d)
                where_parts.append(w)
            if feats:
                where = torch.cat(where_parts)
                emb = emb.index_copy(0, where, torch.cat(feats).to(emb.dtype))
                n_deep = len(deep_parts[0])
                deep = (where, [torch.cat([d[k] for d in deep_parts]) for k in range(n_deep)])
            per_seq = vision.get("blocks_per_sequence")
            if per_seq is None:
                cu_l = (cu_seqlens if isinstance(cu_seqlens, torch.Tensor) else
                        torch.tensor(cu_seqlens.cu_global)).tolist()
                img = self._split_blocks(input_ids, cu_l, self._as_blocks(vision.get("image_grid")), self.image_token_id)
                vid = self._split_blocks(input_ids, cu_l, self._as_blocks(vision.get("video_grid")), self.video_token_id)
                per_seq = list(zip(img, vid))
        cu = cu_seqlens if isinstance(cu_seqlens, torch.Tensor) else torch.tensor(cu_seqlens.cu_global)
        pos3 = self.position_ids(input_ids, cu, per_seq or [])
        return self.language_model(None, pos3, cu_seqlens, max_seqlen, inputs_embeds=emb, deepstack=deep, **kw)

    def _split_blocks(self, input_ids, cu, blocks, token_id):
        """Splits the flat list of one kind's grids over the sequences of the packed batch by counting that kind's
        placeholder tokens."""
        n_seq = len(cu) - 1
        if token_id is None or not blocks:
            return [[] for _ in range(n_seq)]
        vis = (input_ids == token_id)
        s2 = self.vc.spatial_merge ** 2
        out, b = [], 0
        for i in range(n_seq):
            c = int(vis[cu[i]:cu[i + 1]].sum())
            mine = []
            while c > 0 and b < len(blocks):
                t, h, w = blocks[b]
                c -= t * h * w // s2
                mine.append(blocks[b])
                b += 1
            assert c == 0, "visual placeholder tokens and grids of a sequence disagree"
            out.append(mine)
        return out
