"""Packed (THD) micro-batches.

A micro-batch is a flat token stream with ``cu_seqlens``; per-token fields live on the same axis.  The log-prob axis
follows the reference (gpatch_v4/utils/training_utils.py:1139-1208): position ``t`` of a sequence predicts token
``t+1``, the last position of every sequence has no target and is masked; the response mask covers
``[prompt_len-1, seq_len-1)`` (gpatch_v4/utils/ppo_utils.py:123-148).

Micro-batch formation: fixed sequence count (``train_mbs``) or a token budget packed first-fit-decreasing
(the reference's dynamic micro-batch, megatron_backend/mixin.py:2749-2769), plus Karmarkar-Karp balancing of
sequences across data-parallel ranks (gpatch_v4/core/seqlen_balancing.py).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch


@dataclass
class PackedBatch:
    tokens: torch.Tensor          # [T] int64
    position_ids: torch.Tensor    # [T] int32
    cu_seqlens: torch.Tensor      # [B+1] int32
    max_seqlen: int
    targets: torch.Tensor         # [T] int64 (next token; 0 at sequence ends)
    loss_mask: torch.Tensor       # [T] float32 on the log-prob axis
    seq_ids: torch.Tensor         # [T] int32 index of the owning sequence inside the batch
    sample_index: List[int] = field(default_factory=list)  # indices into the originating sample list
    fields: Dict[str, torch.Tensor] = field(default_factory=dict)  # extra per-token tensors on the log-prob axis
    pad_tokens: int = 0
    cp_ctx: Optional[object] = None  # parallel.cp.CPContext when the token axis is sharded over context-parallel ranks
    # vision-language batches: (patches [sum(h*w), patch_dim], [(h, w), ...]), or with videos a dict of
    # image_patches / image_grid / video_patches / video_grid
    vision: Optional[object] = None
    # context-parallel shards of models with multi-token prediction: the tokens / targets / loss_mask / seq_ids of the
    # first positions behind this rank's chunk (seq_ids -1 past the end of the stream)
    halo: Optional[Dict[str, torch.Tensor]] = None

    def _vision_to(self, kw):
        v = self.vision
        if v is None:
            return None
        if isinstance(v, dict):
            return {k: (x.to(**kw) if isinstance(x, torch.Tensor) else x) for k, x in v.items()}
        return (v[0].to(**kw), v[1])

    @property
    def num_seqs(self):
        return self.cu_seqlens.numel() - 1

    def to(self, device, non_blocking=True):
        kw = dict(device=device, non_blocking=non_blocking)
        return PackedBatch(self.tokens.to(**kw), self.position_ids.to(**kw), self.cu_seqlens.to(**kw),
                           self.max_seqlen, self.targets.to(**kw), self.loss_mask.to(**kw), self.seq_ids.to(**kw),
                           self.sample_index, {k: v.to(**kw) for k, v in self.fields.items()}, self.pad_tokens,
                           self.cp_ctx,
                           self._vision_to(kw),
                           None if self.halo is None else {k: v.to(**kw) for k, v in self.halo.items()})


def response_mask(prompt_len: int, seq_len: int) -> torch.Tensor:
    """Mask over the S positions of the log-prob axis (last position always 0)."""
    m = torch.zeros(seq_len, dtype=torch.float32)
    m[max(prompt_len - 1, 0):max(seq_len - 1, 0)] = 1.0
    return m


def pack_samples(samples: Sequence[Dict], indices: Sequence[int], per_token_keys: Sequence[str] = (),
                 pad_to_multiple: int = 1, pin: bool = False) -> PackedBatch:
    """``samples[i]`` needs ``tokens`` (1-D long).  ``loss_mask`` (length S, log-prob axis) is used when present,
    else it is derived from ``prompt_length``.  Per-token keys of length S-1 are right-padded with one zero."""
    toks, pos, tgt, mask, sid = [], [], [], [], []
    extra: Dict[str, List[torch.Tensor]] = {k: [] for k in per_token_keys}
    cu = [0]
    max_len = 0
    for j, i in enumerate(indices):
        s = samples[i]
        t = torch.as_tensor(s["tokens"], dtype=torch.int64)
        S = t.numel()
        toks.append(t)
        pos.append(torch.arange(S, dtype=torch.int32))
        nxt = torch.zeros(S, dtype=torch.int64)
        nxt[:-1] = t[1:]
        tgt.append(nxt)
        if "loss_mask" in s and s["loss_mask"] is not None:
            m = torch.as_tensor(s["loss_mask"], dtype=torch.float32)
            if m.numel() == S - 1:
                m = torch.cat([m, m.new_zeros(1)])
            m = m.clone()
            m[-1] = 0.0
        else:
            m = response_mask(int(s.get("prompt_length", 0)), S)
        mask.append(m)
        sid.append(torch.full((S,), j, dtype=torch.int32))
        for k in per_token_keys:
            v = torch.as_tensor(s[k], dtype=torch.float32).reshape(-1)
            if v.numel() == S - 1:
                v = torch.cat([v, v.new_zeros(1)])
            elif v.numel() == 1:
                v = v.expand(S).clone()
            assert v.numel() == S, f"field {k}: length {v.numel()} vs sequence {S}"
            extra[k].append(v)
        cu.append(cu[-1] + S)
        max_len = max(max_len, S)
    T = cu[-1]
    pad = (-T) % pad_to_multiple
    if pad:
        # padding is an extra masked pseudo-sequence so attention never mixes it with real tokens
        toks.append(torch.zeros(pad, dtype=torch.int64))
        pos.append(torch.arange(pad, dtype=torch.int32))
        tgt.append(torch.zeros(pad, dtype=torch.int64))
        mask.append(torch.zeros(pad, dtype=torch.float32))
        sid.append(torch.full((pad,), len(indices), dtype=torch.int32))
        for k in per_token_keys:
            extra[k].append(torch.zeros(pad, dtype=torch.float32))
        cu.append(cu[-1] + pad)
        max_len = max(max_len, pad)

    def cat(xs, dtype=None):
        out = torch.cat(xs)
        return out.pin_memory() if pin else out

    vision = None
    imgs = [(samples[i]["pixel_patches"], samples[i]["image_grid"]) for i in indices if "pixel_patches" in samples[i]]
    vids = [(samples[i]["video_patches"], samples[i]["video_grid"]) for i in indices if "video_patches" in samples[i]]
    if imgs:
        grids = [tuple(g) for _, gs in imgs for g in (gs if isinstance(gs[0], (list, tuple)) else [gs])]
        vision = (cat([torch.as_tensor(p, dtype=torch.float32) for p, _ in imgs]), grids)
    if vids:
        # videos ride in a dict next to the images (models that take videos read the dict form)
        vgrids = [tuple(g) for _, gs in vids for g in (gs if isinstance(gs[0], (list, tuple)) else [gs])]
        vision = {"image_patches": vision[0] if vision else None, "image_grid": vision[1] if vision else [],
                  "video_patches": cat([torch.as_tensor(p, dtype=torch.float32) for p, _ in vids]),
                  "video_grid": vgrids}
    return PackedBatch(cat(toks), cat(pos), torch.tensor(cu, dtype=torch.int32), max_len, cat(tgt), cat(mask),
                       cat(sid), list(indices), {k: cat(v) for k, v in extra.items()}, pad, None, vision)


# ------------------------------------------------------------------------------------------------ planners
def _runtime():
    from ..ops._lib import runtime
    return runtime()


def ffd_pack(lengths: Sequence[int], capacity: int) -> List[List[int]]:
    """First-fit-decreasing bins of at most ``capacity`` tokens (native planner, python fallback)."""
    n = len(lengths)
    if n == 0:
        return []
    try:
        lib = _runtime()
        arr = (ctypes.c_int64 * n)(*[int(x) for x in lengths])
        out = (ctypes.c_int * n)()
        lib.gkrt_ffd_pack.restype = ctypes.c_int
        nb = lib.gkrt_ffd_pack(arr, n, ctypes.c_int64(capacity), out)
        bins: List[List[int]] = [[] for _ in range(nb)]
        for i in range(n):
            bins[out[i]].append(i)
        return bins
    except Exception:
        order = sorted(range(n), key=lambda i: -lengths[i])
        bins, load = [], []
        for i in order:
            for b in range(len(bins)):
                if load[b] + lengths[i] <= capacity:
                    bins[b].append(i)
                    load[b] += lengths[i]
                    break
            else:
                bins.append([i])
                load.append(lengths[i])
        return bins


def kk_partition(lengths: Sequence[int], k: int, equal_size: bool = False) -> List[List[int]]:
    """Karmarkar-Karp k-way partition minimising the spread of part sums."""
    n = len(lengths)
    lib = _runtime()
    arr = (ctypes.c_int64 * n)(*[int(x) for x in lengths])
    out = (ctypes.c_int * n)()
    lib.gkrt_kk_partition.restype = ctypes.c_int
    rc = lib.gkrt_kk_partition(arr, n, k, int(equal_size), out)
    if rc != 0:
        raise ValueError(f"kk_partition failed ({rc}): n={n}, k={k}, equal_size={equal_size}")
    parts: List[List[int]] = [[] for _ in range(k)]
    for i in range(n):
        parts[out[i]].append(i)
    return parts


def make_microbatches(lengths: Sequence[int], mbs: Optional[int] = None, max_tokens: Optional[int] = None,
                      sort: bool = False) -> List[List[int]]:
    idx = list(range(len(lengths)))
    if max_tokens:
        return ffd_pack(lengths, max_tokens)
    if sort:
        idx.sort(key=lambda i: -lengths[i])
    mbs = mbs or 1
    return [idx[i:i + mbs] for i in range(0, len(idx), mbs)]
