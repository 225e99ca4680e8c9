"""Per-token rewards computed on a re-encoded response (decode -> re-tokenise, e.g. by a reward service with its own
tokenizer pass) mapped back onto the tokens the policy actually sampled.

The two id sequences are aligned by their longest common subsequence (``runtime/csrc/align.cpp``, Myers' O(ND)
algorithm: the sequences differ in ~1 % of the positions, so D is small).  A matched token copies its reward; the
tokens of a differing region share the mean reward of the corresponding re-encoded region, or, when that region is
empty, the mean of the rewards on either side of the gap (the behaviour of the reference's
``gpatch_v4/utils/reward_redist.py``).
"""
from __future__ import annotations

import ctypes
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional, Sequence, Tuple

import torch


def _lcs_python(a: Sequence[int], b: Sequence[int]) -> Tuple[List[int], List[int]]:
    """Quadratic dynamic programme; oracle and fallback when the native runtime is unavailable."""
    n, m = len(a), len(b)
    L = [[0] * (m + 1) for _ in range(n + 1)]
    for i in range(n - 1, -1, -1):
        for j in range(m - 1, -1, -1):
            L[i][j] = L[i + 1][j + 1] + 1 if a[i] == b[j] else max(L[i + 1][j], L[i][j + 1])
    ia, ib, i, j = [], [], 0, 0
    while i < n and j < m:
        if a[i] == b[j]:
            ia.append(i)
            ib.append(j)
            i += 1
            j += 1
        elif L[i + 1][j] >= L[i][j + 1]:
            i += 1
        else:
            j += 1
    return ia, ib


def lcs_match(a: Sequence[int], b: Sequence[int], max_d: Optional[int] = None, native: bool = True):
    """Index pairs ``(ia, ib)`` of one longest common subsequence of ``a`` and ``b`` (both increasing); ``None`` when
    the sequences differ in more than ``max_d`` positions."""
    a, b = list(map(int, a)), list(map(int, b))
    n, m = len(a), len(b)
    if n == 0 or m == 0:
        return [], []
    lib = None
    if native:
        try:
            from ..ops import _lib
            lib = _lib.runtime()
            if not hasattr(lib, "gkrt_lcs_match"):
                lib = None
        except Exception:  # noqa: BLE001 - no compiler / library on this machine
            lib = None
    if lib is None:
        return _lcs_python(a, b)
    A = (ctypes.c_int64 * n)(*a)
    B = (ctypes.c_int64 * m)(*b)
    cap = min(n, m)
    ia, ib = (ctypes.c_int * cap)(), (ctypes.c_int * cap)()
    lib.gkrt_lcs_match.restype = ctypes.c_int
    k = lib.gkrt_lcs_match(A, n, B, m, int(max_d if max_d is not None else n + m), ia, ib, cap)
    if k < 0:
        return None
    return list(ia[:k]), list(ib[:k])


def redistribute_rewards(orig_ids: Sequence[int], reenc_ids: Sequence[int], rewards, max_d: Optional[int] = None,
                         native: bool = True) -> torch.Tensor:
    """``rewards[j]`` belongs to ``reenc_ids[j]``; returns one reward per token of ``orig_ids``."""
    r = torch.as_tensor(rewards, dtype=torch.float32)
    n, m = len(orig_ids), len(reenc_ids)
    assert r.numel() == m, f"{r.numel()} rewards for {m} re-encoded tokens"
    out = torch.zeros(n, dtype=torch.float32)
    if n == 0:
        return out
    match = lcs_match(orig_ids, reenc_ids, max_d, native)
    if match is None:   # too different to align: spread the total evenly
        return out + (float(r.sum()) / n if m else 0.0)
    ia, ib = match
    out[torch.tensor(ia, dtype=torch.long)] = r[torch.tensor(ib, dtype=torch.long)] if ia else out[:0]
    # differing regions between consecutive matches (with sentinels in front and behind)
    pa, pb = [-1] + ia + [n], [-1] + ib + [m]
    for k in range(len(pa) - 1):
        a0, a1 = pa[k] + 1, pa[k + 1]          # orig tokens without a partner
        b0, b1 = pb[k] + 1, pb[k + 1]          # re-encoded tokens without a partner
        if a1 <= a0:
            continue
        if b1 > b0:
            val = float(r[b0:b1].mean())
        else:
            side = [float(r[pb[k]])] if pb[k] >= 0 else []
            side += [float(r[pb[k + 1]])] if pb[k + 1] < m else []
            val = sum(side) / len(side) if side else 0.0
        out[a0:a1] = val
    return out


def redistribute_rewards_batch(orig: Sequence[Sequence[int]], reenc: Sequence[Sequence[int]], rewards: Sequence,
                               workers: int = 8, max_d: Optional[int] = None) -> List[torch.Tensor]:
    """One alignment per sample on a thread pool (the native routine releases the interpreter lock)."""
    if len(orig) <= 1 or workers <= 1:
        return [redistribute_rewards(a, b, r, max_d) for a, b, r in zip(orig, reenc, rewards)]
    with ThreadPoolExecutor(max_workers=workers) as pool:
        return list(pool.map(lambda t: redistribute_rewards(*t, max_d), zip(orig, reenc, rewards)))
