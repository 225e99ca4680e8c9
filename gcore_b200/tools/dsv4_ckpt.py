"""DeepSeek-V4 checkpoint formats: conversion between the published layout (fp4 experts packed two codes per byte
with one power-of-two scale per 1x32 block, fp8 dense projections with power-of-two 128x128 scales, fp8 ``attn.wo_a``),
the fp8 serving layout (fp8 experts and dense projections with fp32 128x128 scales, bf16 ``attn.wo_a``) and plain bf16
for training; plus a value-level comparison of two checkpoint directories.  Same jobs as the reference's
tools/dsv4_quant_and_dequant/convert.py:160-330, tools/dsv4_quant_and_dequant/compare_hf_ckpts.py and
tools/convert_deepseek_v4_fp4_to_bf16.py:25-80, done shard by shard on safetensors files.

    python -m gcore_b200.tools.dsv4_ckpt convert --direction published2fp8 --src in --dst out
    python -m gcore_b200.tools.dsv4_ckpt convert --direction fp82published --src in --dst out
    python -m gcore_b200.tools.dsv4_ckpt convert --direction to_bf16       --src in --dst out
    python -m gcore_b200.tools.dsv4_ckpt compare --a dir_a --b dir_b

Several ranks (``torchrun``: RANK / WORLD_SIZE in the environment) split the shard files by size, largest first
onto the least loaded rank; every rank writes its own shards and a fragment of the weight map, rank 0 merges the
fragments into ``model.safetensors.index.json`` once all fragments are on disk (no collective, no process group).

Exactness.  Every e2m1 value times a power of two is an e4m3 value as long as the 1x32 scales inside a 128x128 block
span at most 2^8 (e2m1's smallest value 0.5 can move down eight binades into e4m3's subnormals), so published -> fp8
is lossless up to that span, and the tool counts the blocks beyond it.  fp8 -> published re-quantises to fp4; values
that came from fp4 survive exactly (they are m * 2^e with a one-bit mantissa, and the re-derived scale is never
coarser than the original), anything else is rounded to the nearest e2m1 code.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import re
import shutil
import time
from typing import Dict, Optional, Tuple

import torch

E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])
E8M0 = getattr(torch, "float8_e8m0fnu", None)
_EXPERT = re.compile(r"(?:^|\.)experts\.\d+\.w[123]\.weight$")
_WO_A = re.compile(r"(?:^|\.)attn\.wo_a\.weight$")


def is_expert(name: str) -> bool:
    return _EXPERT.search(name) is not None and "shared_experts" not in name


def is_wo_a(name: str) -> bool:
    return _WO_A.search(name) is not None


def scale_name(weight_name: str) -> str:
    return weight_name[:-len("weight")] + "scale"


# ---------------------------------------------------------------------------------------------- scalar formats
def e8m0_to_f32(s: torch.Tensor) -> torch.Tensor:
    """Power-of-two scales stored as an exponent byte (value 2^(code - 127)); accepts the float8_e8m0fnu dtype, raw
    uint8 codes, or fp32 (returned as is)."""
    if s.dtype == torch.float32:
        return s
    if E8M0 is not None and s.dtype == E8M0:
        s = s.view(torch.uint8)
    assert s.dtype == torch.uint8, s.dtype
    return torch.exp2(s.to(torch.float32) - 127.0)


def f32_to_e8m0(s: torch.Tensor, as_dtype: bool = True) -> Tuple[torch.Tensor, int]:
    """fp32 scales -> exponent bytes, rounding up to the next power of two (a scale may grow, never shrink, so no
    quantised value overflows).  Returns the codes and how many scales were not powers of two already."""
    e = torch.ceil(torch.log2(s.float().clamp_min(2.0 ** -127)))
    inexact = int((torch.exp2(e) != s.float()).sum())
    codes = (e + 127).clamp(0, 254).to(torch.uint8)
    return (codes.view(E8M0) if (as_dtype and E8M0 is not None) else codes), inexact


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    """[rows, cols / 2] bytes -> fp32 [rows, cols]; the low nibble of a byte is the even column."""
    b = packed.view(torch.uint8)
    lut = E2M1.to(b.device)
    return torch.stack([lut[(b & 0xF).long()], lut[(b >> 4).long()]], dim=-1).flatten(-2)


def pack_fp4(x: torch.Tensor) -> torch.Tensor:
    """fp32 values on the e2m1 grid (already divided by their scale) -> packed int8, nearest code, ties to even."""
    a = x.abs()
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=x.device)
    closed = [True, False, True, False, True, False, True]   # tie goes to the code with an even mantissa
    code = torch.zeros_like(a, dtype=torch.uint8)
    for bnd, cr in zip(bounds.tolist(), closed):
        code += ((a > bnd) if cr else (a >= bnd)).to(torch.uint8)
    code |= ((x < 0) | ((x == 0) & torch.signbit(x))).to(torch.uint8) << 3
    return (code[..., 0::2] | (code[..., 1::2] << 4)).view(torch.int8)


def _expand(s: torch.Tensor, rows: int, cols: int, br: int, bc: int) -> torch.Tensor:
    return s.repeat_interleave(br, 0)[:rows].repeat_interleave(bc, 1)[:, :cols]


# ---------------------------------------------------------------------------------------------- tensor conversions
def fp4_dequant(packed: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 value of an fp4 tensor with one scale per 1x32 block."""
    v = unpack_fp4(packed)
    return v * _expand(e8m0_to_f32(scale), v.shape[0], v.shape[1], 1, 32)


def fp8_dequant(w: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 value of an e4m3 tensor with one scale per 128x128 block."""
    return w.float() * _expand(e8m0_to_f32(scale), w.shape[0], w.shape[1], 128, 128)


def fp4_to_fp8(packed: torch.Tensor, scale: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """fp4 (1x32 power-of-two scales) -> e4m3 with one fp32 scale per 128x128 block = the largest 1x32 scale inside.
    Returns (weight, scale, number of elements that were not represented exactly)."""
    v = unpack_fp4(packed)
    rows, cols = v.shape
    s32 = e8m0_to_f32(scale)                                           # [rows, cols / 32]
    nbr, nbc = (rows + 127) // 128, (cols + 127) // 128
    pad = torch.zeros(nbr * 128, nbc * 4, dtype=torch.float32, device=v.device)
    pad[:rows, :s32.shape[1]] = s32
    s128 = pad.view(nbr, 128, nbc, 4).amax(dim=(1, 3))                  # a power of two
    ratio = s32 / _expand(s128, rows, s32.shape[1], 128, 4)             # <= 1, a power of two
    y = v * ratio.repeat_interleave(32, 1)
    q = y.to(torch.float8_e4m3fn)
    return q, s128, int((q.float() != y).sum())


def fp8_to_fp4(w: torch.Tensor, scale: torch.Tensor, as_dtype: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """e4m3 with 128x128 scales -> packed fp4 with one power-of-two scale per 1x32 block (amax / 6 rounded up)."""
    x = fp8_dequant(w, scale)
    rows, cols = x.shape
    blk = x.view(rows, cols // 32, 32)
    s = torch.exp2(torch.ceil(torch.log2(blk.abs().amax(-1).clamp_min(2.0 ** -126) / 6.0)))
    packed = pack_fp4((blk / s[..., None]).clamp(-6.0, 6.0).view(rows, cols))
    codes, _ = f32_to_e8m0(s, as_dtype)
    return packed, codes


def bf16_to_fp8(x: torch.Tensor, pow2: bool = True, as_dtype: bool = True):
    """bf16 -> e4m3 with one scale per 128x128 block (amax / 448; power of two and stored as an exponent byte for the
    published layout)."""
    rows, cols = x.shape
    nbr, nbc = (rows + 127) // 128, (cols + 127) // 128
    pad = torch.zeros(nbr * 128, nbc * 128, dtype=torch.float32, device=x.device)
    pad[:rows, :cols] = x.float().abs()
    s = pad.view(nbr, 128, nbc, 128).amax(dim=(1, 3)).clamp_min(2.0 ** -126) / 448.0
    if pow2:
        s = torch.exp2(torch.ceil(torch.log2(s)))
    q = (x.float() / _expand(s, rows, cols, 128, 128)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    if pow2:
        return q, f32_to_e8m0(s, as_dtype)[0]
    return q, s


# ---------------------------------------------------------------------------------------------- one shard
def convert_tensors(sd: Dict[str, torch.Tensor], direction: str, stats: Optional[dict] = None):
    """Converts the tensors of one shard (a weight and its ``.scale`` always share a shard).  Returns the new dict."""
    stats = stats if stats is not None else {}
    out: Dict[str, torch.Tensor] = {}
    for name, w in sd.items():
        if name.endswith(".scale"):
            continue   # handled with its weight
        sc = sd.get(scale_name(name)) if name.endswith(".weight") else None
        quantised = sc is not None
        if direction == "to_bf16":
            if quantised and w.dtype == torch.int8:
                out[name] = fp4_dequant(w, sc).to(torch.bfloat16)
            elif quantised and w.dtype == torch.float8_e4m3fn:
                out[name] = fp8_dequant(w, sc).to(torch.bfloat16)
            else:
                out[name] = w
        elif direction == "published2fp8":
            if is_expert(name):
                assert quantised and w.dtype == torch.int8, f"{name}: expected packed fp4 with a scale"
                q, s, bad = fp4_to_fp8(w, sc)
                out[name], out[scale_name(name)] = q, s
                stats["inexact_elements"] = stats.get("inexact_elements", 0) + bad
            elif is_wo_a(name):
                assert quantised, f"{name}: expected fp8 with a scale"
                out[name] = fp8_dequant(w, sc).to(torch.bfloat16)      # no scale key in the serving layout
            elif quantised:
                out[name], out[scale_name(name)] = w, e8m0_to_f32(sc)  # bytes unchanged, scale dtype only
            else:
                out[name] = w
        elif direction == "fp82published":
            if is_expert(name):
                assert quantised and w.dtype == torch.float8_e4m3fn, f"{name}: expected fp8 with a scale"
                out[name], out[scale_name(name)] = fp8_to_fp4(w, sc)
            elif is_wo_a(name):
                if w.dtype == torch.bfloat16:
                    out[name], out[scale_name(name)] = bf16_to_fp8(w)
                else:
                    assert quantised, f"{name}: fp8 without a scale"
                    out[name] = w
                    out[scale_name(name)], bad = f32_to_e8m0(sc)
                    stats["rounded_scales"] = stats.get("rounded_scales", 0) + bad
            elif quantised:
                out[name] = w
                out[scale_name(name)], bad = f32_to_e8m0(sc)
                stats["rounded_scales"] = stats.get("rounded_scales", 0) + bad
            else:
                out[name] = w
        else:
            raise ValueError(f"unknown direction {direction!r}")
    return out


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def _rank_world() -> Tuple[int, int]:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def split_by_size(files, world: int):
    """Largest file first onto the least loaded rank; returns one list per rank (deterministic)."""
    loads, parts = [0] * world, [[] for _ in range(world)]
    for f in sorted(files, key=lambda p: (-os.path.getsize(p), p)):
        r = min(range(world), key=lambda i: (loads[i], i))
        parts[r].append(f)
        loads[r] += os.path.getsize(f)
    return parts


def convert_dir(src: str, dst: str, direction: str, device: str = "cpu", wait_s: float = 3600.0) -> dict:
    from safetensors import safe_open
    from safetensors.torch import save_file
    rank, world = _rank_world()
    os.makedirs(dst, exist_ok=True)
    files = sorted(glob.glob(os.path.join(src, "*.safetensors")))
    assert files, f"no safetensors shards in {src}"
    stats: dict = {}
    weight_map, total = {}, 0
    for path in split_by_size(files, world)[rank]:
        sd = {}
        with safe_open(path, framework="pt", device=device) as f:
            for k in f.keys():
                sd[k] = f.get_tensor(k)
        new = convert_tensors(sd, direction, stats)
        base = os.path.basename(path)
        save_file({k: v.contiguous().cpu() for k, v in new.items()}, os.path.join(dst, base))
        for k, v in new.items():
            weight_map[k] = base
            total += _nbytes(v)
    frag = os.path.join(dst, f".index_fragment_{rank}.json")
    with open(frag + ".tmp", "w") as f:
        json.dump({"weight_map": weight_map, "total_size": total, "stats": stats}, f)
    os.replace(frag + ".tmp", frag)
    if rank != 0:
        return stats
    # rank 0: auxiliary files, configuration, merged index
    for p in glob.glob(os.path.join(src, "*")):
        b = os.path.basename(p)
        if os.path.isfile(p) and not b.endswith(".safetensors") and b not in ("model.safetensors.index.json",
                                                                              "config.json"):
            shutil.copy2(p, os.path.join(dst, b))
    cfg_path = os.path.join(src, "config.json")
    if os.path.exists(cfg_path):
        cfg = json.load(open(cfg_path))
        if direction == "fp82published":
            cfg["expert_dtype"] = "fp4"
        else:
            cfg.pop("expert_dtype", None)
        if direction == "to_bf16":
            cfg.pop("quantization_config", None)
        json.dump(cfg, open(os.path.join(dst, "config.json"), "w"), indent=2)
    merged, size, deadline = {}, 0, time.time() + wait_s
    for r in range(world):
        fr = os.path.join(dst, f".index_fragment_{r}.json")
        while not os.path.exists(fr):
            if time.time() > deadline:
                raise TimeoutError(f"rank {r} wrote no index fragment within {wait_s:.0f} s")
            time.sleep(0.2)
        d = json.load(open(fr))
        merged.update(d["weight_map"])
        size += d["total_size"]
        for k, v in d["stats"].items():
            stats[k] = stats.get(k, 0) + v if r else stats.get(k, v)
        os.remove(fr)
    with open(os.path.join(dst, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": size}, "weight_map": dict(sorted(merged.items()))}, f, indent=2)
    return stats


# ---------------------------------------------------------------------------------------------- comparison
def _load_dir(d: str):
    from safetensors import safe_open
    handles = {}
    for path in sorted(glob.glob(os.path.join(d, "*.safetensors"))):
        f = safe_open(path, framework="pt", device="cpu")
        for k in f.keys():
            handles[k] = f
    return handles


def _value(handles, name: str) -> torch.Tensor:
    w = handles[name].get_tensor(name)
    sk = scale_name(name) if name.endswith(".weight") else None
    if sk in handles:
        sc = handles[sk].get_tensor(sk)
        return fp4_dequant(w, sc) if w.dtype == torch.int8 else fp8_dequant(w, sc)
    return w.float() if w.is_floating_point() else w


def compare_dirs(a: str, b: str, atol: float = 0.0) -> dict:
    """Dequantises both checkpoints tensor by tensor (this rank's share of the names, round-robin) and reports names
    on one side only (a bf16 ``wo_a`` has no scale: scale keys without a weight-side partner are not counted), shape
    mismatches and the largest absolute difference."""
    rank, world = _rank_world()
    ha, hb = _load_dir(a), _load_dir(b)
    wa = {k for k in ha if not k.endswith(".scale")}
    wb = {k for k in hb if not k.endswith(".scale")}
    rep = {"only_a": sorted(wa - wb), "only_b": sorted(wb - wa), "shape_mismatch": [], "max_abs_diff": 0.0,
           "worst": None, "different": 0, "compared": 0}
    for name in sorted(wa & wb)[rank::world]:
        va, vb = _value(ha, name), _value(hb, name)
        if va.shape != vb.shape:
            rep["shape_mismatch"].append(name)
            continue
        d = float((va.double() - vb.double()).abs().max()) if va.numel() else 0.0
        rep["compared"] += 1
        if d > atol:
            rep["different"] += 1
        if d > rep["max_abs_diff"]:
            rep["max_abs_diff"], rep["worst"] = d, name
    rep["equal"] = not (rep["only_a"] or rep["only_b"] or rep["shape_mismatch"] or rep["different"])
    return rep


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("convert")
    c.add_argument("--direction", required=True, choices=["published2fp8", "fp82published", "to_bf16"])
    c.add_argument("--src", required=True)
    c.add_argument("--dst", required=True)
    c.add_argument("--device", default="cpu")
    m = sub.add_parser("compare")
    m.add_argument("--a", required=True)
    m.add_argument("--b", required=True)
    m.add_argument("--atol", type=float, default=0.0)
    a = ap.parse_args(argv)
    if a.cmd == "convert":
        stats = convert_dir(a.src, a.dst, a.direction, a.device)
        if _rank_world()[0] == 0:
            print(json.dumps({"direction": a.direction, **stats}))
        return 0
    rep = compare_dirs(a.a, a.b, a.atol)
    print(json.dumps(rep, indent=1))
    return 0 if rep["equal"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
