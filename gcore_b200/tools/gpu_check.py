"""Pre-flight check of the GPUs of one node (the reference's GPU-check tool): for every visible device a short
GEMM compared with a host result, a device-to-device copy bandwidth figure, the peer-access matrix, and whether the
native kernel library loads.  Read-only with respect to GPU settings; short, bounded work only.

    python -m gcore_b200.tools.gpu_check [--json out.json] [--mb 256]
"""
from __future__ import annotations

import argparse
import json

import torch


def check_device(i: int, mb: int = 256) -> dict:
    dev = torch.device("cuda", i)
    props = torch.cuda.get_device_properties(i)
    out = {"index": i, "name": props.name, "sm_count": props.multi_processor_count,
           "memory_gb": round(props.total_memory / 2**30, 1), "capability": f"{props.major}.{props.minor}"}
    g = torch.Generator().manual_seed(i)
    a, b = torch.randn(256, 192, generator=g), torch.randn(192, 128, generator=g)
    ref = a @ b
    got = (a.to(dev).bfloat16() @ b.to(dev).bfloat16()).float().cpu()
    out["gemm_max_err"] = float((got - ref).abs().max())
    out["gemm_ok"] = out["gemm_max_err"] < 0.5
    n = mb * 2**20 // 4
    x = torch.empty(n, dtype=torch.float32, device=dev)
    y = torch.empty_like(x)
    for _ in range(2):
        y.copy_(x)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    s.record(torch.cuda.current_stream(dev))
    for _ in range(5):
        y.copy_(x)
    e.record(torch.cuda.current_stream(dev))
    torch.cuda.synchronize(dev)
    out["copy_gbs"] = round(5 * 2 * n * 4 / (s.elapsed_time(e) * 1e-3) / 1e9, 1)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--mb", type=int, default=256)
    a = ap.parse_args(argv)
    rep = {"cuda_available": torch.cuda.is_available(), "devices": [], "peer_access": [], "native_library": None}
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        for i in range(n):
            with torch.cuda.device(i):
                rep["devices"].append(check_device(i, a.mb))
        rep["peer_access"] = [[bool(i == j or torch.cuda.can_device_access_peer(i, j)) for j in range(n)]
                              for i in range(n)]
        try:
            from ..ops import _lib
            _lib.kernels()
            rep["native_library"] = True
        except Exception as e:  # noqa: BLE001
            rep["native_library"] = f"failed: {e}"
    rep["ok"] = bool(rep["devices"]) and all(d["gemm_ok"] for d in rep["devices"]) and rep["native_library"] is True
    print(json.dumps(rep, indent=1))
    if a.json:
        json.dump(rep, open(a.json, "w"), indent=1)
    return rep


if __name__ == "__main__":
    main()
