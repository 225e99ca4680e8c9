"""ctypes bindings for the in-tree native libraries.

``kernels()`` returns the CUDA kernel library (``_gk_kernels.so``) and ``runtime()`` the host C++ runtime
(``_gk_runtime.so``).  On a machine with a GPU a missing kernel library is an error: the GPU code path never
silently degrades to eager PyTorch.  ``GCORE_B200_FORCE_EAGER=1`` selects the PyTorch reference path on purpose
(used for the ``nccl_eager`` baseline backend and for debugging).
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_KERNELS = None
_RUNTIME = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


def force_eager() -> bool:
    return os.environ.get("GCORE_B200_FORCE_EAGER", "0") == "1"


def kernels_available() -> bool:
    return (_HERE / "_gk_kernels.so").exists()


def use_native(t: torch.Tensor | None = None) -> bool:
    """True when the op should run the hand-written sm_100a kernel."""
    if force_eager():
        return False
    if t is not None and not t.is_cuda:
        return False
    if t is None and not torch.cuda.is_available():
        return False
    return True


def kernels() -> ctypes.CDLL:
    global _KERNELS
    if _KERNELS is None:
        path = _HERE / "_gk_kernels.so"
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: run `python -m gcore_b200.build_native` (the GPU path does not fall back "
                "to eager PyTorch)")
        lib = ctypes.CDLL(str(path))
        _declare_kernels(lib)
        st2 = os.environ.get("GCORE_2CTA_STAGES")
        if st2 is not None and hasattr(lib, "gk_gemm_2cta_set_stages"):
            lib.gk_gemm_2cta_set_stages(int(st2))
        gm = os.environ.get("GCORE_GEMM_GROUP_M")      # tile rows per band of the dense GEMMs' tile order (0 = row-fastest)
        if gm is not None and hasattr(lib, "gk_gemm_set_raster"):
            lib.gk_gemm_set_raster(int(gm))
        tsp = os.environ.get("GCORE_WIDE_TAIL_SPLIT")   # 0: the wide GEMM's partial last wave is not split along K
        if tsp is not None and hasattr(lib, "gk_gemm_wide_set_tail_split"):
            lib.gk_gemm_wide_set_tail_split(int(tsp))
        stg = os.environ.get("GCORE_WIDE_STAGED")       # 0: the wide GEMM's epilogue stores rows per thread
        if stg is not None and hasattr(lib, "gk_gemm_wide_set_staged"):
            lib.gk_gemm_wide_set_staged(int(stg))
        pt = os.environ.get("GCORE_PAGED_TARGET_CTAS")  # CTAs the paged decode kernel sizes its KV splits for (444)
        if pt is not None and hasattr(lib, "gk_paged_set_target_ctas"):
            lib.gk_paged_set_target_ctas(int(pt))
        cap = os.environ.get("GCORE_DECODE_SMEM_KB")   # shared-memory budget of decode GEMM CTAs (0 = full ring)
        if cap is not None and hasattr(lib, "gk_gemm_set_decode_smem_cap"):
            lib.gk_gemm_set_decode_smem_cap(int(cap) * 1024)
        _KERNELS = lib
    return _KERNELS


def runtime() -> ctypes.CDLL:
    global _RUNTIME
    if _RUNTIME is None:
        path = _HERE.parent / "runtime" / "_gk_runtime.so"
        if not path.exists():
            from .. import build_native
            build_native.build_runtime()
        lib = ctypes.CDLL(str(path))
        _RUNTIME = lib
    return _RUNTIME


def ptr(t: torch.Tensor | None):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def stream_ptr():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"gcore_b200 native call {what} failed with code {rc}")


_ERR_FLAGS: dict[int, torch.Tensor] = {}


def err_flag(device) -> torch.Tensor:
    """Per-device int32 the kernels write a non-zero code into when a bounded wait expires."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _ERR_FLAGS:
        _ERR_FLAGS[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
    return _ERR_FLAGS[idx]


def check_device_errors(device=None):
    """Synchronising check of the kernel error word; raises if any kernel gave up on a wait."""
    if not torch.cuda.is_available():
        return
    dev = device if device is not None else torch.cuda.current_device()
    idx = torch.device(dev).index if not isinstance(dev, int) else dev
    if idx in _ERR_FLAGS:
        code = int(_ERR_FLAGS[idx].item())
        if code != 0:
            _ERR_FLAGS[idx].zero_()
            raise RuntimeError(f"gcore_b200 kernel reported a timed-out wait (code {code})")


def _declare_kernels(lib: ctypes.CDLL):
    def d(name, argtypes, restype=c_int):
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = argtypes
            fn.restype = restype

    P, I, L, F = c_void_p, c_int, c_ll, c_float
    d("gk_gemm_bf16", [P, L, L, I, P, L, L, I, P, L, I, I, I, P, I, I, F, I, I, I, I, I, I, I, P, I, L, I, P, P, P, P])
    d("gk_gemm_wide", [P, L, L, I, P, L, L, I, P, L, I, I, P, I, F, I, I, I, P, L, P, I, P, P])
    d("gk_gemm_wide_set_tail_split", [I], None)
    d("gk_dsv4_indexer_fwd", [P, P, P, P, P, P, I, I, I, I, F, P])
    d("gk_dsv4_indexer_bwd", [P, P, P, P, P, P, P, P, I, I, I, I, I, F, P])
    d("gk_dsv4_sparse_mqa_fwd", [P, P, P, P, P, P, I, I, I, I, I, F, P])
    d("gk_dsv4_sparse_mqa_bwd", [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, F, P])
    d("gk_hadamard", [P, P, L, I, P])
    d("gk_rope_table", [P, P, P, I, I, I, I, L, I, I, P])
    d("gk_gemm_2cta", [P, L, L, I, P, L, L, I, P, L, I, I, P, I, F, I, I, I, P, P])
    d("gk_gemm_set_decode_smem_cap", [I], None)
    d("gk_gemm_set_raster", [I], None)
    d("gk_gemm_wide_set_staged", [I], None)
    d("gk_gemm_skinny", [P, L, P, L, P, L, I, P, I, I, I, I, I, I, P, P])
    d("gk_gemm_skinny_max_clusters", [I, I, I])
    d("gk_gemm_comm", [I, P, L, P, L, L, I, P, L, P, I, I, I, I, I, I, I, ctypes.c_uint, P, L, P, P])
    d("gk_act_quant_1x128", [P, P, P, P, L, I, I, P])
    d("gk_weight_quant_128x128", [P, P, P, P, I, I, I, P])
    d("gk_fp4_quant_1x32", [P, P, P, P, P, L, P])
    d("gk_gemm_fp8_blockscaled", [P, L, P, L, P, P, P, L, I, I, I, I, P, P])
    d("gk_gemm_fp8_grouped", [P, L, P, L, P, P, P, L, I, I, I, I, P, I, P, P])
    d("gk_zero1_step", [I, P, I, I, L, L, P, P, P, P, F, P, P, F, F, F, F, F, I, I, P])
    d("gk_peer_barrier", [P, I, I, I, ctypes.c_uint, P, P])
    d("gk_peer_barrier_dev", [P, I, I, I, P, P, P])
    d("gk_ep_plan_dev", [P, P, I, I, I, I, I, P, P, P, P, P, P])
    d("gk_ep_plan", [P, P, I, I, I, I, I, ctypes.c_uint, P, P, P, P, P])
    d("gk_ep_push", [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, L, P])
    d("gk_ep_copy_rows", [P, P, P, I, P])
    d("gk_ep_local_plan", [P, I, I, I, P, P, P, P, P, P])
    d("gk_ep_pull", [P, P, P, P, P, I, I, I, I, L, P])
    d("gk_peer_copy_2d", [P, L, P, L, L, I, P])
    d("gk_set_pdl", [I], None)
    d("gk_set_peer_wait_budget", [L], None)
    d("gk_peer_rows", [P, L, I, P, P])
    d("gk_allreduce_oneshot", [P, P, L, I, I, L, P, P, P, P])
    d("gk_allreduce_rmsnorm", [P, P, P, P, P, I, I, F, I, I, L, P, P, P, P])
    d("gk_gemm_splitk_scratch", [I, I, I, I, ctypes.POINTER(L), ctypes.POINTER(L)], None)
    d("gk_rmsnorm_fwd", [P, P, P, P, P, P, I, I, F, P])
    d("gk_rmsnorm_bwd_parts", [I])
    d("gk_rmsnorm_bwd", [P, P, P, P, P, P, P, P, I, I, I, P])
    d("gk_rope", [P, P, I, I, I, I, L, F, I, I, P])
    d("gk_qk_headnorm", [P, P, P, L, I, I, I, L, F, P])
    d("gk_swiglu_fwd", [P, P, L, I, P])
    d("gk_swiglu_fwd_rows", [P, P, L, I, P, P])
    d("gk_swiglu_bwd", [P, P, P, L, I, P])
    d("gk_adam", [P, P, P, P, I, P, L, F, F, F, F, F, I, P, F, P])
    d("gk_sumsq", [P, I, L, P, P])
    d("gk_axpy_cast", [P, I, P, I, L, F, I, P])
    d("gk_logprob_entropy_fwd", [P, I, L, P, F, I, I, L, P, P, P, P, P])
    d("gk_logprob_entropy_combine", [P, I, L, P, P, P, P])
    d("gk_router_fwd", [P, P, P, P, P, L, I, I, I, I, I, I, F, P])
    d("gk_router_bwd", [P, P, P, P, L, I, I, I, I, F, P])
    d("gk_linear_ce_splits", [I, I])
    d("gk_linear_ce_fwd", [P, L, P, L, P, F, I, I, I, I, I, P, P, P])
    d("gk_logprob_entropy_bwd", [P, I, L, P, P, P, P, P, F, I, I, L, P])
    d("gk_sample", [P, I, L, I, I, F, I, P, P, P, P, P, I, I, P])
    d("gk_sample_combine", [P, I, I, P, P, P])
    d("gk_sample_filtered", [P, I, L, I, F, I, F, F, I, P, P, P, P, P, I, P])
    d("gk_grpo_loss", [P, P, P, P, P, L, F, F, F, F, F, F, P, P, P, P])
    d("gk_gae", [P, P, P, P, P, I, I, F, F, P])
    d("gk_kv_append_rope", [P, P, P, P, P, I, I, I, I, I, I, F, I, P])
    d("gk_paged_decode", [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P])
    d("gk_paged_decode_scratch", [I, I, I, I, ctypes.POINTER(L)], None)
    d("gk_paged_decode_append", [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, F, P])
    d("gk_paged_set_target_ctas", [I], None)
    d("gk_mla_paged_decode", [P, L, L, P, L, L, P, P, P, P, L, L, P, I, I, I, I, I, I, I, F, P])
    d("gk_mla_decode_scratch", [I, I, I, I, ctypes.POINTER(L)], None)
    d("gk_mla_decode_supported", [I, I])
    d("gk_mla_set_target_ctas", [I], None)
    d("gk_attn_fwd", [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P, P])
    d("gk_attn_bwd", [P, P, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P, P])
    d("gk_attn_bwd_dv", [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, I, P, P])
