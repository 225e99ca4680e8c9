"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the moment they call it (a frozen memory pool, a
serving loop that must not trigger a synchronising cudaMalloc, a host application with a fixed memory budget).  For
them ``gk_rmsnorm_bwd_noalloc`` keeps its scratch in a device array built into the library.  This test checks it
against the regular entry point (caller-provided scratch) on two calls in a row, so stale scratch contents from the
first call would show up in the second.  It is collected last on purpose.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gcore_b200", "ops", "_gk_kernels.so")


def _lib():
    lib = ctypes.CDLL(LIB)
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.gk_rmsnorm_bwd_noalloc.argtypes = [P, P, P, P, P, P, P, I, I, I, P]
    lib.gk_rmsnorm_bwd_noalloc.restype = I
    lib.gk_rmsnorm_bwd.argtypes = [P, P, P, P, P, P, P, P, I, I, I, P]
    lib.gk_rmsnorm_bwd.restype = I
    lib.gk_rmsnorm_bwd_parts.argtypes = [I]
    lib.gk_rmsnorm_bwd_parts.restype = I
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _case(lib, T, H, seed, with_res):
    g = torch.Generator(device="cuda").manual_seed(seed)
    gy = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).bfloat16()
    dres = torch.randn(T, H, device="cuda", generator=g).bfloat16() if with_res else None
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # existing entry point: the caller brings the scratch
    parts = lib.gk_rmsnorm_bwd_parts(T)
    scratch = torch.empty(parts * H, dtype=torch.float32, device="cuda")
    dx_ref = torch.empty_like(x)
    dw_ref = torch.empty(H, dtype=torch.float32, device="cuda")
    assert lib.gk_rmsnorm_bwd(_p(gy), _p(x), _p(w), _p(rstd), _p(dres), _p(dx_ref), _p(scratch), _p(dw_ref), 0, T, H,
                              stream) == 0
    # new entry point: every output is allocated before the call, the call itself allocates nothing
    dx = torch.empty_like(x)
    dw = torch.empty(H, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    assert lib.gk_rmsnorm_bwd_noalloc(_p(gy), _p(x), _p(w), _p(rstd), _p(dres), _p(dx), _p(dw), 0, T, H, stream) == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.allclose(dx.float(), dx_ref.float(), rtol=2e-2, atol=2e-2)
    assert torch.allclose(dw, dw_ref, rtol=2e-2, atol=2e-2 * max(1.0, float(dw_ref.abs().max())))
    # and against plain PyTorch fp32 autograd of the same op
    xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    y.backward(gy.float())
    want_dx = xf.grad + (dres.float() if with_res else 0)
    assert (dx.float() - want_dx).abs().max() <= 5e-2 * max(1.0, float(want_dx.abs().max()))
    assert (dw - wf.grad).abs().max() <= 2e-2 * max(1.0, float(wf.grad.abs().max()))


def test_noalloc_rmsnorm_bwd_matches_regular_entry_twice_in_a_row():
    lib = _lib()
    _case(lib, T=777, H=3584, seed=1, with_res=True)   # first call on the device also resolves the scratch address
    _case(lib, T=65, H=256, seed=2, with_res=False)    # smaller shape right after: stale partials must not leak in


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    lib = _lib()
    t = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    rc = lib.gk_rmsnorm_bwd_noalloc(_p(t), _p(t), _p(t), _p(t), None, _p(t), _p(t), 0, 1, 8192 + 8,
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -2
    rc = lib.gk_rmsnorm_bwd_noalloc(_p(t), _p(t), _p(t), _p(t), None, _p(t), _p(t), 0, 1, 12,
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -1
