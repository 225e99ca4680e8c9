"""Block-scaled fp8 / fp4 quantisation and the block-scaled fp8 GEMM (``csrc/quant.cu``, ``csrc/gemm_fp8.cu``).

Eager definitions (``*_ref``) are the oracle and the CPU path; they follow the reference's eager quantisers
(gpatch_v4/kernel/quantize/eager_quant_kernels.py:63-233): e4m3 with 1x128 (activations) or 128x128 (weights) blocks,
fp32 or power-of-two scales, e2m1 1x32 with e8m0 scales, and quantise->dequantise round trips for QAT.
"""
from __future__ import annotations


import torch

from . import _lib

E4M3_MAX = 448.0
E2M1_MAX = 6.0
E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
LAUNCHES = {"quant": 0}


def _pow2_ceil(s: torch.Tensor) -> torch.Tensor:
    return torch.exp2(torch.ceil(torch.log2(s)))


def act_quant_1x128_ref(x: torch.Tensor, pow2: bool = False):
    M, K = x.shape
    xb = x.float().view(M, K // 128, 128)
    s = xb.abs().amax(-1).clamp_min(1e-10) / E4M3_MAX
    if pow2:
        s = _pow2_ceil(s)
    q = (xb / s[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(M, K), s


def weight_quant_128x128_ref(w: torch.Tensor, pow2: bool = False):
    N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    wp = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blk = wp.view(nb, 128, kb, 128)
    s = blk.abs().amax(dim=(1, 3)).clamp_min(1e-10) / E4M3_MAX
    if pow2:
        s = _pow2_ceil(s)
    q = (blk / s[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(nb * 128, kb * 128)[:N, :K].contiguous(), s


def dequant_1x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    M, K = q.shape
    return (q.float().view(M, K // 128, 128) * s[..., None]).view(M, K)


def dequant_128x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    return q.float() * s.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]


def fp4_quant_1x32_ref(x: torch.Tensor):
    """Returns (codes uint8 [numel] with sign in bit 3, scale fp32 [numel/32], dequantised fp32)."""
    xf = x.float().reshape(-1, 32)
    s = _pow2_ceil(xf.abs().amax(-1).clamp_min(1e-10) / E2M1_MAX)
    y = (xf / s[:, None]).clamp(-E2M1_MAX, E2M1_MAX)
    vals = E2M1_VALUES.to(x.device)
    a = y.abs()
    # nearest representable, ties to the even code (bounds 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5)
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=x.device)
    closed_right = torch.tensor([True, False, True, False, True, False, True], device=x.device)
    code = torch.zeros_like(a, dtype=torch.int64)
    for b, cr in zip(bounds.tolist(), closed_right.tolist()):
        code += (a > b).long() if cr else (a >= b).long()
    dq = vals[code] * torch.sign(y) * s[:, None]
    codes = (code | ((y < 0).long() << 3)).to(torch.uint8)
    return codes.reshape(-1), s, dq.reshape(x.shape)


# ------------------------------------------------------------------------------------------------ native wrappers
def quant_act_1x128(x: torch.Tensor, pow2: bool = False):
    """x bf16 [M, K] (K % 128 == 0) -> (q float8_e4m3fn [M, K], scales fp32 [M, K/128])."""
    if not (_lib.use_native(x) and x.dtype == torch.bfloat16 and x.is_contiguous()):
        return act_quant_1x128_ref(x, pow2)
    M, K = x.shape
    q = torch.empty(M, K, dtype=torch.uint8, device=x.device)
    s = torch.empty(M, K // 128, dtype=torch.float32, device=x.device)
    LAUNCHES["quant"] += 1
    _lib.check(_lib.kernels().gk_act_quant_1x128(_lib.ptr(x), _lib.ptr(q), _lib.ptr(s), None, M, K, int(pow2),
                                                 _lib.stream_ptr()), "act_quant")
    return q.view(torch.float8_e4m3fn), s


def quant_weight_128x128(w: torch.Tensor, pow2: bool = False):
    if not (_lib.use_native(w) and w.dtype == torch.bfloat16 and w.is_contiguous()):
        return weight_quant_128x128_ref(w, pow2)
    N, K = w.shape
    q = torch.empty(N, K, dtype=torch.uint8, device=w.device)
    s = torch.empty((N + 127) // 128, (K + 127) // 128, dtype=torch.float32, device=w.device)
    LAUNCHES["quant"] += 1
    _lib.check(_lib.kernels().gk_weight_quant_128x128(_lib.ptr(w), _lib.ptr(q), _lib.ptr(s), None, N, K, int(pow2),
                                                      _lib.stream_ptr()), "weight_quant")
    return q.view(torch.float8_e4m3fn), s


def qat_fp8_(x: torch.Tensor, block: str = "1x128", pow2: bool = True) -> torch.Tensor:
    """In-place quantise -> dequantise round trip (fake quant for QAT) on a bf16 tensor."""
    if _lib.use_native(x) and x.dtype == torch.bfloat16 and x.is_contiguous():
        lib = _lib.kernels()
        LAUNCHES["quant"] += 1
        if block == "1x128":
            x2 = x.view(-1, x.shape[-1])
            _lib.check(lib.gk_act_quant_1x128(_lib.ptr(x2), None, None, _lib.ptr(x2), x2.shape[0], x2.shape[1], int(pow2),
                                              _lib.stream_ptr()), "qat_1x128")
        else:
            _lib.check(lib.gk_weight_quant_128x128(_lib.ptr(x), None, None, _lib.ptr(x), x.shape[0], x.shape[1],
                                                   int(pow2), _lib.stream_ptr()), "qat_128x128")
        return x
    if block == "1x128":
        q, s = act_quant_1x128_ref(x.view(-1, x.shape[-1]), pow2)
        x.copy_(dequant_1x128(q, s).view(x.shape).to(x.dtype))
    else:
        q, s = weight_quant_128x128_ref(x, pow2)
        x.copy_(dequant_128x128(q, s).to(x.dtype))
    return x


def quant_fp4_1x32(x: torch.Tensor):
    """bf16 -> (packed uint8 [numel/2] two e2m1 codes per byte, scale_e8m0 uint8 [numel/32], scale fp32)."""
    n = x.numel()
    if not (_lib.use_native(x) and x.dtype == torch.bfloat16 and x.is_contiguous()):
        codes, s, _ = fp4_quant_1x32_ref(x)
        packed = (codes[0::2] | (codes[1::2] << 4)).to(torch.uint8)
        e8 = (torch.log2(s).round().long() + 127).clamp(0, 254).to(torch.uint8)
        return packed, e8, s
    packed = torch.empty(n // 2, dtype=torch.uint8, device=x.device)
    e8 = torch.empty(n // 32, dtype=torch.uint8, device=x.device)
    s = torch.empty(n // 32, dtype=torch.float32, device=x.device)
    LAUNCHES["quant"] += 1
    _lib.check(_lib.kernels().gk_fp4_quant_1x32(_lib.ptr(x), _lib.ptr(packed), _lib.ptr(e8), _lib.ptr(s), None, n,
                                                _lib.stream_ptr()), "fp4_quant")
    return packed, e8, s


def fp4_to_fp8_rebase(packed: torch.Tensor, scale_f32: torch.Tensor, shape):
    """Lossless re-base of fp4 (e2m1 x power-of-two scale) into e4m3 codes with one fp32 scale per 1x128 block
    (deployment format of the reference's ``fp4_qat_then_to_fp8``): every e2m1 value times a power of two is exactly
    representable in e4m3 as long as the four 1x32 scales inside a 128 block differ by at most 2^6."""
    codes = torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(-1).long()
    vals = E2M1_VALUES.to(packed.device)[codes & 7] * torch.where((codes & 8) > 0, -1.0, 1.0)
    x = (vals.view(-1, 32) * scale_f32[:, None]).view(shape)
    M, K = x.shape
    blk = x.view(M, K // 128, 128)
    s128 = scale_f32.view(M, K // 128, 4).amax(-1)  # power of two
    q = (blk / s128[..., None]).to(torch.float8_e4m3fn)
    return q.view(M, K), s128


def gemm_fp8_blockscaled(a_q, a_s, b_q, b_s, out_dtype=torch.bfloat16):
    """``C = dequant(a_q, a_s) @ dequant(b_q, b_s)^T`` with a_q [M,K] (1x128 scales [M,K/128]) and b_q [N,K]
    (128x128 scales)."""
    M, K = a_q.shape
    N = b_q.shape[0]
    if not _lib.use_native(a_q):
        return (dequant_1x128(a_q, a_s) @ dequant_128x128(b_q, b_s).t()).to(out_dtype)
    out = torch.empty(M, N, dtype=out_dtype, device=a_q.device)
    LAUNCHES["quant"] += 1
    a_s, b_s = a_s.contiguous(), b_s.contiguous()   # named: a temporary must outlive the asynchronous launch
    rc = _lib.kernels().gk_gemm_fp8_blockscaled(_lib.ptr(a_q), a_q.stride(0), _lib.ptr(b_q), b_q.stride(0),
                                                _lib.ptr(a_s), _lib.ptr(b_s), _lib.ptr(out),
                                                out.stride(0), int(out_dtype == torch.float32), M, N, K,
                                                _lib.ptr(_lib.err_flag(a_q.device)), _lib.stream_ptr())
    _lib.check(rc, "gemm_fp8_blockscaled")
    return out


def transpose_weight_128x128(q: torch.Tensor, s: torch.Tensor, groups: int = 1):
    """Transposed copy of a 128x128-block-scaled e4m3 weight (``[G * N, K]`` -> ``[G * K, N]``, scales alike): a
    square scale block is its own transpose, so the codes move and no value is re-quantised.  This is the B operand
    of the fp8 data-gradient GEMM ``dX = dY W``."""
    GN, K = q.shape
    N = GN // groups
    assert N % 128 == 0 and K % 128 == 0, (N, K)
    qt = q.view(torch.uint8).view(groups, N, K).transpose(1, 2).contiguous().view(groups * K, N).view(q.dtype)
    st = s.view(groups, N // 128, K // 128).transpose(1, 2).contiguous().view(groups * (K // 128), N // 128)
    return qt, st


def fp8_dgrad(dy: torch.Tensor, cache: dict, out_dtype, offsets=None, groups: int = 1):
    """``dX = dY W`` on the block-fp8 GEMM: dY quantised 1x128 along the output features (the contraction), W taken
    from the forward's e4m3 cache in transposed form (built once per weight version).  With ``offsets`` the grouped
    (per-expert) form."""
    if cache.get("t_ver") != cache["ver"]:
        qt, st = transpose_weight_128x128(cache["q"], cache["s"], groups)
        cache.update(t_ver=cache["ver"], qt=qt, st=st)
    gq, gs = quant_act_1x128(dy.to(torch.bfloat16).contiguous())
    od = out_dtype if out_dtype in (torch.bfloat16, torch.float32) else torch.bfloat16
    if offsets is None:
        return gemm_fp8_blockscaled(gq, gs, cache["qt"], cache["st"], out_dtype=od)
    return gemm_fp8_grouped(gq, gs, cache["qt"], cache["st"], offsets, groups, out_dtype=od)


def fp8_wgrad(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``dW = dY^T X`` (fp32 [N, K]) on the block-fp8 GEMM: the contraction runs over tokens, so dY^T is quantised
    1x128 along tokens and X^T in 128x128 blocks; token counts are padded to a multiple of 128 with zero rows."""
    M = dy.shape[0]
    pad = (-M) % 128
    dyt = torch.nn.functional.pad(dy.to(torch.bfloat16), (0, 0, 0, pad)).t().contiguous()   # [N, M']
    xt = torch.nn.functional.pad(x.to(torch.bfloat16), (0, 0, 0, pad)).t().contiguous()     # [K, M']
    aq, as_ = quant_act_1x128(dyt)
    bq, bs = quant_weight_128x128(xt)
    return gemm_fp8_blockscaled(aq, as_, bq, bs, out_dtype=torch.float32)


def gemm_fp8_grouped(a_q, a_s, b_q, b_s, offsets, num_groups: int, out_dtype=torch.bfloat16):
    """Ragged-M grouped block-fp8 GEMM (experts): rows ``offsets[g]:offsets[g+1]`` of ``a_q`` [R, K] (multiples of
    128; scales ``a_s`` [R, K/128]) multiply group g's weight ``b_q[g * N:(g + 1) * N]`` ([G * N, K] e4m3, 128x128
    scales ``b_s`` [G * N / 128, K / 128]; N a multiple of 128 so that no scale block spans two experts).  Rows of the
    output beyond ``offsets[G]`` are zero."""
    R, K = a_q.shape
    N = b_q.shape[0] // num_groups
    assert N % 128 == 0 and R % 128 == 0, (N, R)
    if not _lib.use_native(a_q) or not hasattr(_lib.kernels(), "gk_gemm_fp8_grouped"):
        a = dequant_1x128(a_q, a_s)
        b = dequant_128x128(b_q, b_s)[:num_groups * N, :K].view(num_groups, N, K)
        out = torch.zeros(R, N, dtype=torch.float32, device=a_q.device)
        off = offsets.tolist()
        for g in range(num_groups):
            if off[g + 1] > off[g]:
                out[off[g]:off[g + 1]] = a[off[g]:off[g + 1]].float() @ b[g].float().t()
        return out.to(out_dtype)
    out = torch.zeros(R, N, dtype=out_dtype, device=a_q.device)
    LAUNCHES["quant"] += 1
    a_s, b_s, offs = a_s.contiguous(), b_s.contiguous(), offsets.int().contiguous()   # named: they must outlive the launch
    rc = _lib.kernels().gk_gemm_fp8_grouped(_lib.ptr(a_q), a_q.stride(0), _lib.ptr(b_q), b_q.stride(0),
                                            _lib.ptr(a_s), _lib.ptr(b_s), _lib.ptr(out),
                                            out.stride(0), int(out_dtype == torch.float32), R, N, K,
                                            _lib.ptr(offs), num_groups,
                                            _lib.ptr(_lib.err_flag(a_q.device)), _lib.stream_ptr())
    _lib.check(rc, "gemm_fp8_grouped")
    return out


class Fp8Linear(torch.nn.Module):
    """Frozen block-fp8 base weight (e4m3 + 128x128 fp32 scales); activations are quantised 1x128 on the fly.  Used
    for the fp8 rollout path and as the frozen base under LoRA."""

    def __init__(self, weight_bf16: torch.Tensor):
        super().__init__()
        q, s = quant_weight_128x128(weight_bf16.contiguous())
        self.register_buffer("weight_q", q)
        self.register_buffer("weight_scale", s)

    def forward(self, x):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        pad = (-x2.shape[1]) % 128
        assert pad == 0, "fp8 linear needs K % 128 == 0"
        aq, as_ = quant_act_1x128(x2)
        y = gemm_fp8_blockscaled(aq, as_, self.weight_q, self.weight_scale, out_dtype=x.dtype
                                 if x.dtype in (torch.bfloat16, torch.float32) else torch.bfloat16)
        return y.reshape(*shp[:-1], self.weight_q.shape[0])
