"""Operator registry: op name -> implementation, resolved once per process.

The reference dispatches per device family (cuda / mlu / npu / xpu packages registered under a device name,
gpatch_v4/kernel/registry.py:42-173, gpatch_v4/core/device/protocol.py:7-109).  This framework has one target, so the
registry keeps only what is useful on it: two implementations per op, ``native`` (the sm_100a kernel) and ``eager``
(the PyTorch definition used on CPU, as the test oracle and as the ``nccl_eager`` baseline backend), plus user
overrides.  ``resolve(name)`` returns the native one when a GPU and the kernel library are present.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

from . import _lib

_REGISTRY: Dict[str, Dict[str, Callable]] = {}


def register(name: str, impl: str = "native"):
    def deco(fn):
        _REGISTRY.setdefault(name, {})[impl] = fn
        return fn
    return deco


def register_fn(name: str, fn: Callable, impl: str = "native"):
    _REGISTRY.setdefault(name, {})[impl] = fn


def available(name: Optional[str] = None):
    if name is None:
        return sorted(_REGISTRY)
    return sorted(_REGISTRY.get(name, {}))


def resolve(name: str, impl: Optional[str] = None) -> Callable:
    impls = _REGISTRY.get(name)
    if not impls:
        raise KeyError(f"no operator named '{name}' (registered: {sorted(_REGISTRY)})")
    if impl is None:
        impl = "override" if "override" in impls else ("native" if _lib.use_native() and "native" in impls else "eager")
    if impl not in impls:
        raise KeyError(f"operator '{name}' has no '{impl}' implementation (has: {sorted(impls)})")
    return impls[impl]


def _populate():
    from . import attention, fused, gemm, optim, quant, rl, vocab
    for mod, names in ((gemm, ("gemm", "grouped_gemm", "grouped_wgrad", "linear")),
                       (fused, ("rmsnorm", "rope", "swiglu")),
                       (attention, ("flash_attn_varlen", "flash_attn_qkvpacked", "paged_decode", "kv_append_rope")),
                       (vocab, ("linear_logprob_entropy", "sample")),
                       (optim, ("adam_step", "sumsq", "axpy_cast")),
                       (quant, ("quant_act_1x128", "quant_weight_128x128", "quant_fp4_1x32", "gemm_fp8_blockscaled")),
                       (rl, ("fused_grpo_loss", "gae"))):
        for n in names:
            fn = getattr(mod, n, None)
            if fn is not None:
                register_fn(n, fn, "native")
    for n, fn in (("rmsnorm", getattr(fused, "rmsnorm_ref", None)), ("rope", getattr(fused, "rope_ref", None)),
                  ("swiglu", getattr(fused, "swiglu_ref", None)),
                  ("flash_attn_varlen", getattr(attention, "attn_varlen_ref", None)),
                  ("quant_act_1x128", quant.act_quant_1x128_ref), ("quant_weight_128x128", quant.weight_quant_128x128_ref)):
        if fn is not None:
            register_fn(n, fn, "eager")


_populate()
