"""Vocabulary-axis ops: fused linear + log-prob + entropy (never materialises ``[T, V]``), and token sampling.

``linear_logprob_entropy(hidden, weight, targets, temperature, tp_group)`` has the contract of the reference's
``linear_cross_entropy`` (gpatch_v4/kernel/__init__.py:38; Triton kernels gpatch_v4/kernel/triton/
linear_ce_kernels.py:159-1644): ``logp[t] = log softmax(h_t W^T / temperature)[target_t]`` plus the entropy of that
distribution, with ``weight`` optionally sharded over the vocabulary across a tensor-parallel group.

Forward: one kernel (``csrc/linear_ce.cu``) runs the vocabulary GEMM on the tensor cores and folds every finished
256-column tile into per-row (max, sum-exp, sum p*z, target logit) in its epilogue; only ``[splits, T, 4]`` floats
reach memory, and a merge kernel turns them (and, with TP, the all-gathered partials of every rank) into log-prob,
entropy and log-sum-exp.  ``GCORE_FUSED_LINEAR_CE=0`` selects the older chunked form (logits of 4096 tokens at a
time through the plain GEMM, one reduction pass, discard).  Backward recomputes each chunk's logits, overwrites them
with d(logits) in place and feeds the dgrad / wgrad GEMMs.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

import os

from . import _lib
from .gemm import gemm, linear_dgrad, linear_forward, linear_wgrad

LAUNCHES = {"vocab": 0}
CHUNK_TOKENS = 4096
FUSED_FWD = {"enabled": os.environ.get("GCORE_FUSED_LINEAR_CE", "1") != "0"}


def _fused_ok(hidden, weight):
    return (FUSED_FWD["enabled"] and hasattr(_lib.kernels(), "gk_linear_ce_fwd") and weight.dtype == torch.bfloat16
            and hidden.stride(1) == 1 and weight.stride(1) == 1 and hidden.stride(0) % 8 == 0
            and weight.stride(0) % 8 == 0 and hidden.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def fused_linear_stats(hidden, weight, targets, inv_temp, vocab_start):
    """Partials ``[splits, T, 4]`` = (max, sum exp, sum exp * z, target z or -FLT_MAX) of ``hidden @ weight.T *
    inv_temp`` per row and vocabulary split, without the logits."""
    T, K = hidden.shape
    V = weight.shape[0]
    lib = _lib.kernels()
    splits = lib.gk_linear_ce_splits(T, V)
    part = torch.empty(splits, T, 4, dtype=torch.float32, device=hidden.device)
    LAUNCHES["vocab"] += 1
    _lib.check(lib.gk_linear_ce_fwd(_lib.ptr(hidden), hidden.stride(0), _lib.ptr(weight), weight.stride(0),
                                    _lib.ptr(targets), inv_temp, vocab_start, T, V, K, splits, _lib.ptr(part),
                                    _lib.ptr(_lib.err_flag(hidden.device)), _lib.stream_ptr()), "linear_ce_fwd")
    return part


def logprob_entropy_ref(logits, targets, temperature=1.0):
    z = logits.float() / temperature
    lse = torch.logsumexp(z, -1)
    logp = z.gather(-1, targets[:, None]).squeeze(-1) - lse
    p = torch.softmax(z, -1)
    ent = lse - (p * z).sum(-1)
    return logp, ent


def _chunk_stats(logits, targets, inv_temp, vocab_start, partial: bool):
    T, V = logits.shape
    dev = logits.device
    if partial:
        out = torch.empty(T, 4, dtype=torch.float32, device=dev)
        LAUNCHES["vocab"] += 1
        _lib.check(_lib.kernels().gk_logprob_entropy_fwd(
            _lib.ptr(logits), int(logits.dtype == torch.float32), logits.stride(0), _lib.ptr(targets), inv_temp,
            vocab_start, V, T, None, None, None, _lib.ptr(out), _lib.stream_ptr()), "logprob_entropy_fwd")
        return out
    logp = torch.empty(T, dtype=torch.float32, device=dev)
    ent = torch.empty(T, dtype=torch.float32, device=dev)
    lse = torch.empty(T, dtype=torch.float32, device=dev)
    LAUNCHES["vocab"] += 1
    _lib.check(_lib.kernels().gk_logprob_entropy_fwd(
        _lib.ptr(logits), int(logits.dtype == torch.float32), logits.stride(0), _lib.ptr(targets), inv_temp,
        vocab_start, V, T, _lib.ptr(logp), _lib.ptr(ent), _lib.ptr(lse), None, _lib.stream_ptr()),
        "logprob_entropy_fwd")
    return logp, ent, lse


def _combine(partials, T):
    R = partials.shape[0]
    dev = partials.device
    logp = torch.empty(T, dtype=torch.float32, device=dev)
    ent = torch.empty(T, dtype=torch.float32, device=dev)
    lse = torch.empty(T, dtype=torch.float32, device=dev)
    LAUNCHES["vocab"] += 1
    _lib.check(_lib.kernels().gk_logprob_entropy_combine(_lib.ptr(partials), R, T, _lib.ptr(logp), _lib.ptr(ent),
                                                         _lib.ptr(lse), _lib.stream_ptr()), "combine")
    return logp, ent, lse


class _LinearLogprobFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, temperature, tp_group, vocab_start, main_grad, want_entropy):
        T, H = hidden.shape
        inv_temp = 1.0 / float(temperature)
        tp = dist.get_world_size(tp_group) if tp_group is not None else 1
        logp = torch.empty(T, dtype=torch.float32, device=hidden.device)
        ent = torch.empty(T, dtype=torch.float32, device=hidden.device)
        lse = torch.empty(T, dtype=torch.float32, device=hidden.device)
        fused = _fused_ok(hidden, weight)
        if fused:
            part = fused_linear_stats(hidden, weight, targets, inv_temp, vocab_start)
            if tp > 1:
                allp = torch.empty(tp * part.shape[0], T, 4, dtype=torch.float32, device=hidden.device)
                dist.all_gather_into_tensor(allp, part, group=tp_group)
                part = allp
            logp, ent, lse = _combine(part, T)
        for s in range(0, T if not fused else 0, CHUNK_TOKENS):
            e = min(T, s + CHUNK_TOKENS)
            logits = linear_forward(hidden[s:e], weight)
            if tp > 1:
                part = _chunk_stats(logits, targets[s:e], inv_temp, vocab_start, True)
                allp = torch.empty(tp, e - s, 4, dtype=torch.float32, device=hidden.device)
                dist.all_gather_into_tensor(allp, part, group=tp_group)
                lp, en, ls = _combine(allp, e - s)
            else:
                lp, en, ls = _chunk_stats(logits, targets[s:e], inv_temp, vocab_start, False)
            logp[s:e], ent[s:e], lse[s:e] = lp, en, ls
            del logits
        ctx.save_for_backward(hidden, weight, targets, lse, ent)
        ctx.cfg = (inv_temp, tp_group, vocab_start, main_grad, want_entropy)
        return logp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        hidden, weight, targets, lse, ent = ctx.saved_tensors
        inv_temp, tp_group, vocab_start, main_grad, want_entropy = ctx.cfg
        T, H = hidden.shape
        V = weight.shape[0]
        g_lp = g_lp.contiguous().float()
        use_ent = want_entropy and g_ent is not None
        g_ent = g_ent.contiguous().float() if use_ent else None
        d_hidden = torch.empty_like(hidden)
        dw = None
        if main_grad is None and ctx.needs_input_grad[1]:
            dw = torch.zeros(V, H, dtype=torch.float32, device=hidden.device)
        acc_target = main_grad if main_grad is not None else dw
        lib = _lib.kernels()
        for s in range(0, T, CHUNK_TOKENS):
            e = min(T, s + CHUNK_TOKENS)
            logits = linear_forward(hidden[s:e], weight)
            LAUNCHES["vocab"] += 1
            _lib.check(lib.gk_logprob_entropy_bwd(
                _lib.ptr(logits), 0, logits.stride(0), _lib.ptr(targets[s:e]), _lib.ptr(lse[s:e]),
                _lib.ptr(ent[s:e]), _lib.ptr(g_lp[s:e]), _lib.ptr(g_ent[s:e]) if use_ent else None, inv_temp,
                vocab_start, V, e - s, _lib.stream_ptr()), "logprob_entropy_bwd")
            linear_dgrad(logits, weight, out=d_hidden[s:e])
            if acc_target is not None:
                linear_wgrad(logits, hidden[s:e], out=acc_target, accumulate=True)
            del logits
        if tp_group is not None and dist.get_world_size(tp_group) > 1:
            dist.all_reduce(d_hidden, group=tp_group)
        return d_hidden, (dw.to(weight.dtype) if dw is not None else None), None, None, None, None, None, None


def linear_logprob_entropy(hidden, weight, targets, temperature=1.0, tp_group=None, vocab_start=0, main_grad=None,
                           want_entropy=True):
    """Returns ``(logp[T], entropy[T])`` in fp32.  ``hidden`` [T,H] bf16, ``weight`` [V_local,H] bf16, ``targets`` [T]
    int64 global vocabulary ids.  Differentiable w.r.t. ``hidden`` and ``weight``."""
    if hidden.dtype == torch.bfloat16 and _lib.use_native(hidden):
        return _LinearLogprobFn.apply(hidden.contiguous(), weight, targets.contiguous(), temperature, tp_group,
                                      vocab_start, main_grad, want_entropy)
    # eager path (CPU oracle / nccl_eager baseline): chunked, vocab-parallel aware
    T = hidden.shape[0]
    outs_lp, outs_en = [], []
    tp = dist.get_world_size(tp_group) if tp_group is not None else 1
    for s in range(0, T, CHUNK_TOKENS):
        e = min(T, s + CHUNK_TOKENS)
        z = torch.nn.functional.linear(hidden[s:e], weight).float() / temperature
        if tp > 1:
            from ..parallel.tp_ops import vocab_parallel_logprob_entropy
            lp, en = vocab_parallel_logprob_entropy(z, targets[s:e], vocab_start, tp_group)
        else:
            lse = torch.logsumexp(z, -1)
            lp = z.gather(-1, targets[s:e, None]).squeeze(-1) - lse
            p = torch.softmax(z, -1)
            en = lse - (p * z).sum(-1)
        outs_lp.append(lp)
        outs_en.append(en)
    return torch.cat(outs_lp), torch.cat(outs_en)


# ---------------------------------------------------------------------------------------------- sampling
def sample_ref(logits, temperature, seeds, steps, greedy=False):
    z = logits.float() / max(temperature, 1e-6)
    if greedy:
        tok = z.argmax(-1)
    else:
        toks = []
        for b in range(z.shape[0]):
            g = torch.Generator(device="cpu")
            g.manual_seed(int(seeds[b]) * 1000003 + int(steps[b]))
            u = torch.rand(z.shape[1], generator=g).clamp_min(1e-20).to(z.device)
            toks.append((z[b] - torch.log(-torch.log(u) + 1e-20)).argmax())
        tok = torch.stack(toks)
    lp = torch.log_softmax(z, -1).gather(-1, tok[:, None]).squeeze(-1)
    return tok, lp


_LIB_RNG = {"seeded": False}


def _sample_library(logits, temperature, greedy, tp_group):
    """Library sampling on a GPU (the eager baseline backend): vocabulary shards are gathered, then Gumbel-max from
    the device's default generator (which CUDA graphs can capture), seeded alike on every rank at first use so that
    tensor-parallel ranks draw the same tokens; per-request seeds are a property of the native sampler only."""
    if tp_group is not None and dist.get_world_size(tp_group) > 1:
        parts = [torch.empty_like(logits) for _ in range(dist.get_world_size(tp_group))]
        dist.all_gather(parts, logits.contiguous(), group=tp_group)
        logits = torch.cat(parts, dim=1)
    z = logits.float() / max(float(temperature), 1e-6)
    if greedy:
        tok = z.argmax(-1)
    else:
        if not _LIB_RNG["seeded"] and not torch.cuda.is_current_stream_capturing():
            torch.cuda.manual_seed(20240229)
            _LIB_RNG["seeded"] = True
        u = torch.rand(z.shape, device=z.device).clamp_min_(1e-20)
        tok = (z - torch.log(-torch.log(u) + 1e-20)).argmax(-1)
    lp = torch.log_softmax(z, -1).gather(-1, tok[:, None]).squeeze(-1)
    return tok, lp


def sample(logits, temperature, seeds, steps, greedy=False, tp_group=None, vocab_start=0):
    """Draws one token per row from ``softmax(logits / temperature)`` (Gumbel-max) and returns
    ``(tokens int64 [B], logp fp32 [B])``.  ``seeds`` int64 [B], ``steps`` int32 [B] select the random stream; the
    draw for a given (seed, step, token id) is independent of batching and of the vocabulary sharding."""
    B, V = logits.shape
    if not (_lib.use_native(logits) and logits.dtype in (torch.bfloat16, torch.float32)):
        if logits.is_cuda:
            return _sample_library(logits, temperature, greedy, tp_group)
        return sample_ref(logits, temperature, seeds, steps, greedy)
    inv_temp = 1.0 / max(float(temperature), 1e-6)
    tokens = torch.empty(B, dtype=torch.int64, device=logits.device)
    logp = torch.empty(B, dtype=torch.float32, device=logits.device)
    lib = _lib.kernels()
    tp = dist.get_world_size(tp_group) if tp_group is not None else 1
    # a row of a large vocabulary is shared by several CTAs (the random stream is evaluated per element: one CTA per
    # row leaves most of the GPU idle at decode batch sizes); their partials merge like tensor-parallel shards
    slices = max(1, min(8, 592 // max(B, 1))) if V >= 16384 else 1
    LAUNCHES["vocab"] += 1
    if tp == 1 and slices == 1:
        _lib.check(lib.gk_sample(_lib.ptr(logits), int(logits.dtype == torch.float32), logits.stride(0), V, vocab_start,
                                 inv_temp, int(greedy), _lib.ptr(seeds), _lib.ptr(steps), _lib.ptr(tokens),
                                 _lib.ptr(logp), None, B, 1, _lib.stream_ptr()), "sample")
        return tokens, logp
    part = torch.empty(slices, B, 6, dtype=torch.float32, device=logits.device)
    _lib.check(lib.gk_sample(_lib.ptr(logits), int(logits.dtype == torch.float32), logits.stride(0), V, vocab_start,
                             inv_temp, int(greedy), _lib.ptr(seeds), _lib.ptr(steps), None, None, _lib.ptr(part), B,
                             slices, _lib.stream_ptr()), "sample")
    if tp > 1:
        allp = torch.empty(tp * slices, B, 6, dtype=torch.float32, device=logits.device)
        dist.all_gather_into_tensor(allp, part, group=tp_group)
        part = allp
    LAUNCHES["vocab"] += 1
    _lib.check(lib.gk_sample_combine(_lib.ptr(part), part.shape[0], B, _lib.ptr(tokens), _lib.ptr(logp),
                                     _lib.stream_ptr()), "sample_combine")
    return tokens, logp


def sample_filtered(logits, temperature, top_k, top_p, min_p, seeds, steps, greedy=False, return_kept=False):
    """Top-k / top-p / min-p sampling over whole-vocabulary ``logits`` [B, V]: one kernel finds the cut by radix
    selection over counts and probability mass (no sort) and draws with the sampler's counter-based random stream.
    Returns ``(tokens, logp)`` with ``logp`` under the renormalised filtered distribution (the definition:
    ``sample(apply_top_k_top_p(logits / temperature, ...), 1.0, ...)``)."""
    B, V = logits.shape
    if not (_lib.use_native(logits) and logits.dtype in (torch.bfloat16, torch.float32) and logits.stride(1) == 1
            and hasattr(_lib.kernels(), "gk_sample_filtered")):
        z = apply_top_k_top_p(logits / max(float(temperature), 1e-6), top_k, top_p, min_p)
        out = sample(z.contiguous(), 1.0, seeds, steps, greedy)
        return (*out, torch.isfinite(z).sum(-1).int()) if return_kept else out
    tokens = torch.empty(B, dtype=torch.int64, device=logits.device)
    logp = torch.empty(B, dtype=torch.float32, device=logits.device)
    kept = torch.empty(B, dtype=torch.int32, device=logits.device) if return_kept else None
    LAUNCHES["vocab"] += 1
    _lib.check(_lib.kernels().gk_sample_filtered(
        _lib.ptr(logits), int(logits.dtype == torch.float32), logits.stride(0), V, 1.0 / max(float(temperature), 1e-6),
        int(top_k or 0), float(top_p), float(min_p), int(greedy), _lib.ptr(seeds), _lib.ptr(steps), _lib.ptr(tokens),
        _lib.ptr(logp), _lib.ptr(kept), B, _lib.stream_ptr()), "sample_filtered")
    return (tokens, logp, kept) if return_kept else (tokens, logp)


def apply_top_k_top_p(logits, top_k=0, top_p=1.0, min_p=0.0):
    """Masks logits outside the top-k / nucleus / min-p set with -inf (sort based; only used when a request asks
    for it, the default rollout configuration samples from the full distribution)."""
    z = logits.float()
    if top_k and top_k > 0 and top_k < z.shape[-1]:
        kth = torch.topk(z, top_k, dim=-1).values[..., -1:]
        z = z.masked_fill(z < kth, float("-inf"))
    if top_p < 1.0:
        sz, idx = torch.sort(z, dim=-1, descending=True)
        probs = torch.softmax(sz, -1)
        cum = probs.cumsum(-1)
        drop = cum - probs > top_p
        sz = sz.masked_fill(drop, float("-inf"))
        z = torch.full_like(z, float("-inf")).scatter(-1, idx, sz)
    if min_p > 0.0:
        p = torch.softmax(z, -1)
        z = z.masked_fill(p < min_p * p.max(-1, keepdim=True).values, float("-inf"))
    return z
