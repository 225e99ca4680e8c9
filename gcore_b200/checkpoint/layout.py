"""Weight layouts: internal (kernel-friendly) <-> Megatron-Core checkpoint layout <-> HuggingFace.

Megatron side (what mbridge / ``tools/px_ckpt_conv`` produce in the reference, mlm_to_hf.py:61-163,
moe_hf_to_mlm.py:26-244):
  * ``linear_qkv.weight`` rows interleaved per KV group: ``[q_0 .. q_{r-1}, k, v]`` for group 0, then group 1 ...;
  * ``linear_fc1.weight`` = ``cat[gate; up]``; input norms stored as ``linear_qkv.layer_norm_weight`` /
    ``linear_fc1.layer_norm_weight``; embedding / output rows zero-padded to the TP-divisible vocabulary;
  * in a distributed checkpoint the layer index is a prepended axis of the stacked key ``decoder.layers.<rest>``.

``param_chunks`` describes each local parameter as rectangular chunks of a global tensor, which is all the
checkpoint writer / resharding reader need; ``export_full_weights`` gathers TP / EP shards and emits HF names.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..core import parallel_state as ps


@dataclass
class Chunk:
    key: str
    global_shape: Tuple[int, ...]
    offset: Tuple[int, ...]
    tensor: torch.Tensor
    replicated: bool = False  # identical on every TP rank: written once


_LAYER_RE = re.compile(r"^decoder\.layers\.(\d+)\.(.+)$")

_NAME_TO_MCORE = {
    "input_layernorm.weight": "self_attention.linear_qkv.layer_norm_weight",
}


def _mcore_suffix(rest: str, is_moe_layer: bool) -> str:
    if rest == "input_layernorm.weight":
        return "self_attention.linear_qkv.layer_norm_weight"
    if rest == "pre_mlp_layernorm.weight" and not is_moe_layer:
        return "mlp.linear_fc1.layer_norm_weight"
    return rest


def qkv_internal_to_mcore(w: torch.Tensor, hq: int, hk: int, D: int) -> torch.Tensor:
    """rows [Q(hq*D) | K(hk*D) | V(hk*D)] -> per-KV-group interleave.  Works for weights [rows, in] and biases."""
    r = hq // hk
    tail = w.shape[1:]
    q = w[:hq * D].reshape(hk, r * D, *tail)
    k = w[hq * D:(hq + hk) * D].reshape(hk, D, *tail)
    v = w[(hq + hk) * D:].reshape(hk, D, *tail)
    return torch.cat([q, k, v], dim=1).reshape((hq + 2 * hk) * D, *tail)


def qkv_mcore_to_internal(w: torch.Tensor, hq: int, hk: int, D: int) -> torch.Tensor:
    r = hq // hk
    tail = w.shape[1:]
    g = w.reshape(hk, (r + 2) * D, *tail)
    q = g[:, :r * D].reshape(hq * D, *tail)
    k = g[:, r * D:(r + 1) * D].reshape(hk * D, *tail)
    v = g[:, (r + 1) * D:].reshape(hk * D, *tail)
    return torch.cat([q, k, v], dim=0)


def param_chunks(name: str, t: torch.Tensor, cfg, tp_rank: int, tp_size: int, ep_rank: int = 0, ep_size: int = 1,
                 tp_mode: str = "none", num_layers_total: Optional[int] = None) -> List[Chunk]:
    """Chunks of the Megatron-layout global tensor(s) that local parameter ``name`` provides."""
    L = num_layers_total or cfg.num_layers
    m = _LAYER_RE.match(name)
    prefix_shape, prefix_off, key = (), (), name
    is_moe_layer = False
    if m:
        li = int(m.group(1))
        is_moe_layer = cfg.layer_is_moe(li)
        key = "decoder.layers." + _mcore_suffix(m.group(2), is_moe_layer)
        prefix_shape, prefix_off = (L,), (li,)
    D = cfg.head_dim

    def mk(k, gshape, off, ten, rep=False):
        return Chunk(k, prefix_shape + tuple(gshape), prefix_off + tuple(off),
                     ten.unsqueeze(0) if prefix_shape else ten, rep)

    if name.endswith("linear_qkv.weight") or name.endswith("linear_qkv.bias"):
        hq, hk = cfg.num_attention_heads // tp_size, cfg.num_kv_heads // tp_size
        loc = qkv_internal_to_mcore(t, hq, hk, D)
        rows = loc.shape[0]
        return [mk(key, (rows * tp_size,) + tuple(t.shape[1:]), (tp_rank * rows,) + (0,) * (t.dim() - 1), loc)]
    if name.endswith("mlp.linear_fc1.weight") or name.endswith("shared_experts.linear_fc1.weight"):
        tpn = 1 if "shared_experts" in name else tp_size
        tpr = 0 if "shared_experts" in name else tp_rank
        F_l = t.shape[0] // 2
        F = F_l * tpn
        rep = "shared_experts" in name
        return [mk(key, (2 * F, t.shape[1]), (tpr * F_l, 0), t[:F_l], rep),
                mk(key, (2 * F, t.shape[1]), (F + tpr * F_l, 0), t[F_l:], rep)]
    if tp_mode == "expert":
        # [E_local, out, in] -> one key per global expert: experts.linear_fcX.weight{e}
        out = []
        base = key[:-len("weight")]
        for e in range(t.shape[0]):
            ge = ep_rank * t.shape[0] + e
            out.append(mk(f"{base}weight{ge}", tuple(t.shape[1:]), (0,) * (t.dim() - 1), t[e], False))
        return out
    if tp_mode == "column" and tp_size > 1:
        rows = t.shape[0]
        return [mk(key, (rows * tp_size,) + tuple(t.shape[1:]), (tp_rank * rows,) + (0,) * (t.dim() - 1), t)]
    if tp_mode == "row" and tp_size > 1:
        cols = t.shape[1]
        return [mk(key, (t.shape[0], cols * tp_size), (0, tp_rank * cols), t)]
    return [mk(key, tuple(t.shape), (0,) * t.dim(), t, rep=tp_size > 1)]


def assign_from_chunks(name: str, param: torch.Tensor, cfg, tp_rank, tp_size, ep_rank, ep_size, tp_mode, fetch,
                       num_layers_total=None):
    """Inverse of ``param_chunks``: ``fetch(key, global_shape, offset, shape) -> tensor`` reads a region of the
    stored global tensor; the local parameter is rebuilt in internal layout."""
    proto = param_chunks(name, param.detach(), cfg, tp_rank, tp_size, ep_rank, ep_size, tp_mode, num_layers_total)
    pieces = [fetch(c.key, c.global_shape, c.offset, tuple(c.tensor.shape)) for c in proto]
    pieces = [p.squeeze(0) if _LAYER_RE.match(name) else p for p in pieces]
    D = cfg.head_dim
    if name.endswith("linear_qkv.weight") or name.endswith("linear_qkv.bias"):
        hq, hk = cfg.num_attention_heads // tp_size, cfg.num_kv_heads // tp_size
        new = qkv_mcore_to_internal(pieces[0], hq, hk, D)
    elif name.endswith("mlp.linear_fc1.weight") or name.endswith("shared_experts.linear_fc1.weight"):
        new = torch.cat(pieces, 0)
    elif tp_mode == "expert":
        new = torch.stack(pieces, 0)
    else:
        new = pieces[0]
    with torch.no_grad():
        param.copy_(new.to(param.dtype).view_as(param))


# ------------------------------------------------------------------------------------------------ HF names
def _hf_shared(cfg) -> str:
    """HF prefix of the shared expert: ``shared_expert.`` for qwen2_moe, ``shared_experts.`` otherwise."""
    return "shared_expert." if getattr(cfg, "arch", "") == "qwen2_moe" else "shared_experts."


def hf_name_map(cfg) -> Dict[str, str]:
    """internal parameter name pattern -> HF name (``{i}`` layer index, ``{e}`` expert index)."""
    m = {
        "embedding.word_embeddings.weight": "model.embed_tokens.weight",
        "decoder.final_layernorm.weight": "model.norm.weight",
        "output_layer.weight": "lm_head.weight",
        "decoder.layers.{i}.input_layernorm.weight": "model.layers.{i}.input_layernorm.weight",
        "decoder.layers.{i}.pre_mlp_layernorm.weight": "model.layers.{i}.post_attention_layernorm.weight",
        "decoder.layers.{i}.self_attention.linear_proj.weight": "model.layers.{i}.self_attn.o_proj.weight",
        "decoder.layers.{i}.self_attention.q_layernorm.weight": "model.layers.{i}.self_attn.q_norm.weight",
        "decoder.layers.{i}.self_attention.k_layernorm.weight": "model.layers.{i}.self_attn.k_norm.weight",
        "decoder.layers.{i}.self_attention.sinks": "model.layers.{i}.self_attn.sinks",
        "decoder.layers.{i}.mlp.linear_fc2.weight": "model.layers.{i}.mlp.down_proj.weight",
        "decoder.layers.{i}.mlp.router.weight": "model.layers.{i}.mlp.gate.weight",
        "decoder.layers.{i}.mlp.shared_experts.linear_fc2.weight":
            "model.layers.{i}.mlp." + _hf_shared(cfg) + "down_proj.weight",
        "decoder.layers.{i}.mlp.shared_expert_gate.weight": "model.layers.{i}.mlp.shared_expert_gate.weight",
        # MLA
        "decoder.layers.{i}.self_attention.linear_q_down_proj.weight": "model.layers.{i}.self_attn.q_a_proj.weight",
        "decoder.layers.{i}.self_attention.linear_q_up_proj.weight": "model.layers.{i}.self_attn.q_b_proj.weight",
        "decoder.layers.{i}.self_attention.linear_q_proj.weight": "model.layers.{i}.self_attn.q_proj.weight",
        "decoder.layers.{i}.self_attention.linear_kv_down_proj.weight":
            "model.layers.{i}.self_attn.kv_a_proj_with_mqa.weight",
        "decoder.layers.{i}.self_attention.linear_kv_up_proj.weight": "model.layers.{i}.self_attn.kv_b_proj.weight",
        "decoder.layers.{i}.self_attention.kv_layernorm.weight": "model.layers.{i}.self_attn.kv_a_layernorm.weight",
    }
    return m


_MTP_RE = re.compile(r"mtp\.layers\.(\d+)\.(.*)")
_MTP_OWN = {"enorm.weight": "enorm.weight", "hnorm.weight": "hnorm.weight", "eh_proj.weight": "eh_proj.weight",
            "final_layernorm.weight": "shared_head.norm.weight"}


def _mtp_alias(name: str, cfg):
    """Multi-token-prediction blocks are stored the DeepSeek-V3 way, as layers behind the last decoder layer:
    block k's transformer layer under ``model.layers.{L + k}.*`` with the usual names, its own tensors as
    ``enorm`` / ``hnorm`` / ``eh_proj`` / ``shared_head.norm`` of that layer.  Returns ``(name as a decoder-layer
    parameter, None)`` or ``(None, HF key)`` for the block's own tensors; ``(name, None)`` for anything else."""
    m = _MTP_RE.match(name)
    if not m:
        return name, None
    li, rest = cfg.num_layers + int(m.group(1)), m.group(2)
    if rest.startswith("transformer_layer."):
        return f"decoder.layers.{li}." + rest[len("transformer_layer."):], None
    return None, f"model.layers.{li}.{_MTP_OWN[rest]}"


def _gather_tp(t: torch.Tensor, dim: int, group) -> torch.Tensor:
    n = dist.get_world_size(group) if group is not None else 1
    if n == 1:
        return t
    parts = [torch.empty_like(t) for _ in range(n)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim)


def full_hf_tensors(name: str, t: torch.Tensor, cfg, tp_mode: str, tp_group, ep_group=None
                    ) -> Iterator[Tuple[str, torch.Tensor]]:
    """Gathers one local parameter over TP (and EP for experts) and yields its HF-named full tensors."""
    tp = dist.get_world_size(tp_group) if tp_group is not None else 1
    D = cfg.head_dim
    name, own = _mtp_alias(name, cfg)
    if own is not None:
        yield own, t
        return
    m = _LAYER_RE.match(name)
    li = int(m.group(1)) if m else None
    rest = m.group(2) if m else name
    table = hf_name_map(cfg)

    def hf(pattern):
        return table[pattern].replace("{i}", str(li)) if li is not None else table[pattern]

    V = cfg.vocab_size
    if name in ("embedding.word_embeddings.weight", "output_layer.weight"):
        yield table[name], _gather_tp(t, 0, tp_group)[:V]
        return
    if rest in ("self_attention.linear_qkv.weight", "self_attention.linear_qkv.bias"):
        hq, hk = cfg.num_attention_heads // tp, cfg.num_kv_heads // tp
        q, k, v = t.split([hq * D, hk * D, hk * D], 0)
        suf = rest.split(".")[-1]
        for nm, part in (("q_proj", q), ("k_proj", k), ("v_proj", v)):
            yield f"model.layers.{li}.self_attn.{nm}.{suf}", _gather_tp(part, 0, tp_group)
        return
    if rest in ("mlp.linear_fc1.weight", "mlp.shared_experts.linear_fc1.weight"):
        shared = "shared_experts" in rest
        g, u = t.chunk(2, 0)
        pre = f"model.layers.{li}.mlp." + (_hf_shared(cfg) if shared else "")
        grp = None if shared else tp_group
        yield pre + "gate_proj.weight", _gather_tp(g, 0, grp)
        yield pre + "up_proj.weight", _gather_tp(u, 0, grp)
        return
    if tp_mode == "expert":
        ep = dist.get_world_size(ep_group) if ep_group is not None else 1
        full = _gather_tp(t, 0, ep_group) if ep > 1 else t
        for e in range(full.shape[0]):
            if rest.endswith("linear_fc1.weight"):
                g, u = full[e].chunk(2, 0)
                yield f"model.layers.{li}.mlp.experts.{e}.gate_proj.weight", g
                yield f"model.layers.{li}.mlp.experts.{e}.up_proj.weight", u
            else:
                yield f"model.layers.{li}.mlp.experts.{e}.down_proj.weight", full[e]
        return
    pattern = f"decoder.layers.{{i}}.{rest}" if li is not None else name
    if pattern not in table:
        yield name, t
        return
    if tp_mode == "column":
        t = _gather_tp(t, 0, tp_group)
    elif tp_mode == "row":
        t = _gather_tp(t, 1, tp_group)
    yield hf(pattern), t


def export_full_weights(engine, to_hf: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
    model = engine.model
    tp_group = ps.get_tensor_model_parallel_group() if model.tp_size > 1 else None
    ep_group = ps.get_expert_model_parallel_group() if model.ep_size > 1 else None
    modes = {n: getattr(p, "tp_mode", "none") for n, p in model.named_parameters()}
    for name, t in engine.named_local_weights(merged_lora=True):
        yield from full_hf_tensors(name, t, model.cfg, modes[name], tp_group, ep_group)


def load_hf_weights(model, hf_tensors: Dict[str, torch.Tensor], tp_rank: int = 0, ep_rank: int = 0):
    """Fills a (possibly TP / EP sharded) model from a dict of full HF tensors."""
    cfg = model.cfg
    tp, ep = model.tp_size, model.ep_size
    D = cfg.head_dim
    table = hf_name_map(cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if getattr(p, "is_lora", False):
                continue
            name, own = _mtp_alias(name, cfg)
            if own is not None:
                p.copy_(hf_tensors[own])
                continue
            m = _LAYER_RE.match(name)
            li = int(m.group(1)) if m else None
            rest = m.group(2) if m else name
            mode = getattr(p, "tp_mode", "none")
            if name in ("embedding.word_embeddings.weight", "output_layer.weight"):
                src = hf_tensors.get(table[name])
                if src is None and name == "output_layer.weight":
                    src = hf_tensors["model.embed_tokens.weight"]
                full = torch.zeros(p.shape[0] * tp, p.shape[1], dtype=src.dtype)
                full[:src.shape[0]] = src
                p.copy_(full.chunk(tp, 0)[tp_rank])
            elif rest in ("self_attention.linear_qkv.weight", "self_attention.linear_qkv.bias"):
                suf = rest.split(".")[-1]
                parts = [hf_tensors[f"model.layers.{li}.self_attn.{nm}.{suf}"].chunk(tp, 0)[tp_rank]
                         for nm in ("q_proj", "k_proj", "v_proj")]
                p.copy_(torch.cat(parts, 0))
            elif rest in ("mlp.linear_fc1.weight", "mlp.shared_experts.linear_fc1.weight"):
                shared = "shared_experts" in rest
                pre = f"model.layers.{li}.mlp." + (_hf_shared(cfg) if shared else "")
                n, r = (1, 0) if shared else (tp, tp_rank)
                p.copy_(torch.cat([hf_tensors[pre + "gate_proj.weight"].chunk(n, 0)[r],
                                   hf_tensors[pre + "up_proj.weight"].chunk(n, 0)[r]], 0))
            elif mode == "expert":
                E_l = p.shape[0]
                for e in range(E_l):
                    ge = ep_rank * E_l + e
                    pre = f"model.layers.{li}.mlp.experts.{ge}."
                    if rest.endswith("linear_fc1.weight"):
                        p[e].copy_(torch.cat([hf_tensors[pre + "gate_proj.weight"], hf_tensors[pre + "up_proj.weight"]]))
                    else:
                        p[e].copy_(hf_tensors[pre + "down_proj.weight"])
            else:
                pattern = f"decoder.layers.{{i}}.{rest}" if li is not None else name
                key = table[pattern].replace("{i}", str(li)) if li is not None else table[pattern]
                src = hf_tensors[key]
                if mode == "column":
                    src = src.chunk(tp, 0)[tp_rank]
                elif mode == "row":
                    src = src.chunk(tp, 1)[tp_rank]
                p.copy_(src)
