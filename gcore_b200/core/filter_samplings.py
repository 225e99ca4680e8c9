"""Filter-sampling strategies: which of the ``sampling_repeat_n`` responses of a prompt reach training.

Two registries, as in the reference (gpatch_v4/utils/filter_samplings.py:10-260): group-level strategies over
per-prompt rollout batches (``all``, ``test``, ``best-and-worst``) and sample-level strategies over flat sample
lists grouped by ``group_id`` (``best-and-worst``, ``sample-mask``, ``valid_group``), plus user functions loaded from
a python file.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, Dict, List

import torch

from ..configs.base import import_from_path

_GROUP: Dict[str, Callable] = {}
_SAMPLE: Dict[str, Callable] = {}


def register_group_filter(name):
    def deco(fn):
        _GROUP[name] = fn
        return fn
    return deco


def register_sample_filter(name):
    def deco(fn):
        _SAMPLE[name] = fn
        return fn
    return deco


def get_group_filter(name: str) -> Callable:
    if name not in _GROUP:
        raise KeyError(f"unknown filter sampling strategy '{name}' (available: {sorted(_GROUP)})")
    return _GROUP[name]


def register_custom_filter_sampling(name: str, py_path: str, fn_name: str = "ppo_filter_samplings"):
    _GROUP[name] = import_from_path(py_path, fn_name)


def _scalar(v) -> float:
    return float(v.reshape(-1)[0]) if torch.is_tensor(v) else float(v)


@register_group_filter("all")
def keep_all(config, groups: List[List[dict]], repeat_n: int, keep_n: int):
    return groups


@register_group_filter("test")
def truncated(config, groups, repeat_n, keep_n):
    return [g[:keep_n] for g in groups]


@register_group_filter("best-and-worst")
def best_and_worst(config, groups, repeat_n, keep_n):
    assert keep_n == 2, "sampling_keep_n must be 2 for the best-and-worst strategy"
    out = []
    for g in groups:
        r = [_scalar(s["rewards"] if "rewards" in s else s["reward"]) for s in g]
        hi, lo = max(range(len(g)), key=r.__getitem__), min(range(len(g)), key=r.__getitem__)
        out.append([g[hi], g[lo]])
    return out


def group_samples(samples: List[dict]) -> "OrderedDict":
    groups: "OrderedDict" = OrderedDict()
    for s in samples:
        groups.setdefault(s.get("group_id", s.get("prompt_id", 0)), []).append(s)
    return groups


@register_sample_filter("best-and-worst")
def filter_best_and_worst(config, samples):
    out = []
    for g in group_samples(samples).values():
        if len(g) < 2:
            out += g
            continue
        order = sorted(g, key=lambda s: _scalar(s.get("rewards", s.get("reward", 0.0))))
        out += [order[0], order[-1]]
    return out


@register_sample_filter("sample-mask")
def filter_sample_mask(config, samples):
    return [s for s in samples if bool(_scalar(s.get("sample_mask", 1.0)))]


@register_sample_filter("valid_group")
def filter_valid_group(config, samples):
    out = []
    for g in group_samples(samples).values():
        if len(g) >= 2:
            out += g
    return out


def filter_rollout_samples(config, samples: List[dict], strategies: List[str]) -> List[dict]:
    """Applies the sample-level strategies in order."""
    for name in strategies:
        if name not in _SAMPLE:
            raise KeyError(f"unknown sample filter '{name}' (available: {sorted(_SAMPLE)})")
        samples = _SAMPLE[name](config, samples)
    return samples
