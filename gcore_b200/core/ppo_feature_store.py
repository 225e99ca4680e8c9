"""Per-process key/value store for scalars that outlive a PPO step: running feature means reduced over data-parallel
ranks at interval boundaries, controller state (adaptive entropy), and step-local tensors.  Persisted next to the
checkpoint as ``ppo_feature_store.pt``.  Semantics follow gpatch_v4/core/ppo_feature_store/state.py:67-420 and
reduce.py:18-131.
"""
from __future__ import annotations

import os
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.distributed as dist

_REDUCERS: Dict[str, Callable] = {}


def register_feature_reduce(name: str):
    def deco(fn):
        _REDUCERS[name] = fn
        return fn
    return deco


def _all_reduce(vals: List[float], op, group):
    t = torch.tensor(vals, dtype=torch.float64)
    if dist.is_initialized() and (group is None or dist.get_world_size(group) > 1):
        if dist.get_backend(group) == "nccl":
            t = t.cuda()
        dist.all_reduce(t, op=op, group=group)
    return t.cpu().tolist()


@register_feature_reduce("mean")
def _reduce_mean(value_sum: float, count: float, group=None) -> Optional[float]:
    s, c = _all_reduce([value_sum, count], dist.ReduceOp.SUM, group)
    return s / c if c > 0 else None


@register_feature_reduce("sum")
def _reduce_sum(value_sum: float, count: float, group=None) -> Optional[float]:
    return _all_reduce([value_sum], dist.ReduceOp.SUM, group)[0]


@register_feature_reduce("max")
def _reduce_max(value_sum: float, count: float, group=None) -> Optional[float]:
    return _all_reduce([value_sum if count > 0 else float("-inf")], dist.ReduceOp.MAX, group)[0]


@register_feature_reduce("min")
def _reduce_min(value_sum: float, count: float, group=None) -> Optional[float]:
    return _all_reduce([value_sum if count > 0 else float("inf")], dist.ReduceOp.MIN, group)[0]


class PpoFeatureStore:
    FILE = "ppo_feature_store.pt"

    def __init__(self):
        self._data: Dict[str, Any] = {}
        self._pending: Dict[str, List[float]] = {}   # feature -> [sum, count] of the open interval
        self._reduce: Dict[str, str] = {}
        self._history: Dict[str, List[float]] = {}
        self._axis_step: Dict[str, int] = {}
        self._step_local: Dict[str, torch.Tensor] = {}
        self.enabled = True

    # ---- plain keys (persisted)
    def get(self, key, default=None):
        return self._data.get(key, default)

    def set(self, key, value):
        self._data[key] = value

    def append(self, key, item):
        self._data.setdefault(key, []).append(item)

    def has(self, key):
        return key in self._data

    def keys(self):
        return sorted(self._data)

    def clear(self, key: Optional[str] = None):
        if key is None:
            self._data.clear()
        else:
            self._data.pop(key, None)

    # ---- step-local tensors (never persisted)
    def set_step_local(self, name, value: torch.Tensor):
        self._step_local[name] = value.detach()

    def get_step_local(self, name):
        return self._step_local[name]

    def clear_step_local(self):
        self._step_local.clear()

    # ---- interval features
    def configure(self, feature: str, reduce: str = "mean"):
        assert reduce in _REDUCERS, f"unknown reduce '{reduce}'"
        self._reduce[feature] = reduce

    def begin_ppo_step_interval(self, ppo_step: int):
        for f in list(self._pending):
            self._axis_step[f] = ppo_step
        self._current_step = ppo_step

    def record(self, feature: str, value, weight: float = 1.0):
        v = float(value.detach().float().sum()) if torch.is_tensor(value) else float(value)
        self.record_weighted_sum(feature, v * weight if not torch.is_tensor(value) else v, weight)

    def record_weighted_sum(self, feature: str, value_sum: float, count: float):
        red = self._reduce.get(feature, "mean")
        p = self._pending.setdefault(feature, [0.0, 0.0] if red in ("mean", "sum") else
                                     [float("-inf") if red == "max" else float("inf"), 0.0])
        if red in ("mean", "sum"):
            p[0] += float(value_sum)
        elif red == "max":
            p[0] = max(p[0], float(value_sum))
        else:
            p[0] = min(p[0], float(value_sum))
        p[1] += float(count)
        self._axis_step[feature] = getattr(self, "_current_step", 0)

    def list_pending_features(self):
        return sorted(self._pending)

    def finalize_feature_interval(self, feature: str, group=None) -> Optional[float]:
        s, c = self._pending.pop(feature, [0.0, 0.0])
        out = _REDUCERS[self._reduce.get(feature, "mean")](s, c, group)
        if out is not None:
            self._history.setdefault(feature, []).append(out)
        return out

    def finalize_all_pending_features(self, group=None) -> Dict[str, Optional[float]]:
        feats = self.list_pending_features()
        if dist.is_initialized() and (group is None or dist.get_world_size(group) > 1):
            allf = [None] * dist.get_world_size(group)
            dist.all_gather_object(allf, feats, group=group)  # ranks may have recorded different features
            feats = sorted(set(f for l in allf for f in l))
        return {f: self.finalize_feature_interval(f, group) for f in feats}

    def get_history_mean(self, feature: str) -> Optional[float]:
        h = self._history.get(feature)
        return sum(h) / len(h) if h else None

    def get_feature_axis_step(self, feature: str) -> Optional[int]:
        return self._axis_step.get(feature)

    # ---- persistence
    def state_dict(self):
        return {"data": dict(self._data), "history": {k: list(v) for k, v in self._history.items()},
                "reduce": dict(self._reduce), "axis_step": dict(self._axis_step)}

    def load_state_dict(self, sd):
        self._data = dict(sd.get("data", {}))
        self._history = {k: list(v) for k, v in sd.get("history", {}).items()}
        self._reduce = dict(sd.get("reduce", {}))
        self._axis_step = dict(sd.get("axis_step", {}))
        self._pending.clear()

    def has_persisted_features(self):
        return bool(self._data or self._history)

    def save_to_ckpt(self, iter_dir: str, ppo_step: int):
        os.makedirs(iter_dir, exist_ok=True)
        torch.save({"ppo_step": ppo_step, "state": self.state_dict()}, os.path.join(iter_dir, self.FILE))

    def load_from_ckpt(self, iter_dir: str, ppo_step: int, strict_step: bool = True) -> bool:
        path = os.path.join(iter_dir, self.FILE)
        if not os.path.exists(path):
            return False
        blob = torch.load(path, weights_only=False)
        if strict_step and blob["ppo_step"] != ppo_step:
            raise ValueError(f"feature store was saved at step {blob['ppo_step']}, resuming at {ppo_step}")
        self.load_state_dict(blob["state"])
        return True

    def broadcast(self, group=None, src: int = 0):
        if dist.is_initialized():
            box = [self.state_dict()]
            dist.broadcast_object_list(box, src=src, group=group)
            self.load_state_dict(box[0])


_STORE: Optional[PpoFeatureStore] = None


def get_ppo_feature_store() -> PpoFeatureStore:
    global _STORE
    if _STORE is None:
        _STORE = PpoFeatureStore()
    return _STORE


def reset_ppo_feature_store():
    global _STORE
    _STORE = None


class ppo_step_interval:
    """``with ppo_step_interval(step): ...`` opens the interval on entry and reduces every pending feature on exit."""

    def __init__(self, ppo_step: int, enabled: bool = True, group=None):
        self.step, self.enabled, self.group, self.results = ppo_step, enabled, group, {}

    def __enter__(self):
        if self.enabled:
            get_ppo_feature_store().begin_ppo_step_interval(self.step)
        return self

    def __exit__(self, et, ev, tb):
        if self.enabled and et is None:
            st = get_ppo_feature_store()
            self.results = st.finalize_all_pending_features(self.group)
            st.clear_step_local()
        return False


# ------------------------------------------------------------------------------------------------ adaptive entropy
LAST_WORLD_ENTROPY_KEY = "adaptive_entropy.last_world_entropy"
ENTROPY_COEF_KEY = "adaptive_entropy.coef"


def get_entropy_bonus_coef(ppo_cfg) -> float:
    """Entropy bonus for the coming step: static, or (adaptive) last step's coefficient, applied only while the
    last measured entropy is at or below the target (gpatch_v4/core/adaptive_entropy.py:22-41)."""
    if not getattr(ppo_cfg, "use_adaptive_entropy", False):
        return float(ppo_cfg.ppo_entropy_bonus)
    st = get_ppo_feature_store()
    coef = st.get(ENTROPY_COEF_KEY, None)
    coef = float(ppo_cfg.ppo_entropy_bonus) if coef is None else float(coef)
    return coef if float(st.get(LAST_WORLD_ENTROPY_KEY, float("inf"))) <= float(ppo_cfg.entropy_target) else 0.0


def update_adaptive_entropy(ppo_cfg, world_entropy: float) -> Dict[str, float]:
    """Lag-1 controller: raise the coefficient by ``entropy_coef_delta`` while entropy is below target, lower it
    otherwise, clamped to [entropy_coef_min, entropy_coef_max] (adaptive_entropy.py:44-90)."""
    if not getattr(ppo_cfg, "use_adaptive_entropy", False):
        return {}
    st = get_ppo_feature_store()
    coef = st.get(ENTROPY_COEF_KEY, None)
    coef = float(ppo_cfg.ppo_entropy_bonus) if coef is None else float(coef)
    if float(world_entropy) <= float(ppo_cfg.entropy_target):
        coef = min(coef + float(ppo_cfg.entropy_coef_delta), float(ppo_cfg.entropy_coef_max))
    else:
        coef = max(coef - float(ppo_cfg.entropy_coef_delta), float(ppo_cfg.entropy_coef_min))
    st.set(LAST_WORLD_ENTROPY_KEY, float(world_entropy))
    st.set(ENTROPY_COEF_KEY, coef)
    return {"policy/entropy_coef": coef, "policy/last_world_entropy": float(world_entropy)}
