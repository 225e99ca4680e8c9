"""Config plumbing: YAML files + dotted command-line overrides merged onto a tree of dataclasses.

Replaces the Hydra/OmegaConf layer of the reference (``merge_hydra_config``, gpatch_v4/configs/utils.py:28-77) with a
dependency-free loader that keeps its surface: ``key.sub=value`` overrides, ``+key=value`` to add free-form keys,
``~key`` to delete, list-of-dataclass fields, ``__post_init__`` validation executed exactly once per node (children
first), and mapping-style access (``cfg["a"]``, ``cfg.get("a")``) like the reference's ``MappingProtocol``.
"""
from __future__ import annotations

import copy
import dataclasses
import typing
from dataclasses import dataclass, field, fields, is_dataclass
from typing import Any, get_args, get_origin, get_type_hints

import yaml


class ConfigError(ValueError):
    pass


class MappingMixin:
    """dict-like read access for dataclass configs."""

    def __getitem__(self, k):
        return getattr(self, k)

    def __contains__(self, k):
        return hasattr(self, k)

    def get(self, k, default=None):
        return getattr(self, k, default)

    def keys(self):
        return [f.name for f in fields(self)]

    def items(self):
        return [(f.name, getattr(self, f.name)) for f in fields(self)]

    def to_dict(self):
        return to_dict(self)


def to_dict(obj):
    if is_dataclass(obj):
        return {f.name: to_dict(getattr(obj, f.name)) for f in fields(obj)}
    if isinstance(obj, dict):
        return {k: to_dict(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [to_dict(v) for v in obj]
    return obj


def _parse_scalar(text: str):
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def apply_overrides(tree: dict, overrides: list[str]) -> dict:
    """Applies ``a.b.c=value`` / ``+a.b=value`` / ``~a.b`` overrides to a nested dict (lists indexable by int)."""
    tree = copy.deepcopy(tree)
    for ov in overrides or []:
        ov = ov.strip()
        if not ov:
            continue
        delete = ov.startswith("~")
        ov = ov.lstrip("+~")
        if delete:
            path, value = ov, None
        else:
            if "=" not in ov:
                raise ConfigError(f"override '{ov}' is not of the form key=value")
            path, text = ov.split("=", 1)
            value = _parse_scalar(text)
        keys = path.split(".")
        node = tree
        for k in keys[:-1]:
            if isinstance(node, list):
                node = node[int(k)]
            else:
                if k not in node or node[k] is None:
                    node[k] = {}
                node = node[k]
        last = keys[-1]
        if delete:
            if isinstance(node, dict):
                node.pop(last, None)
        elif isinstance(node, list):
            node[int(last)] = value
        else:
            node[last] = value
    return tree


def _strip_optional(tp):
    if get_origin(tp) is typing.Union or str(get_origin(tp)) == "<class 'types.UnionType'>":
        args = [a for a in get_args(tp) if a is not type(None)]
        if len(args) == 1:
            return args[0]
    return tp


def _build(tp, value, path):
    tp = _strip_optional(tp)
    if value is None:
        return None
    if is_dataclass(tp):
        if is_dataclass(value):
            return value
        if not isinstance(value, dict):
            raise ConfigError(f"{path}: expected a mapping for {tp.__name__}, got {type(value).__name__}")
        return from_dict(tp, value, path)
    origin = get_origin(tp)
    if origin in (list, typing.List):
        (inner,) = get_args(tp) or (Any,)
        if isinstance(value, dict) and value and all(str(k).isdigit() for k in value):
            # an override such as ``a.0.b=c`` on a list that the YAML did not spell out
            value = [value.get(str(i), value.get(i, {})) for i in range(max(int(k) for k in value) + 1)]
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"{path}: expected a list")
        return [_build(inner, v, f"{path}[{i}]") for i, v in enumerate(value)]
    if origin in (dict, typing.Dict):
        return dict(value)
    if tp is float and isinstance(value, (int, str)) and not isinstance(value, bool):
        try:
            return float(value)
        except ValueError:
            return value
    if tp is int and isinstance(value, float) and value.is_integer():
        return int(value)
    return value


def from_dict(cls, data: dict, path: str = ""):
    """Instantiates dataclass ``cls`` from a nested dict.  Unknown keys are an error unless the class defines
    ``_allow_extra = True`` (then they land in ``extra``).  A class attribute ``_aliases = {other_name: field}``
    accepts a second spelling of a field (the reference's name where this package shortened it); giving both is an
    error."""
    data = dict(data or {})
    for other, name in (getattr(cls, "_aliases", None) or {}).items():
        if other in data:
            if name in data:
                raise ConfigError(f"{path or cls.__name__}: both '{other}' and its alias '{name}' are set")
            data[name] = data.pop(other)
    hints = get_type_hints(cls)
    kwargs = {}
    names = {f.name for f in fields(cls)}
    extra = {}
    for k, v in data.items():
        if k in names:
            kwargs[k] = _build(hints.get(k, Any), v, f"{path}.{k}" if path else k)
        elif getattr(cls, "_allow_extra", False):
            extra[k] = v
        else:
            raise ConfigError(f"unknown config key '{path + '.' if path else ''}{k}' for {cls.__name__}")
    if extra and "extra" in names:
        kwargs.setdefault("extra", {}).update(extra)
    try:
        return cls(**kwargs)
    except TypeError as e:
        raise ConfigError(f"{path or cls.__name__}: {e}") from e


def load_yaml(path: str, _seen: tuple = ()) -> dict:
    """Reads a YAML file.  A top-level ``base: other.yaml`` (relative to the file, or a list of them) is loaded first
    and this file's keys are merged over it, so a recipe variant only spells what it changes."""
    import os
    real = os.path.realpath(path)
    if real in _seen:
        raise ConfigError(f"recipe files include each other in a cycle: {' -> '.join(_seen + (real,))}")
    with open(path) as f:
        tree = yaml.safe_load(f) or {}
    bases = tree.pop("base", None)
    if not bases:
        return tree
    merged: dict = {}
    for b in ([bases] if isinstance(bases, str) else list(bases)):
        _deep_update(merged, load_yaml(os.path.join(os.path.dirname(path), b), _seen + (real,)))
    return _deep_update(merged, tree)


def load_config(cls, yaml_path: str | None = None, overrides: list[str] | None = None, base: dict | None = None):
    """YAML (optional) + overrides -> validated config object of type ``cls``."""
    tree = copy.deepcopy(base) if base else {}
    if yaml_path:
        _deep_update(tree, load_yaml(yaml_path))
    tree = apply_overrides(tree, overrides or [])
    return from_dict(cls, tree)


def _deep_update(dst: dict, src: dict):
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _deep_update(dst[k], v)
        else:
            dst[k] = v
    return dst


def import_from_path(py_path: str, name: str):
    """Loads attribute ``name`` from the python file ``py_path`` (the reference's py_path / fn_name plug-in
    convention, e.g. data.py_path + data.fn_name, actor/grpo_train_actor.py:812-852)."""
    import importlib.util
    import os
    import sys

    if not os.path.exists(py_path):
        mod = __import__(py_path, fromlist=[name])
        return getattr(mod, name)
    mod_name = "_gcore_plugin_" + os.path.splitext(os.path.basename(py_path))[0] + f"_{abs(hash(py_path)) % 10**8}"
    if mod_name in sys.modules:
        return getattr(sys.modules[mod_name], name)
    spec = importlib.util.spec_from_file_location(mod_name, py_path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[mod_name] = mod
    spec.loader.exec_module(mod)
    return getattr(mod, name)


__all__ = ["ConfigError", "MappingMixin", "apply_overrides", "from_dict", "load_config", "load_yaml", "to_dict",
           "import_from_path", "dataclass", "field"]
