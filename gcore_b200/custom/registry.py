"""Registry of user python files (datasets, rewards, losses, ...) by module name, shared by every process of a job
through one json file whose path travels in an environment variable (gpatch_v4/custom/registry.py): the launcher
registers ``name -> path`` once, workers import the module by name, a second registration of the same name with a
different file is an error."""
from __future__ import annotations

import importlib.util
import json
import os
import sys
import tempfile
import threading
from typing import Dict, Optional

ENV = "GCORE_CUSTOM_MODULE_REGISTRY_PATH"
_LOCK = threading.Lock()


def _path(create: bool) -> Optional[str]:
    p = os.environ.get(ENV)
    if p or not create:
        return p
    fd, p = tempfile.mkstemp(prefix="gcore_custom_registry_", suffix=".json")
    os.close(fd)
    with open(p, "w") as f:
        json.dump({}, f)
    os.environ[ENV] = p
    return p


def load_custom_module_registry() -> Dict[str, str]:
    p = _path(False)
    if not p or not os.path.exists(p):
        return {}
    with open(p) as f:
        reg = json.load(f)
    if not isinstance(reg, dict):
        raise ValueError(f"invalid custom module registry: {p}")
    return reg


def register_custom_module(mod_name: str, py_path: str) -> None:
    p = _path(True)
    ap = os.path.abspath(py_path)
    with _LOCK:
        reg = load_custom_module_registry()
        if reg.get(mod_name, ap) != ap:
            raise ValueError(f"custom module registry collision: {mod_name} maps to {reg[mod_name]}, not {ap}")
        reg[mod_name] = ap
        tmp = p + ".tmp"
        with open(tmp, "w") as f:
            json.dump(reg, f)
        os.replace(tmp, p)


def load_custom_module(mod_name: str):
    if mod_name in sys.modules:
        return sys.modules[mod_name]
    reg = load_custom_module_registry()
    if mod_name not in reg:
        raise KeyError(f"custom module '{mod_name}' is not registered (known: {sorted(reg)})")
    spec = importlib.util.spec_from_file_location(mod_name, reg[mod_name])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[mod_name] = mod
    spec.loader.exec_module(mod)
    return mod
