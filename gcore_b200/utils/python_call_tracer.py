"""``sys.setprofile`` based call tracer restricted to chosen source roots: logs call / return with argument summaries
(tensor shape / dtype / device instead of values).  Debugging aid equivalent to the reference's ``PythonCallTracer``
(gpatch_v4/utils/python_call_tracer.py:12-865)."""
from __future__ import annotations

import os
import sys
import threading
import time
from typing import Iterable, Optional


def _summ(v, depth=0):
    try:
        import torch
        if isinstance(v, torch.Tensor):
            return f"Tensor{tuple(v.shape)}:{str(v.dtype).replace('torch.', '')}:{v.device.type}"
    except Exception:  # noqa: BLE001
        pass
    if isinstance(v, (int, float, bool, type(None))):
        return repr(v)
    if isinstance(v, str):
        return repr(v[:40])
    if isinstance(v, (list, tuple)) and depth < 1:
        return f"{type(v).__name__}[{len(v)}]({', '.join(_summ(x, depth + 1) for x in v[:3])}{'...' if len(v) > 3 else ''})"
    if isinstance(v, dict) and depth < 1:
        return f"dict[{len(v)}]({', '.join(list(map(str, v.keys()))[:5])})"
    return type(v).__name__


class PythonCallTracer:
    def __init__(self, roots: Iterable[str], out_path: Optional[str] = None, max_depth: int = 12):
        self.roots = tuple(os.path.abspath(r) for r in roots)
        self.out = open(out_path, "w") if out_path else sys.stderr
        self.max_depth = max_depth
        self.depth = threading.local()
        self.t0 = time.time()
        self.calls = 0

    def _in_roots(self, filename):
        return filename.startswith(self.roots)

    def _profile(self, frame, event, arg):
        if event not in ("call", "return"):
            return
        co = frame.f_code
        if not self._in_roots(co.co_filename):
            return
        d = getattr(self.depth, "v", 0)
        if event == "call":
            self.depth.v = d + 1
            if d < self.max_depth:
                names = co.co_varnames[:co.co_argcount]
                args = ", ".join(f"{n}={_summ(frame.f_locals.get(n))}" for n in names if n != "self")
                self.out.write(f"{time.time() - self.t0:9.4f} {'  ' * d}> {os.path.basename(co.co_filename)}:"
                               f"{co.co_firstlineno} {co.co_name}({args})\n")
                self.calls += 1
        else:
            self.depth.v = max(d - 1, 0)
            if d - 1 < self.max_depth:
                self.out.write(f"{time.time() - self.t0:9.4f} {'  ' * max(d - 1, 0)}< {co.co_name} -> {_summ(arg)}\n")

    def __enter__(self):
        sys.setprofile(self._profile)
        threading.setprofile(self._profile)
        return self

    def __exit__(self, *exc):
        sys.setprofile(None)
        threading.setprofile(None)
        if self.out is not sys.stderr:
            self.out.close()
        return False
