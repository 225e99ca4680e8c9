"""Process groups that can be torn down and rebuilt.

A NCCL communicator pins device memory (its buffers and channels) for as long as it lives.  While the rollout engine
owns the GPU the trainer's communicators are dead weight, so they can be destroyed before a rollout and re-created
after it (``policy.offload_process_group``); the reference does this with a registry that records how every group was
made (gpatch_v4/utils/reloadable_process_group.py:116-287, use site rollout_generator/base_generator.py:226-258).

``ReloadableGroup`` is a handle that stays valid across reloads: code holds the handle, asks it for the current
``torch.distributed`` group when it issues a collective (``handle.group``), and ``offload_all`` / ``reload_all`` walk
the registry.  ``dist.new_group`` is collective over the default group, so both calls must run on every rank in the
same order - the registry keeps creation order.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch.distributed as dist

_REGISTRY: List["ReloadableGroup"] = []


class ReloadableGroup:
    def __init__(self, ranks: Sequence[int], backend: Optional[str] = None, timeout=None, name: str = ""):
        self.ranks, self.backend, self.timeout, self.name = list(ranks), backend, timeout, name
        self._group = None
        self.loads = 0
        self._create()
        _REGISTRY.append(self)

    def _create(self):
        kw = {}
        if self.backend:
            kw["backend"] = self.backend
        if self.timeout is not None:
            kw["timeout"] = self.timeout
        self._group = dist.new_group(self.ranks, **kw)
        self.loads += 1

    @property
    def group(self):
        if self._group is None:
            raise RuntimeError(f"process group {self.name or self.ranks} is offloaded: call reload_all() first")
        return self._group

    @property
    def loaded(self) -> bool:
        return self._group is not None

    def offload(self):
        if self._group is not None:
            if dist.get_rank() in self.ranks:
                dist.destroy_process_group(self._group)
            self._group = None

    def reload(self):
        if self._group is None:
            self._create()

    def size(self) -> int:
        return len(self.ranks)

    def rank(self) -> int:
        return self.ranks.index(dist.get_rank()) if dist.get_rank() in self.ranks else -1


def new_reloadable_group(ranks: Sequence[int], backend: Optional[str] = None, timeout=None, name: str = ""):
    return ReloadableGroup(ranks, backend, timeout, name)


def offload_all(only_backend: Optional[str] = "nccl") -> int:
    """Destroys every registered group (of ``only_backend``; None = all), in creation order.  Returns how many."""
    n = 0
    for g in _REGISTRY:
        if g.loaded and (only_backend is None or (g.backend or dist.get_backend()) == only_backend):
            g.offload()
            n += 1
    return n


def reload_all() -> int:
    n = 0
    for g in _REGISTRY:
        if not g.loaded:
            g.reload()
            n += 1
    return n


def registered() -> List[ReloadableGroup]:
    return list(_REGISTRY)


def clear_registry():
    _REGISTRY.clear()
