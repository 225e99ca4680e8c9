"""TransferQueue: rows of named tensors keyed ``step{n}:{uid}:{field}`` put by producers (rollout) and fetched by
consumers (trainer ranks), with consumption tracking so that every row is trained on once
(gpatch_v4/transfer/tq_connector.py:29-175, transfer/utils.py).  ``SimpleStorage`` keeps rows in host memory (pinned
when CUDA is present, so a later host-to-device copy is asynchronous); the Mooncake (tcp / rdma) store of the
reference is an external service and is not provided.
"""
from __future__ import annotations

import threading
from collections import OrderedDict
from typing import Dict, Iterable, List, Optional, Sequence

import torch


def make_key(step: int, uid, field: str = "") -> str:
    return f"step{step}:{uid}:{field}" if field else f"step{step}:{uid}"


class SimpleStorage:
    def __init__(self, pin: bool = False):
        self._rows: "OrderedDict[str, Dict[str, torch.Tensor]]" = OrderedDict()
        self._lock = threading.Lock()
        self.pin = pin and torch.cuda.is_available()

    def put(self, key: str, row: Dict[str, torch.Tensor]):
        row = {k: (v.detach().cpu().pin_memory() if (self.pin and torch.is_tensor(v)) else
                   (v.detach().cpu() if torch.is_tensor(v) else v)) for k, v in row.items()}
        with self._lock:
            self._rows.setdefault(key, {}).update(row)

    def get(self, key: str, fields: Optional[Sequence[str]] = None):
        with self._lock:
            row = self._rows[key]
            return dict(row) if fields is None else {f: row[f] for f in fields}

    def keys(self, prefix: str = "") -> List[str]:
        with self._lock:
            return [k for k in self._rows if k.startswith(prefix)]

    def clear(self, prefix: str = ""):
        with self._lock:
            for k in [k for k in self._rows if k.startswith(prefix)]:
                del self._rows[k]

    def __len__(self):
        return len(self._rows)


class TransferQueue:
    def __init__(self, storage: Optional[SimpleStorage] = None):
        self.storage = storage or SimpleStorage()
        self._consumed: Dict[str, set] = {}
        self._lock = threading.Lock()

    def put_batch(self, step: int, uids: Iterable, rows: Iterable[Dict[str, torch.Tensor]]):
        for uid, row in zip(uids, rows):
            self.storage.put(make_key(step, uid), row)

    def ready(self, step: int, fields: Sequence[str]) -> List[str]:
        """Keys of ``step`` whose rows already hold every field in ``fields``."""
        out = []
        for k in self.storage.keys(f"step{step}:"):
            row = self.storage.get(k)
            if all(f in row for f in fields):
                out.append(k)
        return out

    def get_batch(self, step: int, fields: Sequence[str], n: int, consumer: str = "train",
                  dp_rank: int = 0, dp_size: int = 1) -> List[Dict[str, torch.Tensor]]:
        """Up to ``n`` unconsumed ready rows for this consumer; rows are split over DP ranks by a stable hash."""
        with self._lock:
            seen = self._consumed.setdefault(f"{consumer}:{step}", set())
            mine = [k for i, k in enumerate(sorted(self.storage.keys(f"step{step}:"))) if i % dp_size == dp_rank]
            ready = set(self.ready(step, fields))
            keys = [k for k in mine if k in ready and k not in seen][:n]
            seen.update(keys)
        return [dict(self.storage.get(k, fields), _key=k) for k in keys]

    def clear_step(self, step: int):
        self.storage.clear(f"step{step}:")
        with self._lock:
            for k in [k for k in self._consumed if k.endswith(f":{step}")]:
                del self._consumed[k]
