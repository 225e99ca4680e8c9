"""Trainer -> role RPC layer.

Roles (sampler, generative reward model, Bradley-Terry reward model, teacher, KV store) are reached through an
``RpcClient``: in-process (the colocated SPMD layout: the engine object lives in the same process), or HTTP to a
``serve()`` endpoint for disaggregated roles.  Endpoint choice follows the reference's data-parallel mapping
(gpatch_v4/rpc_client/base_rpc_client.py:52-65) with an optional load-aware override that asks every endpoint for its
queue length first (gpatch_v4/client/sampler_client.py:22-165).  The ZeroMQ transport of the reference is a stub
that raises; it is not provided here.
"""
from __future__ import annotations

import io
import threading
import urllib.request
from typing import Any, Callable, Dict, List, Optional

import torch


def pick_endpoint_idx(dp_rank: int, dp_size: int, num_clusters: int, sample_idx: int = 0) -> int:
    """Client DP rank -> server cluster index."""
    if dp_size == num_clusters:
        ep = dp_rank
    elif dp_size < num_clusters:
        ep = dp_rank * (num_clusters // dp_size) + sample_idx
    else:
        ep = dp_rank // (dp_size // num_clusters) + sample_idx
    return ep % num_clusters


class RpcClient:
    def __init__(self, dp_rank: int = 0, dp_size: int = 1, load_aware: bool = False):
        self.dp_rank, self.dp_size, self.load_aware = dp_rank, dp_size, load_aware

    @property
    def num_clusters(self) -> int:
        raise NotImplementedError

    def call_endpoint(self, ep_idx: int, action: str, data: Dict[str, Any]) -> Any:
        raise NotImplementedError

    def pick(self, sample_idx: int = 0) -> int:
        if self.load_aware and self.num_clusters > 1:
            loads = [self.call_endpoint(i, "get_load", {}) for i in range(self.num_clusters)]
            return min(range(len(loads)), key=lambda i: (loads[i], (i - self.dp_rank) % len(loads)))
        return pick_endpoint_idx(self.dp_rank, self.dp_size, self.num_clusters, sample_idx)

    def call(self, action: str, data: Optional[Dict[str, Any]] = None, sample_idx: int = 0) -> Any:
        return self.call_endpoint(self.pick(sample_idx), action, data or {})

    def multicast(self, action: str, data: Optional[Dict[str, Any]] = None) -> List[Any]:
        """Same call on every endpoint (weight updates, sleep / wake, flush)."""
        return [self.call_endpoint(i, action, data or {}) for i in range(self.num_clusters)]


class LocalRpcClient(RpcClient):
    """Endpoints are Python objects in this process; ``action`` names a method."""

    def __init__(self, endpoints: List[Any], **kw):
        super().__init__(**kw)
        self.endpoints = list(endpoints)

    @property
    def num_clusters(self):
        return len(self.endpoints)

    def call_endpoint(self, ep_idx, action, data):
        return getattr(self.endpoints[ep_idx], action)(**data)


def _dumps(obj) -> bytes:
    buf = io.BytesIO()
    torch.save(obj, buf)
    return buf.getvalue()


def _loads(b: bytes):
    return torch.load(io.BytesIO(b), weights_only=False)


class HttpRpcClient(RpcClient):
    def __init__(self, urls: List[str], timeout_s: float = 600.0, **kw):
        super().__init__(**kw)
        self.urls, self.timeout = list(urls), timeout_s

    @property
    def num_clusters(self):
        return len(self.urls)

    def call_endpoint(self, ep_idx, action, data):
        req = urllib.request.Request(f"{self.urls[ep_idx]}/rpc/{action}", data=_dumps(data),
                                     headers={"Content-Type": "application/octet-stream"})
        with urllib.request.urlopen(req, timeout=self.timeout) as r:
            return _loads(r.read())


def serve(target: Any, host: str = "127.0.0.1", port: int = 0, allowed: Optional[List[str]] = None):
    """Serves ``target``'s methods at ``/rpc/<name>`` on a background thread.  Returns (server, url)."""
    from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_POST(self):
            name = self.path.rsplit("/", 1)[-1]
            if not self.path.startswith("/rpc/") or name.startswith("_") or (allowed and name not in allowed):
                self.send_response(404)
                self.end_headers()
                return
            data = _loads(self.rfile.read(int(self.headers.get("Content-Length", "0"))))
            try:
                out, code = getattr(target, name)(**data), 200
            except Exception as e:
                out, code = {"error": f"{type(e).__name__}: {e}"}, 500
            body = _dumps(out)
            self.send_response(code)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

    srv = ThreadingHTTPServer((host, port), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv, f"http://{host}:{srv.server_address[1]}"
