"""Role clients on top of ``RpcClient``: sampler, generative / Bradley-Terry reward models, teacher, KV store
(gpatch_v4/client/{sampler_client,gen_rm_client,bt_rm_client,teacher_client,kv_store_client,infer_client}.py)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import torch

from .rpc import RpcClient


class SamplerClient:
    def __init__(self, rpc: RpcClient):
        self.rpc = rpc

    def generate(self, prompts: Sequence[Sequence[int]], sampling_params=None, sample_idx: int = 0):
        return self.rpc.call("generate", dict(prompts=[list(p) for p in prompts], params=sampling_params), sample_idx)

    def update_weights(self, named_tensors=None, **kw):
        return self.rpc.multicast("update_weights", dict(named_tensors=named_tensors, **kw))

    def sleep(self):
        return self.rpc.multicast("sleep")

    def wake_up(self):
        return self.rpc.multicast("wake_up")

    def flush_cache(self):
        return self.rpc.multicast("flush_cache")

    def get_load(self) -> List[int]:
        return self.rpc.multicast("get_load")


class GenRmClient:
    """Generative reward model: the RM writes a critique; ``parse_fn`` turns it into a score."""

    def __init__(self, rpc: RpcClient, build_prompt, parse_fn, sampling_params=None):
        self.rpc, self.build_prompt, self.parse_fn, self.params = rpc, build_prompt, parse_fn, sampling_params

    def score(self, samples: Sequence[dict]) -> torch.Tensor:
        prompts = [self.build_prompt(s) for s in samples]
        outs = self.rpc.call("generate", dict(prompts=prompts, params=self.params))
        return torch.tensor([float(self.parse_fn(o, s)) for o, s in zip(outs, samples)])


class BtRmClient:
    """Bradley-Terry reward model: one forward pass per sequence, scalar at the last token; requests are batched and
    scored once (gpatch_v4/actor/grpo_bt_rm_actor.py:15)."""

    def __init__(self, rpc: RpcClient):
        self.rpc = rpc

    def score(self, samples: Sequence[dict]) -> torch.Tensor:
        out = self.rpc.call("score", dict(sequences=[s["tokens"].tolist() if torch.is_tensor(s["tokens"]) else
                                                     list(s["tokens"]) for s in samples]))
        return torch.as_tensor(out, dtype=torch.float32)


class TeacherClient:
    def __init__(self, rpc: RpcClient):
        self.rpc = rpc

    def logprobs(self, samples: Sequence[dict], top_k: int = 0):
        return self.rpc.call("teacher_logprobs", dict(sequences=[list(map(int, s["tokens"])) for s in samples],
                                                      top_k=top_k))


class KvStoreClient:
    def __init__(self, rpc: RpcClient):
        self.rpc = rpc

    def put(self, key: str, value: Any):
        return self.rpc.call("put", dict(key=key, value=value))

    def get(self, key: str, default=None):
        return self.rpc.call("get", dict(key=key, default=default))

    def delete(self, key: str):
        return self.rpc.call("delete", dict(key=key))


class KvStore:
    """The serving side of ``KvStoreClient`` (gpatch_v4/actor KvStoreActor)."""

    def __init__(self):
        self._d: Dict[str, Any] = {}

    def put(self, key, value):
        self._d[key] = value
        return True

    def get(self, key, default=None):
        return self._d.get(key, default)

    def delete(self, key):
        return self._d.pop(key, None) is not None

    def get_load(self):
        return len(self._d)
