"""Disaggregated placement: trainer ranks and rollout-engine ranks are different processes on different GPUs.

The default process group spans both roles; every role lays out its own parallel groups inside its slice
(``parallel_state.initialize_model_parallel(ranks=...)``).  Three things cross the role boundary, all through the
default group:

* **weights** — after every optimizer step the trainers stream the model to the rollout ranks in buckets: a tensor is
  made whole inside the trainer's tensor-parallel group, packed into a flat bucket of at most
  ``update_weight_max_size_mb`` and broadcast from the first trainer rank; every rollout rank cuts the rows of ITS
  tensor-parallel shard out of the bucket straight into the engine's tensors.  (The reference's non-colocated path:
  gather to the (pp, tp) head, NCCL bucket broadcast to all inference ranks, gpatch_v4/client/
  update_weight_factory.py:381-445, 491-517.)
* **prompts** — gathered from the trainer data-parallel ranks, broadcast to the rollout ranks, split over the engine
  replicas.
* **samples** — token ids and log-probs of every response, gathered on the first rollout rank and broadcast back; a
  trainer rank keeps the groups of its own prompts.

Rollout ranks run ``SamplerServer.serve()``: a loop over commands (update weights / generate / stop) that the first
trainer rank announces with a small broadcast.  Trainer ranks use ``RemoteRollout`` in place of a colocated engine.
Role layout and GPU accounting: ``orches/resource_allocator.py``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..core import parallel_state as ps
from .engine import InferEngine, RolloutWeights, SamplingParams
from .weight_sync import _engine_tensor_map, _rows_for_rank, plan_buckets

OP_STOP, OP_WEIGHTS, OP_GENERATE = 0, 1, 2


@dataclass
class RoleLayout:
    """Trainer ranks come first (so that global rank 0 is a trainer), rollout ranks after them."""
    world: int
    n_train: int
    sampler_tp: int = 1

    def __post_init__(self):
        if not 0 < self.n_train < self.world:
            raise ValueError(f"disaggregated placement needs both roles: {self.n_train} trainer ranks of {self.world}")
        if (self.world - self.n_train) % self.sampler_tp:
            raise ValueError("rollout ranks must be a multiple of the rollout tensor-parallel size")

    @property
    def train_ranks(self) -> List[int]:
        return list(range(self.n_train))

    @property
    def sampler_ranks(self) -> List[int]:
        return list(range(self.n_train, self.world))

    @property
    def n_engines(self) -> int:
        return (self.world - self.n_train) // self.sampler_tp

    def role(self, rank: int) -> str:
        return "train" if rank < self.n_train else "sampler"

    def engine_of(self, rank: int) -> int:
        return (rank - self.n_train) // self.sampler_tp


def setup_roles(layout: RoleLayout, train_parallel: Dict[str, int]):
    """Creates both roles' parallel groups (collective over the default group: every rank creates every group, in the
    same order) and leaves this rank with the state of its own role."""
    global _XFER
    ps.initialize_model_parallel(ranks=layout.train_ranks, **train_parallel)
    ps.initialize_model_parallel(ranks=layout.sampler_ranks, tp=layout.sampler_tp)
    # the weights travel on a group of their own: the first trainer rank and every rollout rank
    _XFER = dist.new_group([0] + layout.sampler_ranks)
    return layout.role(dist.get_rank())


_XFER = None


def _dev():
    return torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")


def _announce(op: int, arg: int = 0, src: int = 0) -> Tuple[int, int]:
    t = torch.tensor([op, arg], dtype=torch.int64, device=_dev())
    dist.broadcast(t, src=src)
    return int(t[0]), int(t[1])


# ---------------------------------------------------------------------------------------------------- weights
def _full_tensor(name: str, local: torch.Tensor, mode: str, tp: int, group, cfg) -> torch.Tensor:
    """The whole tensor from this rank's tensor-parallel shard (column / row modes are cut along dim 0 / dim 1; the
    fused projections interleave their parts per rank, which ``weight_sync._rows_for_rank`` describes)."""
    if tp == 1 or mode not in ("column", "row"):
        return local
    shards = [torch.empty_like(local) for _ in range(tp)]
    dist.all_gather(shards, local.contiguous(), group=group)
    if mode == "row":
        return torch.cat(shards, dim=1)
    full_rows = local.shape[0] * tp
    out = torch.empty(full_rows, *local.shape[1:], dtype=local.dtype, device=local.device)
    for r, sh in enumerate(shards):
        at = 0
        for a, b in _rows_for_rank(name, full_rows, tp, r, cfg):
            out[a:b] = sh[at:at + (b - a)]
            at += b - a
    return out


def _cut_for_rank(name: str, full: torch.Tensor, mode: str, tp: int, rank: int, cfg) -> torch.Tensor:
    if tp == 1 or mode not in ("column", "row"):
        return full
    if mode == "row":
        w = full.shape[1] // tp
        return full[:, rank * w:(rank + 1) * w]
    return torch.cat([full[a:b] for a, b in _rows_for_rank(name, full.shape[0], tp, rank, cfg)], 0)


def weight_manifest(policy_engine) -> List[Tuple[str, Tuple[int, ...], str]]:
    """(name, full shape, tensor-parallel mode) of every tensor the rollout engine needs, in transfer order."""
    model = policy_engine.model
    tp = model.tp_size
    out = []
    params = dict(model.named_parameters())
    for n, p in policy_engine.named_local_weights(merged_lora=True):
        mode = getattr(params.get(n), "tp_mode", "none")
        shape = list(p.shape)
        if tp > 1 and mode == "column":
            shape[0] *= tp
        elif tp > 1 and mode == "row":
            shape[1] *= tp
        out.append((n, tuple(shape), mode))
    return out


def send_weights(policy_engine, bucket_mb: int = 512) -> Dict[str, float]:
    """Trainer side of the bucket broadcast (all trainer ranks call it: the gathers inside the trainer's
    tensor-parallel group are collective; only the first trainer rank feeds the broadcast)."""
    model = policy_engine.model
    cfg = model.cfg
    tp = model.tp_size
    group = ps.get_tensor_model_parallel_group() if tp > 1 else None
    head = dist.get_rank() == 0
    manifest = weight_manifest(policy_engine)
    _announce(OP_WEIGHTS, 0)        # every rank of the default group hears every command
    src = dict(policy_engine.named_local_weights(merged_lora=True))
    wire = next(iter(src.values())).dtype   # one wire dtype for the whole model (bf16 on GPUs)
    if head:
        dist.broadcast_object_list([manifest, [int(bucket_mb), str(wire).split(".")[-1]]], src=0, group=_XFER)
    esz = torch.empty(0, dtype=wire).element_size()
    numel = {n: int(torch.Size(shape).numel()) for n, shape, _ in manifest}
    sizes = [(n, numel[n] * esz) for n, _, _ in manifest]
    modes = {n: m for n, _, m in manifest}
    moved, nb = 0, 0
    dev = _dev()
    for bucket in plan_buckets(sizes, bucket_mb << 20):
        flat = torch.empty(sum(numel[n] for n in bucket), dtype=wire, device=dev)
        at = 0
        for n in bucket:
            full = _full_tensor(n, src[n].detach(), modes[n], tp, group, cfg)
            flat[at:at + full.numel()] = full.reshape(-1).to(wire)
            at += full.numel()
        if head:
            dist.broadcast(flat, src=0, group=_XFER)
            moved += flat.numel() * esz
            nb += 1
    return {"bytes": float(moved), "buckets": float(nb)}


def recv_weights(infer_engine: InferEngine, model_for_names, layout: RoleLayout) -> Dict[str, float]:
    """Rollout side: receives the buckets and writes this rank's tensor-parallel shard of every tensor."""
    box = [None, None]
    dist.broadcast_object_list(box, src=0, group=_XFER)
    manifest, (bucket_mb, wire_name) = box
    wire = getattr(torch, wire_name)
    esz = torch.empty(0, dtype=wire).element_size()
    dst = _engine_tensor_map(infer_engine, model_for_names)
    tp = layout.sampler_tp
    tpr = (dist.get_rank() - layout.n_train) % tp
    numel = {n: int(torch.Size(shape).numel()) for n, shape, _ in manifest}
    sizes = [(n, numel[n] * esz) for n, _, _ in manifest]
    info = {n: (shape, mode) for n, shape, mode in manifest}
    dev = _dev()
    moved = 0
    for bucket in plan_buckets(sizes, bucket_mb << 20):
        flat = torch.empty(sum(numel[n] for n in bucket), dtype=wire, device=dev)
        dist.broadcast(flat, src=0, group=_XFER)
        at = 0
        for n in bucket:
            shape, mode = info[n]
            if n in dst:
                full = flat[at:at + numel[n]].view(shape)
                piece = _cut_for_rank(n, full, mode, tp, tpr, infer_engine.cfg)
                dst[n].copy_(piece.to(dst[n].dtype))
                moved += piece.numel() * esz
            at += numel[n]
    infer_engine.update_weights(infer_engine.w)
    return {"bytes": float(moved)}


# ---------------------------------------------------------------------------------------------------- rollout ranks
class SamplerServer:
    """What a rollout rank runs: an engine with weights of its own, served until the trainers say stop."""

    def __init__(self, cfg, model_cfg, layout: RoleLayout, device=None):
        from ..models.gpt import GPTModel
        self.cfg, self.layout = cfg, layout
        self.rank = dist.get_rank()
        self.device = device or _dev()
        tp = layout.sampler_tp
        # a model skeleton in the rollout layout: it names the tensors and gives the engine storage of its own
        torch.manual_seed(cfg.training.seed)
        dt = "bfloat16" if self.device.type == "cuda" else model_cfg.dtype
        import dataclasses
        self.model_cfg = dataclasses.replace(model_cfg, dtype=dt)
        self.model = GPTModel(self.model_cfg, tp_size=tp, device=self.device)
        for p in self.model.parameters():
            p.requires_grad_(False)
        ie = cfg.sampler.infer_engine_configs[0]
        t = cfg.training
        n_req = max(t.rollout_gbs // max(layout.n_engines, 1), 1) * t.sampling_repeat_n
        self.engine = InferEngine(
            self.model_cfg, RolloutWeights.from_model(self.model, clone=False), tp_size=tp,
            tp_group=ps.get_tensor_model_parallel_group() if tp > 1 else None,
            max_running_requests=ie.max_running_requests or n_req,
            max_model_len=ie.max_model_len or (cfg.data.max_prompt_length + ie.generate_max_tokens),
            kv_block_size=ie.kv_block_size, num_kv_blocks=ie.num_kv_blocks,
            gpu_memory_utilization=ie.gpu_memory_utilization, max_prefill_tokens=ie.max_prefill_tokens,
            use_cuda_graph=not ie.disable_cuda_graph, device=self.device)
        self.stats = dict(weight_updates=0, generate_calls=0)

    def serve(self):
        while True:
            op, arg = _announce(0, 0)
            if op == OP_STOP:
                return self.stats
            if op == OP_WEIGHTS:
                recv_weights(self.engine, self.model, self.layout)
                self.stats["weight_updates"] += 1
            elif op == OP_GENERATE:
                self._generate()
                self.stats["generate_calls"] += 1

    def _generate(self):
        box = [None]
        dist.broadcast_object_list(box, src=0)
        job = box[0]
        prompts, n, sp = job["prompts"], job["n"], SamplingParams(**job["sampling"])
        lay = self.layout
        e = lay.engine_of(self.rank)
        mine = list(range(e, len(prompts), lay.n_engines))            # prompt indices of this engine replica
        out = []
        if mine:
            self.engine.wake_up(("kv_cache",))
            reqs = self.engine.generate([prompts[i] for i in mine], sp, n=n)
            self.engine.sleep(("kv_cache",))
            for k, r in enumerate(reqs):
                out.append((mine[k // n], k % n, r.out_tokens, r.out_logprobs, r.finish_reason))
        # the tensor-parallel ranks of an engine hold the same result: its first rank reports
        report = out if (self.rank - lay.n_train) % lay.sampler_tp == 0 else []
        gathered = [None] * len(lay.sampler_ranks)
        dist.all_gather_object(gathered, report, group=ps.get_world_group()) if len(lay.sampler_ranks) > 1 \
            else gathered.__setitem__(0, report)
        head = lay.sampler_ranks[0]
        res = [x for part in gathered for x in part] if self.rank == head else None
        dist.broadcast_object_list([res], src=head)


# ---------------------------------------------------------------------------------------------------- trainer ranks
class RemoteRollout:
    """Trainer-side handle of the rollout ranks (the role an engine client plays for the reference's trainers)."""

    def __init__(self, layout: RoleLayout):
        self.layout = layout
        self.rank = dist.get_rank()

    def update_weights(self, policy_engine, bucket_mb: int = 512):
        return send_weights(policy_engine, bucket_mb)

    def generate(self, prompts: Sequence[Sequence[int]], n: int, sampling: SamplingParams) -> List[dict]:
        """Every trainer data-parallel head passes its prompts; returns, per prompt and sample, the response."""
        lay = self.layout
        dp_heads = ps.get_tensor_model_parallel_rank() == 0 and ps.get_pipeline_model_parallel_rank() == 0 \
            and ps.get_context_parallel_rank() == 0
        parts = [None] * len(lay.train_ranks)
        mine = [list(map(int, p)) for p in prompts] if dp_heads else None
        if len(lay.train_ranks) > 1:
            dist.all_gather_object(parts, mine, group=ps.get_world_group())
        else:
            parts[0] = mine
        offsets, flat = {}, []
        for r, p in enumerate(parts):
            if p is not None:
                offsets[r] = (len(flat), len(p))
                flat += p
        _announce(OP_GENERATE, len(flat))
        dist.broadcast_object_list([{"prompts": flat, "n": int(n), "sampling": dict(sampling.__dict__)}], src=0)
        box = [None]
        dist.broadcast_object_list(box, src=lay.sampler_ranks[0])
        # model-parallel peers of a data-parallel head take the head's slice
        head_rank = ps.get_state().group_ranks.get("mp_cp", [self.rank])[0] if not dp_heads else self.rank
        start, count = offsets[lay.train_ranks.index(head_rank)]
        res = {(i, k): (toks, lps, why) for i, k, toks, lps, why in box[0]}
        out = []
        for i in range(start, start + count):
            for k in range(n):
                toks, lps, why = res[(i, k)]
                out.append(dict(prompt=flat[i], out_tokens=toks, out_logprobs=lps, finish_reason=why))
        return out

    def stop(self):
        _announce(OP_STOP, 0)
