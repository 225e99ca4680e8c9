"""``torch_dist`` checkpoints: the on-disk format of ``torch.distributed.checkpoint`` (``.metadata`` +
``__{rank}_{k}.distcp`` files whose items are ``torch.save`` payloads) with Megatron-Core's key names, stacked-layer
axis and sidecars (``common.pt``, ``metadata.json``, ``latest_checkpointed_iteration.txt``, ``iter_{step:07d}/``), as
written by the reference (gpatch_v4/training_backend/megatron_backend/checkpoint.py:837-1070, 1354-1765).

Every rank writes the chunks it owns in-process (no forked writer), work is spread over data-parallel ranks
(model weights by the DP-rank-0 replica, optimizer buckets round-robin over DP ranks - the role of the reference's
``FullyParallelSaveStrategyWrapper``), and loading reads whatever regions the current topology needs, so a checkpoint
can be resumed under a different TP / DP size.  The files are readable by ``torch.distributed.checkpoint`` itself
(``FileSystemReader``), which the tests use as an independent check of the format.
"""
from __future__ import annotations

import io
import json
import os
import pickle
import random
import shutil
import threading
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist
from torch.distributed.checkpoint.filesystem import _StorageInfo
from torch.distributed.checkpoint.metadata import (BytesStorageMetadata, ChunkStorageMetadata, Metadata, MetadataIndex,
                                                   TensorProperties, TensorStorageMetadata)

from ..core import parallel_state as ps
from .layout import Chunk, assign_from_chunks, param_chunks

LATEST = "latest_checkpointed_iteration.txt"


def iter_dir(root: str, step: int) -> str:
    return os.path.join(root, f"iter_{step:07d}")


def read_latest_step(root: str) -> Optional[int]:
    p = os.path.join(root, LATEST)
    if not os.path.exists(p):
        return None
    txt = open(p).read().strip()
    return int(txt) if txt.isdigit() else None


# ------------------------------------------------------------------------------------------------ writer
class _ShardWriter:
    def __init__(self, path: str, rank: int):
        self.rel = f"__{rank}_0.distcp"
        self.f = open(os.path.join(path, self.rel), "wb")
        self.tensors: Dict[str, dict] = {}
        self.bytes_items: Dict[str, BytesStorageMetadata] = {}
        self.storage: Dict[MetadataIndex, _StorageInfo] = {}

    def add_chunk(self, c: Chunk):
        t = c.tensor.detach().cpu().contiguous()
        off = self.f.tell()
        torch.save(t, self.f)
        length = self.f.tell() - off
        ent = self.tensors.setdefault(c.key, dict(dtype=t.dtype, size=tuple(c.global_shape), chunks=[]))
        assert ent["size"] == tuple(c.global_shape), f"{c.key}: inconsistent global shape"
        ent["chunks"].append((tuple(c.offset), tuple(t.shape)))
        self.storage[MetadataIndex(c.key, torch.Size(c.offset))] = _StorageInfo(self.rel, off, length)

    def add_object(self, key: str, obj):
        # a sharded object travels as a BytesIO holding its torch.save image, and torch.distributed.checkpoint stores
        # non-tensor items with torch.save again: readers unwrap twice (Megatron's ShardedObject convention)
        inner = io.BytesIO()
        torch.save(obj, inner)
        inner.seek(0)
        buf = io.BytesIO()
        torch.save(inner, buf)
        off = self.f.tell()
        self.f.write(buf.getvalue())
        self.bytes_items[key] = BytesStorageMetadata()
        self.storage[MetadataIndex(key)] = _StorageInfo(self.rel, off, self.f.tell() - off)

    def close(self):
        self.f.flush()
        os.fsync(self.f.fileno())
        self.f.close()
        return dict(tensors=self.tensors, bytes_items=self.bytes_items, storage=self.storage)


def _merge_metadata(parts: List[dict]) -> Metadata:
    sdm: Dict[str, object] = {}
    storage: Dict[MetadataIndex, _StorageInfo] = {}
    for part in parts:
        for k, ent in part["tensors"].items():
            if k not in sdm:
                sdm[k] = TensorStorageMetadata(TensorProperties(dtype=ent["dtype"]), torch.Size(ent["size"]), [])
            for off, sizes in ent["chunks"]:
                sdm[k].chunks.append(ChunkStorageMetadata(torch.Size(off), torch.Size(sizes)))
        for k, v in part["bytes_items"].items():
            sdm[k] = v
        storage.update(part["storage"])
    return Metadata(state_dict_metadata=sdm, storage_data=storage)


def get_rng_state() -> dict:
    """Field names of Megatron's ``rng_state`` object (gpatch_v4/training_backend/megatron_backend/checkpoint.py:
    753-797).  ``rng_tracker_states`` holds the named CUDA generators of a tensor-parallel RNG tracker; this package
    draws its parallel randomness (initialisation, dropout-free training) from the default generators, so the entry
    carries the default CUDA state under the tracker's default name."""
    st = {"random_rng_state": random.getstate(), "np_rng_state": np.random.get_state(),
          "torch_rng_state": torch.get_rng_state(), "rng_tracker_states": {}}
    if torch.cuda.is_available():
        st["cuda_rng_state"] = torch.cuda.get_rng_state()
        st["rng_tracker_states"] = {"model-parallel-rng": st["cuda_rng_state"]}
    return st


def set_rng_state(st):
    if isinstance(st, (list, tuple)):   # the object is a list with one entry per data-parallel random stream
        st = st[0]
    random.setstate(st.get("random_rng_state", st.get("random")))
    np.random.set_state(st.get("np_rng_state", st.get("numpy")))
    torch.set_rng_state(st.get("torch_rng_state", st.get("torch")))
    cuda = st.get("cuda_rng_state", st.get("cuda"))
    if cuda is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(cuda)


def rng_object_key(pp: int, tp: int, pp_size: int, tp_size: int, dp: int = 0) -> str:
    """Storage key of the ``rng_state`` sharded object: global shape (pp_size, tp_size), offset (pp, tp); the object
    of data-parallel replica 0 is the one Megatron stores, the other replicas' streams are kept under a sibling name
    (they differ here because every data-parallel rank seeds its rollout sampler differently)."""
    base = "rng_state" if dp == 0 else f"rng_state_dp{dp}"
    return f"{base}/shard_{pp}_{tp}_{pp_size}_{tp_size}"


def scheduler_state(opt_cfg, optimizer, total_steps) -> dict:
    """``OptimizerParamScheduler.state_dict`` fields."""
    return {"max_lr": opt_cfg.lr, "lr_warmup_steps": opt_cfg.lr_warmup_steps, "num_steps": optimizer.step_count,
            "lr_decay_style": opt_cfg.lr_decay_style, "lr_decay_steps": opt_cfg.lr_decay_steps or total_steps,
            "min_lr": opt_cfg.min_lr, "start_wd": opt_cfg.weight_decay, "end_wd": opt_cfg.weight_decay,
            "wd_incr_style": "constant", "wd_incr_steps": opt_cfg.lr_decay_steps or total_steps}


def _canonical(model, name: str) -> str:
    """Parameter name in the unpartitioned model: a pipeline stage numbers its layers from zero, the checkpoint uses
    the global layer index (the stacked-layer axis spans all stages), so any pipeline layout can load any other's."""
    fn = getattr(model, "canonical_name", None)
    if fn is not None:
        return fn(name)
    inner = getattr(model, "language_model", None)  # vision-language wrapper
    if inner is not None and name.startswith("language_model."):
        return "language_model." + inner.canonical_name(name[len("language_model."):])
    return name


def _model_chunks(engine) -> List[Chunk]:
    st = ps.get_state()
    model = engine.model
    tp_rank, tp = (ps.get_tensor_model_parallel_rank(), model.tp_size)
    ep_rank, ep = (ps.get_expert_model_parallel_rank(), model.ep_size)
    dp_rank = ps.get_data_parallel_rank(with_context_parallel=True)
    edp_rank = st.rank_in("edp") if st.initialized else 0
    out = []
    for name, p in model.named_parameters():
        mode = getattr(p, "tp_mode", "none")
        owner_dp = edp_rank if mode == "expert" else dp_rank
        if owner_dp != 0:
            continue
        for c in param_chunks(_canonical(model, name), p.detach(), model.cfg, tp_rank if tp > 1 else 0, tp, ep_rank, ep,
                              mode):
            if c.replicated and tp_rank != 0:
                continue
            out.append(c)   # the key is the parameter's path in the model, without a prefix (Megatron builds the
            #                 model's sharded state dict with an empty prefix)
    return out


def _optimizer_chunks(engine) -> List[Chunk]:
    """Per-parameter optimizer state (fp32 master, exp_avg, exp_avg_sq) in the parameter's own sharding; each bucket is
    reassembled from its DP shards and written by DP rank ``bucket_index % dp``."""
    opt = engine.optimizer
    model = engine.model
    tp_rank, tp = ps.get_tensor_model_parallel_rank(), model.tp_size
    ep_rank, ep = ps.get_expert_model_parallel_rank(), model.ep_size
    names = {id(p): _canonical(model, n) for n, p in model.named_parameters()}
    out = []
    for bi, sh in enumerate(opt.shards):
        buf, bucket = sh["buf"], sh["bucket"]
        full = {}
        for k in ("master", "m", "v"):
            loc = sh[k].to(buf.param_data.device) if sh[k].device != buf.param_data.device else sh[k]
            if buf.dp > 1 and buf.use_distributed_optimizer:
                g = torch.empty(bucket.end - bucket.start, dtype=torch.float32, device=loc.device)
                dist.all_gather_into_tensor(g, loc.contiguous(), group=buf.group)
            else:
                g = loc
            full[k] = g
        if bi % buf.dp != buf.dp_rank:
            continue
        for p in bucket.params:
            o = buf.offsets[id(p)] - bucket.start
            name = names[id(p)]
            mode = getattr(p, "tp_mode", "none")
            for k, label in (("master", "fp32_param"), ("m", "exp_avg"), ("v", "exp_avg_sq")):
                t = full[k][o:o + p.numel()].view(p.shape)
                for c in param_chunks(name, t, model.cfg, tp_rank if tp > 1 else 0, tp, ep_rank, ep, mode):
                    if c.replicated and tp_rank != 0:
                        continue
                    c.key = f"optimizer.state.{label}.{c.key}"
                    out.append(c)
    return out


_PENDING: List[dict] = []   # at most one asynchronous save in flight per process


def _finish_save(h: dict):
    """Second half of a save: every rank has written its shard and left its part file; rank 0 merges the metadata,
    writes the sidecars and moves ``latest`` forward (only now does the checkpoint exist for a reader)."""
    path, root, step, rank, world = h["path"], h["root"], h["step"], h["rank"], h["world"]
    if h.get("thread") is not None:
        h["thread"].join()
        if h.get("error"):
            raise RuntimeError(f"asynchronous checkpoint write failed: {h['error']}")
    if world > 1:
        ps.cpu_barrier()
    if rank == 0:
        parts = []
        for r in range(world):
            with open(os.path.join(path, f".part_{r}.pkl"), "rb") as f:
                parts.append(pickle.load(f))
        md = _merge_metadata(parts)
        tmp = os.path.join(path, ".metadata.tmp")
        with open(tmp, "wb") as f:
            pickle.dump(md, f)
        os.replace(tmp, os.path.join(path, ".metadata"))
        torch.save(h["common"], os.path.join(path, "common.pt"))
        with open(os.path.join(path, "metadata.json"), "w") as f:
            json.dump({"sharded_backend": "torch_dist", "sharded_backend_version": 1, "common_backend": "torch",
                       "common_backend_version": 1}, f)
        for r in range(world):
            os.remove(os.path.join(path, f".part_{r}.pkl"))
        with open(os.path.join(root, LATEST), "w") as f:
            f.write(str(step))
        _rotate(root, *h["rotate"])
    if world > 1:
        ps.cpu_barrier()


def wait_for_async_save():
    """Completes the asynchronous save in flight, if any (collective: every rank calls it)."""
    while _PENDING:
        _finish_save(_PENDING.pop(0))


def save_checkpoint(engine, root: str, step: int, extra_state: Optional[dict] = None, save_optim: bool = True,
                    save_total_limit: Optional[int] = None, save_retain_interval: Optional[int] = None,
                    async_delete: bool = True, async_save: bool = False) -> str:
    """``async_save``: tensors are copied to host memory before the call returns (a consistent snapshot of this
    step), the shard file is written by a background thread while training goes on, and the checkpoint is published
    (metadata, ``latest``) by the next ``save_checkpoint`` / ``wait_for_async_save`` call."""
    wait_for_async_save()
    path = iter_dir(root, step)
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    if rank == 0:
        os.makedirs(path, exist_ok=True)
    if world > 1:
        ps.cpu_barrier()
    chunks = _model_chunks(engine)
    if save_optim and engine.optimizer is not None:
        chunks += _optimizer_chunks(engine)
    if async_save:
        for c in chunks:   # snapshot: training may overwrite the device tensors while the file is being written
            c.tensor = c.tensor.detach().to("cpu", copy=True)
    pp, tp = ps.get_pipeline_model_parallel_rank(), ps.get_tensor_model_parallel_rank()
    dp = ps.get_data_parallel_rank(with_context_parallel=True)
    rng_key = rng_object_key(pp, tp, ps.get_pipeline_model_parallel_world_size(),
                             ps.get_tensor_model_parallel_world_size(), dp)
    rng_state = [get_rng_state()]
    common = {"iteration": step, "checkpoint_version": 3.0,
              "optimizer_step": engine.optimizer.step_count if engine.optimizer is not None else 0,
              "engine_step": engine.step, "model_config": engine.model_cfg.to_dict(),
              "topology": dict(tp=engine.model.tp_size, ep=engine.model.ep_size,
                               pp=ps.get_pipeline_model_parallel_world_size(), world=world),
              "extra_state": extra_state or {}}
    if engine.optimizer is not None and save_optim:
        oc = engine.opt_cfg
        common["optimizer"] = {"optimizer": {"param_groups": [
            {"lr": oc.lr, "betas": (oc.adam_beta1, oc.adam_beta2), "eps": oc.adam_eps, "weight_decay": oc.weight_decay,
             "step": engine.optimizer.step_count}]}, "param_state_sharding_type": "fully_sharded_model_space"}
        common["lr_scheduler"] = scheduler_state(oc, engine.optimizer, engine.total_steps)
    h = dict(path=path, root=root, step=step, rank=rank, world=world, common=common, thread=None, error=None,
             rotate=(save_total_limit, save_retain_interval, async_delete))

    def write():
        try:
            w = _ShardWriter(path, rank)
            for c in chunks:
                w.add_chunk(c)
            w.add_object(rng_key, rng_state)
            part = w.close()
            tmp = os.path.join(path, f".part_{rank}.pkl.tmp")
            with open(tmp, "wb") as f:
                pickle.dump(part, f)
            os.replace(tmp, os.path.join(path, f".part_{rank}.pkl"))
        except Exception as e:  # noqa: BLE001 - reported by the thread's owner
            h["error"] = repr(e)
            if not async_save:
                raise

    if async_save:
        h["thread"] = threading.Thread(target=write, daemon=True)
        h["thread"].start()
        _PENDING.append(h)
    else:
        write()
        _finish_save(h)
    return path


def _rotate(root, limit, retain_interval, async_delete):
    """Keeps the newest ``limit`` checkpoints plus every ``retain_interval``-th step; deletion runs off-thread."""
    if not limit:
        return
    steps = sorted(int(d.split("_")[1]) for d in os.listdir(root) if d.startswith("iter_") and d[5:].isdigit())
    victims = [s for s in steps[:-limit] if not (retain_interval and s % retain_interval == 0)]

    def rm():
        for s in victims:
            shutil.rmtree(iter_dir(root, s), ignore_errors=True)

    if async_delete:
        threading.Thread(target=rm, daemon=True).start()
    else:
        rm()


# ------------------------------------------------------------------------------------------------ reader
class CheckpointReader:
    def __init__(self, path: str):
        self.path = path
        with open(os.path.join(path, ".metadata"), "rb") as f:
            self.md: Metadata = pickle.load(f)
        self._files: Dict[str, object] = {}

    def keys(self):
        return list(self.md.state_dict_metadata.keys())

    def _read(self, info: _StorageInfo):
        f = self._files.get(info.relative_path)
        if f is None:
            f = open(os.path.join(self.path, info.relative_path), "rb")
            self._files[info.relative_path] = f
        f.seek(info.offset)
        return torch.load(io.BytesIO(f.read(info.length)), map_location="cpu", weights_only=False)

    def read_object(self, key: str):
        obj = self._read(self.md.storage_data[MetadataIndex(key)])
        if isinstance(obj, io.BytesIO):   # the object's own torch.save image (see ``_ShardWriter.add_object``)
            obj.seek(0)
            obj = torch.load(obj, map_location="cpu", weights_only=False)
        return obj

    def read_region(self, key: str, offset: Tuple[int, ...], shape: Tuple[int, ...]) -> torch.Tensor:
        """Assembles ``global[key][offset : offset + shape]`` from the stored chunks that overlap it."""
        tm = self.md.state_dict_metadata[key]
        out = torch.empty(shape, dtype=tm.properties.dtype)
        covered = 0
        for ch in tm.chunks:
            lo = [max(o, co) for o, co in zip(offset, ch.offsets)]
            hi = [min(o + s, co + cs) for o, s, co, cs in zip(offset, shape, ch.offsets, ch.sizes)]
            if any(h <= l for l, h in zip(lo, hi)):
                continue
            src = self._read(self.md.storage_data[MetadataIndex(key, ch.offsets)])
            src_sl = tuple(slice(l - co, h - co) for l, h, co in zip(lo, hi, ch.offsets))
            dst_sl = tuple(slice(l - o, h - o) for l, h, o in zip(lo, hi, offset))
            out[dst_sl] = src[src_sl]
            n = 1
            for l, h in zip(lo, hi):
                n *= h - l
            covered += n
        total = 1
        for s in shape:
            total *= s
        if covered < total:
            raise KeyError(f"checkpoint does not cover {key}[{offset}+{shape}] ({covered}/{total} elements)")
        return out

    def full_tensor(self, key: str) -> torch.Tensor:
        tm = self.md.state_dict_metadata[key]
        return self.read_region(key, (0,) * len(tm.size), tuple(tm.size))

    def close(self):
        for f in self._files.values():
            f.close()
        self._files.clear()


def load_checkpoint(engine, root: str, step: Optional[int] = None, load_optim: bool = True, load_rng: bool = True,
                    strict: bool = True) -> Optional[int]:
    """Loads ``iter_{step}`` (default: the latest).  Returns the step, or None when there is nothing to load."""
    if step is None:
        step = read_latest_step(root)
        if step is None:
            return None
    path = iter_dir(root, step)
    rd = CheckpointReader(path)
    model = engine.model
    tp_rank, tp = ps.get_tensor_model_parallel_rank(), model.tp_size
    ep_rank, ep = ps.get_expert_model_parallel_rank(), model.ep_size
    have = set(rd.keys())

    def fetch_with(prefix):
        def fetch(key, gshape, offset, shape):
            return rd.read_region(prefix + key, offset, shape)
        return fetch

    missing = []
    for name, p in model.named_parameters():
        name = _canonical(model, name)
        mode = getattr(p, "tp_mode", "none")
        probe = param_chunks(name, p.detach(), model.cfg, tp_rank if tp > 1 else 0, tp, ep_rank, ep, mode)
        # parameter paths carry no prefix; trees written by earlier versions of this package had "model." in front
        prefix = next((pre for pre in ("", "model.") if all((pre + c.key) in have for c in probe)), None)
        if prefix is None:
            missing.append(name)
            continue
        assign_from_chunks(name, p.data, model.cfg, tp_rank if tp > 1 else 0, tp, ep_rank, ep, mode,
                           fetch_with(prefix))
    if missing and strict:
        raise KeyError(f"checkpoint {path} lacks parameters: {missing[:8]}{'...' if len(missing) > 8 else ''}")
    common = torch.load(os.path.join(path, "common.pt"), map_location="cpu", weights_only=False)
    opt = engine.optimizer
    if opt is not None:
        has_opt = any(k.startswith("optimizer.state.") for k in have)
        if load_optim and has_opt:
            names = {id(p): _canonical(model, n) for n, p in model.named_parameters()}
            for sh in opt.shards:
                buf, bucket = sh["buf"], sh["bucket"]
                s, e = sh["s"], sh["e"]
                for p in bucket.params:
                    o = buf.offsets[id(p)]
                    lo, hi = max(o, s), min(o + p.numel(), e)
                    if hi <= lo:
                        continue
                    name, mode = names[id(p)], getattr(p, "tp_mode", "none")
                    for k, label in (("master", "fp32_param"), ("m", "exp_avg"), ("v", "exp_avg_sq")):
                        tmp = torch.empty(p.shape, dtype=torch.float32)
                        assign_from_chunks(name, tmp, model.cfg, tp_rank if tp > 1 else 0, tp, ep_rank, ep, mode,
                                           fetch_with(f"optimizer.state.{label}."))
                        sh[k][lo - s:hi - s].copy_(tmp.reshape(-1)[lo - o:hi - o])
            opt.step_count = common.get("optimizer_step", common.get("lr_scheduler", {}).get("num_steps", 0))
        else:
            opt.reload_master_from_params()
    engine.step = common.get("engine_step", step)
    if load_rng:
        pp = ps.get_pipeline_model_parallel_rank()
        dp = ps.get_data_parallel_rank(with_context_parallel=True)
        sizes = (ps.get_pipeline_model_parallel_world_size(), ps.get_tensor_model_parallel_world_size())
        for key in (rng_object_key(pp, tp_rank, *sizes, dp), rng_object_key(pp, tp_rank, *sizes, 0),
                    f"rng_state/shard_{pp}_{tp_rank}_{dp}"):
            if key in have:
                set_rng_state(rd.read_object(key))
                break
    rd.close()
    engine.loaded_extra_state = common.get("extra_state", {})
    return step
