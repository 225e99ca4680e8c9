"""Process-group topology: TP x CP x DP x PP with an independent expert decomposition (ETP x EP x EDP x PP).

Rank order is ``tp-cp-ep-dp-pp`` (tensor-parallel fastest), the order the reference passes to Megatron's
``initialize_model_parallel`` (gpatch_v4/core/parallel_state.py:224-300).  Besides the NCCL groups it creates the
gloo side groups the reference adds for host barriers and pickled-object traffic (:295-298, :403-436) and the
combined model-parallel x context-parallel group used to broadcast rollout batches.

Everything is derived from ``torch.distributed`` only; on CPU the default backend is gloo, so the same code runs the
world-size-2 CPU tests.
"""
from __future__ import annotations

import datetime
import os
import random
from dataclasses import dataclass, field
from itertools import product
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist


@dataclass
class ParallelState:
    world_size: int = 1
    rank: int = 0
    tp: int = 1
    cp: int = 1
    dp: int = 1
    pp: int = 1
    ep: int = 1
    etp: int = 1
    edp: int = 1
    coords: Dict[str, int] = field(default_factory=dict)
    groups: Dict[str, Optional[dist.ProcessGroup]] = field(default_factory=dict)
    group_ranks: Dict[str, List[int]] = field(default_factory=dict)
    gloo_groups: Dict[str, Optional[dist.ProcessGroup]] = field(default_factory=dict)
    initialized: bool = False

    def group(self, name):
        return self.groups.get(name)

    def size(self, name):
        return len(self.group_ranks.get(name, [self.rank]))

    def rank_in(self, name):
        ranks = self.group_ranks.get(name, [self.rank])
        return ranks.index(self.rank)


_STATE = ParallelState()


def get_state() -> ParallelState:
    return _STATE


def _enumerate_groups(sizes: Dict[str, int], order: List[str], select: List[str]):
    """All rank lists obtained by varying the dims in ``select`` and fixing the others; ``order`` lists dims from
    fastest to slowest varying."""
    strides, s = {}, 1
    for d in order:
        strides[d] = s
        s *= sizes[d]
    others = [d for d in order if d not in select]
    out = []
    for fixed in product(*[range(sizes[d]) for d in others]):
        base = sum(strides[d] * v for d, v in zip(others, fixed))
        ranks = []
        sel_sorted = [d for d in order if d in select]  # fastest first
        for vals in product(*[range(sizes[d]) for d in reversed(sel_sorted)]):
            r = base + sum(strides[d] * v for d, v in zip(reversed(sel_sorted), vals))
            ranks.append(r)
        out.append(sorted(ranks))
    return out


def rank_coords(rank: int, sizes: Dict[str, int], order: List[str]) -> Dict[str, int]:
    c = {}
    for d in order:
        c[d] = rank % sizes[d]
        rank //= sizes[d]
    return c


def plan_groups(world_size: int, tp: int = 1, pp: int = 1, cp: int = 1, ep: int = 1, etp: Optional[int] = None):
    """Pure function (no process groups): returns ``{name: [rank lists]}`` for every group family.  Used by
    ``initialize_model_parallel`` and directly by the placement / planning tests."""
    # experts are never tensor-sharded in this package: every TP rank holds whole experts and routes the tokens of its
    # own sequence-parallel shard, so by default the TP ranks belong to the expert-data-parallel group (their expert
    # gradients are summed like those of data-parallel replicas)
    etp = etp if etp is not None else 1
    if world_size % (tp * pp * cp):
        raise ValueError(f"world_size {world_size} not divisible by tp*pp*cp = {tp * pp * cp}")
    dp = world_size // (tp * pp * cp)
    if world_size % (etp * ep * pp):
        raise ValueError(f"world_size {world_size} not divisible by etp*ep*pp = {etp * ep * pp}")
    edp = world_size // (etp * ep * pp)
    if (dp * cp * tp) % (ep * etp):
        raise ValueError("expert parallel size must divide dp*cp*tp/etp")
    dense = {"tp": tp, "cp": cp, "dp": dp, "pp": pp}
    order = ["tp", "cp", "dp", "pp"]
    fam = {
        "tp": _enumerate_groups(dense, order, ["tp"]),
        "cp": _enumerate_groups(dense, order, ["cp"]),
        "dp": _enumerate_groups(dense, order, ["dp"]),
        "pp": _enumerate_groups(dense, order, ["pp"]),
        # a second communicator over the same ranks: gradients travel on it, so that with two stages (where the next
        # and the previous stage are the same peer) forward and backward messages never share a FIFO
        "pp_bwd": _enumerate_groups(dense, order, ["pp"]),
        # interleaved stages close the ring (last stage -> first stage); that traffic gets communicators of its own so
        # that on each communicator the send / receive dependencies form a line, never a cycle: a send that has to
        # wait for its receiver then cannot hold up the receive its receiver is waiting for
        "pp_wrap": _enumerate_groups(dense, order, ["pp"]),
        "pp_bwd_wrap": _enumerate_groups(dense, order, ["pp"]),
        "dp_cp": _enumerate_groups(dense, order, ["dp", "cp"]),
        "tp_cp": _enumerate_groups(dense, order, ["tp", "cp"]),
        "mp": _enumerate_groups(dense, order, ["tp", "pp"]),
        "mp_cp": _enumerate_groups(dense, order, ["tp", "pp", "cp"]),
        "tp_dp_cp": _enumerate_groups(dense, order, ["tp", "dp", "cp"]),
    }
    expert = {"etp": etp, "ep": ep, "edp": edp, "pp": pp}
    eorder = ["etp", "ep", "edp", "pp"]
    fam.update({
        "etp": _enumerate_groups(expert, eorder, ["etp"]),
        "ep": _enumerate_groups(expert, eorder, ["ep"]),
        "edp": _enumerate_groups(expert, eorder, ["edp"]),
        "etp_ep": _enumerate_groups(expert, eorder, ["etp", "ep"]),
    })
    return fam, dense, expert


def initialize_model_parallel(tp: int = 1, pp: int = 1, cp: int = 1, ep: int = 1, etp: Optional[int] = None,
                              create_gloo: bool = True, timeout_minutes: int = 30,
                              ranks: Optional[List[int]] = None) -> ParallelState:
    """``ranks``: the ranks of the default group that form this role's world (disaggregated placement: trainer ranks
    and rollout ranks each lay out their own parallel groups inside their slice).  Every rank of the default group must
    make the call, with the same arguments, because group creation is collective; a rank outside ``ranks`` takes part
    in the creation and keeps the state it had."""
    global _STATE
    assert dist.is_initialized(), "call init_distributed() first"
    rank = dist.get_rank()
    world_ranks = list(ranks) if ranks is not None else list(range(dist.get_world_size()))
    world = len(world_ranks)
    member = rank in world_ranks
    fam, dense, expert = plan_groups(world, tp, pp, cp, ep, etp)
    local = world_ranks.index(rank) if member else 0
    st = ParallelState(world_size=world, rank=rank, tp=tp, cp=cp, dp=dense["dp"], pp=pp, ep=ep,
                       etp=expert["etp"], edp=expert["edp"])
    st.coords = rank_coords(local, dense, ["tp", "cp", "dp", "pp"])
    st.coords.update(rank_coords(local, expert, ["etp", "ep", "edp", "pp"]))
    timeout = datetime.timedelta(minutes=timeout_minutes)
    backend_is_nccl = dist.get_backend() == "nccl"
    for name, lists in fam.items():
        for idx in lists:
            grp = [world_ranks[i] for i in idx]
            # every rank must create every group, in the same order
            g = dist.new_group(grp, timeout=timeout) if len(grp) > 1 else None
            gg = None
            if create_gloo and backend_is_nccl and name in ("dp", "mp", "mp_cp", "dp_cp", "tp") and len(grp) > 1:
                gg = dist.new_group(grp, backend="gloo", timeout=timeout)
            if member and rank in grp:
                st.groups[name] = g
                st.group_ranks[name] = grp
                st.gloo_groups[name] = gg if gg is not None else g
    if ranks is None:
        st.groups["world"] = dist.group.WORLD
    else:
        st.groups["world"] = dist.new_group(world_ranks, timeout=timeout)   # also for a one-rank role: passing no
        # group to a collective would address the default group, i.e. both roles
    st.group_ranks["world"] = world_ranks
    if create_gloo and backend_is_nccl:
        st.gloo_groups["world"] = dist.new_group(world_ranks, backend="gloo", timeout=timeout)
    else:
        st.gloo_groups["world"] = st.groups["world"]
    if not member:
        return _STATE
    st.initialized = True
    st.sub_world = ranks is not None
    _STATE = st
    return st


def get_world_group():
    """The group of all ranks of this role (the default group unless the job runs disaggregated roles)."""
    st = _STATE
    if st.initialized and getattr(st, "sub_world", False):
        return st.groups["world"]
    return dist.group.WORLD if dist.is_initialized() else None


def get_world_size() -> int:
    st = _STATE
    if st.initialized:
        return st.world_size
    return dist.get_world_size() if dist.is_initialized() else 1


def offload_process_groups() -> int:
    """Destroys the model-parallel communicators of the default backend (their device buffers return to the
    allocator while the rollout engine owns the GPU; ``policy.offload_process_group``,
    gpatch_v4/utils/reloadable_process_group.py:116-287).  Collective.  The gloo side groups and the default group
    stay.  Returns the number of groups destroyed."""
    st = _STATE
    assert st.initialized
    n = 0
    for name, g in list(st.groups.items()):
        if name == "world" or g is None:
            continue
        same = st.gloo_groups.get(name) is g
        dist.destroy_process_group(g)
        st.groups[name] = None
        if same:
            st.gloo_groups[name] = None
        n += 1
    st.offloaded = True
    return n


def reload_process_groups(timeout_minutes: int = 30) -> int:
    """Re-creates what ``offload_process_groups`` destroyed: every rank walks the same group plan in the same order
    (``dist.new_group`` is collective over the default group)."""
    st = _STATE
    if not getattr(st, "offloaded", False):
        return 0
    fam, _, _ = plan_groups(st.world_size, st.tp, st.pp, st.cp, st.ep, st.etp)
    timeout = datetime.timedelta(minutes=timeout_minutes)
    world_ranks = st.group_ranks["world"]
    me = st.rank
    n = 0
    for name, lists in fam.items():
        for idx in lists:
            ranks = [world_ranks[i] for i in idx]
            g = dist.new_group(ranks, timeout=timeout) if len(ranks) > 1 else None
            if me in ranks and g is not None:
                st.groups[name] = g
                if st.gloo_groups.get(name) is None:
                    st.gloo_groups[name] = g
                n += 1
    st.offloaded = False
    return n


def destroy_model_parallel():
    global _STATE
    _STATE = ParallelState()


def init_distributed(backend: Optional[str] = None, timeout_minutes: int = 30):
    """Joins the default process group from the torchrun environment (RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT)
    and selects this process's GPU."""
    if dist.is_initialized():
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    kwargs = {}
    if backend == "nccl":
        torch.cuda.set_device(local)
        kwargs["device_id"] = torch.device("cuda", local)
    dist.init_process_group(backend, rank=rank, world_size=world,
                            timeout=datetime.timedelta(minutes=timeout_minutes), **kwargs)


# ------------------------------------------------------------------------------------------------ accessors
def _size(name):
    return _STATE.size(name) if _STATE.initialized else 1


def _rank(name):
    return _STATE.rank_in(name) if _STATE.initialized else 0


def get_tensor_model_parallel_group():
    return _STATE.group("tp")


def get_tensor_model_parallel_world_size():
    return _size("tp")


def get_tensor_model_parallel_rank():
    return _rank("tp")


def get_pipeline_model_parallel_group():
    return _STATE.group("pp")


def get_pipeline_backward_group():
    return _STATE.group("pp_bwd")


def get_pipeline_wrap_groups():
    return _STATE.group("pp_wrap"), _STATE.group("pp_bwd_wrap")


def get_pipeline_model_parallel_world_size():
    return _size("pp")


def get_pipeline_model_parallel_rank():
    return _rank("pp")


def get_context_parallel_group():
    return _STATE.group("cp")


def get_context_parallel_world_size():
    return _size("cp")


def get_context_parallel_rank():
    return _rank("cp")


def get_data_parallel_group(with_context_parallel: bool = False):
    return _STATE.group("dp_cp" if with_context_parallel else "dp")


def get_data_parallel_world_size(with_context_parallel: bool = False):
    return _size("dp_cp" if with_context_parallel else "dp")


def get_data_parallel_rank(with_context_parallel: bool = False):
    return _rank("dp_cp" if with_context_parallel else "dp")


def get_expert_model_parallel_group():
    return _STATE.group("ep")


def get_expert_model_parallel_world_size():
    return _size("ep")


def get_expert_model_parallel_rank():
    return _rank("ep")


def get_expert_data_parallel_group():
    return _STATE.group("edp")


def get_model_parallel_group(with_context_parallel: bool = False):
    return _STATE.group("mp_cp" if with_context_parallel else "mp")


def get_gloo_group(name: str = "world"):
    return _STATE.gloo_groups.get(name)


def is_pipeline_first_stage():
    return get_pipeline_model_parallel_rank() == 0


def is_pipeline_last_stage():
    return get_pipeline_model_parallel_rank() == get_pipeline_model_parallel_world_size() - 1


def is_mp_cp_head() -> bool:
    """True on the one rank of each model-parallel x context-parallel group that talks to the rollout side."""
    return _rank("mp_cp") == 0


def is_last_rank() -> bool:
    """Last rank of this role's world (the reporting rank)."""
    if not dist.is_initialized():
        return True
    st = _STATE
    if st.initialized and st.group_ranks.get("world"):
        return dist.get_rank() == st.group_ranks["world"][-1]
    return dist.get_rank() == dist.get_world_size() - 1


def cpu_barrier(name: str = "world"):
    """Host-side barrier on a gloo group (does not touch the GPU streams)."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        g = get_gloo_group(name)
        dist.barrier(group=g)


# ------------------------------------------------------------------------------------------------ seeds / determinism
def set_seed(seed: int, tp_offset: bool = False):
    """Same seed on every rank of a model-parallel group unless ``tp_offset`` (dropout inside TP regions)."""
    s = seed + (100 * get_pipeline_model_parallel_rank())
    if tp_offset:
        s += 2718 + get_tensor_model_parallel_rank()
    random.seed(s)
    np.random.seed(s % (2 ** 32))
    torch.manual_seed(s)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(s)


def apply_deterministic_mode():
    """One switch for bit-wise reruns (gpatch_v4/core/parallel_state.py:160-195): deterministic torch algorithms,
    ring-only NCCL, no TF32, deterministic attention backward (the native backward is atomic-free already)."""
    os.environ["NCCL_ALGO"] = "Ring"
    os.environ["CUBLAS_WORKSPACE_CONFIG"] = ":4096:8"
    os.environ["GCORE_B200_DETERMINISTIC"] = "1"
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.use_deterministic_algorithms(True, warn_only=True)
