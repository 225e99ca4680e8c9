"""GPU budgeting per role and placement modes, as pure functions (testable without a cluster).

Mirrors ``allocation_from_config`` / ``ResourceAllocation.validate`` (gpatch_v4/orches/resource_allocator.py:157-347) and
the bundle slicing of ``create_placement_groups`` (gpatch_v4/orches/placement_group.py:235-383):
  colocate           every role uses the same GPUs (time-sharing)
  disaggregated      roles get disjoint GPU ranges: train | sampler | gen_rm | critic
  partial_colocated  sampler shares the train GPUs, reward-model engines get their own
Bundles are ordered by (node, gpu id); a rollout engine's TP group never straddles nodes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class RoleAllocation:
    role: str
    gpus: List[int]                 # global bundle indices
    tp: int = 1
    pp: int = 1
    cp: int = 1
    ep: int = 1

    @property
    def num_gpus(self):
        return len(self.gpus)

    @property
    def dp(self):
        return max(self.num_gpus // (self.tp * self.pp * self.cp), 1)

    def engines(self) -> List[List[int]]:
        """Rollout roles: one engine ("cluster") per TP group."""
        per = self.tp * self.pp
        return [self.gpus[i:i + per] for i in range(0, len(self.gpus), per)]


@dataclass
class ResourceAllocation:
    placement_type: str
    num_gpus_per_node: int
    nnodes: int
    roles: Dict[str, RoleAllocation] = field(default_factory=dict)

    @property
    def total_gpus(self):
        return self.num_gpus_per_node * self.nnodes

    def validate(self):
        for name, r in self.roles.items():
            mp = r.tp * r.pp * r.cp
            if r.num_gpus == 0 or r.num_gpus % mp:
                raise ValueError(f"role {name}: {r.num_gpus} GPUs is not a multiple of tp*pp*cp = {mp}")
            if any(g < 0 or g >= self.total_gpus for g in r.gpus):
                raise ValueError(f"role {name}: GPU index outside the {self.total_gpus}-GPU job")
            if name != "train":
                for eng in r.engines():
                    nodes = {g // self.num_gpus_per_node for g in eng}
                    if len(nodes) > 1:
                        raise ValueError(f"role {name}: engine {eng} straddles nodes")
                if r.pp != 1:
                    raise ValueError(f"role {name}: rollout engines require pipeline_model_parallel_size == 1")
        if self.placement_type == "disaggregated":
            seen: Dict[int, str] = {}
            for name, r in self.roles.items():
                for g in r.gpus:
                    if g in seen:
                        raise ValueError(f"disaggregated placement: GPU {g} assigned to both {seen[g]} and {name}")
                    seen[g] = name
        return self


def expected_nnodes(total_gpus_needed: int, num_gpus_per_node: int) -> int:
    return (total_gpus_needed + num_gpus_per_node - 1) // num_gpus_per_node


def _dist(cfg) -> Tuple[int, int, int, int]:
    return (cfg.tensor_model_parallel_size, cfg.pipeline_model_parallel_size, cfg.context_parallel_size,
            cfg.expert_model_parallel_size)


def allocation_from_config(config, nnodes: Optional[int] = None, role_gpus: Optional[Dict[str, int]] = None
                           ) -> ResourceAllocation:
    """``role_gpus`` gives the GPU count of each role for the non-colocated modes (default: an even split)."""
    d = config.policy.dist_config
    per_node = d.num_gpus_per_node
    n = nnodes if nnodes is not None else (d.nnodes if d.nnodes > 0 else 1)
    total = per_node * n
    alloc = ResourceAllocation(config.placement_type, per_node, n)
    tp, pp, cp, ep = _dist(d)
    roles = ["train", "sampler"]
    has_gen_rm = getattr(config, "gen_rm", None) is not None
    has_critic = getattr(config, "critic", None) is not None
    if has_gen_rm:
        roles.append("gen_rm")
    sd = config.sampler.infer_engine_configs[0].dist_config
    stp = sd.tensor_model_parallel_size
    if config.placement_type == "colocate":
        allg = list(range(total))
        alloc.roles["train"] = RoleAllocation("train", allg, tp, pp, cp, ep)
        alloc.roles["sampler"] = RoleAllocation("sampler", allg, stp)
        if has_gen_rm:
            gtp = config.gen_rm.infer_engine_configs[0].dist_config.tensor_model_parallel_size
            alloc.roles["gen_rm"] = RoleAllocation("gen_rm", allg, gtp)
        if has_critic:
            c = config.critic.dist_config
            alloc.roles["critic"] = RoleAllocation("critic", allg, *_dist(c))
    else:
        counts = dict(role_gpus or {})
        if config.placement_type == "partial_colocated":
            shared = counts.get("train", total // (2 if has_gen_rm else 1))
            alloc.roles["train"] = RoleAllocation("train", list(range(shared)), tp, pp, cp, ep)
            alloc.roles["sampler"] = RoleAllocation("sampler", list(range(shared)), stp)
            off = shared
            if has_gen_rm:
                gtp = config.gen_rm.infer_engine_configs[0].dist_config.tensor_model_parallel_size
                alloc.roles["gen_rm"] = RoleAllocation("gen_rm", list(range(off, total)), gtp)
        else:
            share = total // len(roles)
            off = 0
            for r in roles:
                k = counts.get(r, share)
                g = list(range(off, off + k))
                off += k
                if r == "train":
                    alloc.roles[r] = RoleAllocation(r, g, tp, pp, cp, ep)
                elif r == "sampler":
                    alloc.roles[r] = RoleAllocation(r, g, stp)
                else:
                    gtp = config.gen_rm.infer_engine_configs[0].dist_config.tensor_model_parallel_size
                    alloc.roles[r] = RoleAllocation(r, g, gtp)
    return alloc.validate()


def sort_bundles(probed: List[Tuple[str, int]]) -> List[int]:
    """Order bundle indices by (node ip, gpu id), the order the reference sorts its placement-group bundles in."""
    return [i for i, _ in sorted(enumerate(probed), key=lambda kv: (kv[1][0], kv[1][1]))]
