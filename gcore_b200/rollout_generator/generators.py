"""Rollout strategies on top of ``GrpoTrainer.rollout`` / ``score``:

* ``BaseRolloutGenerator``      - fixed: ``rollout_gbs`` prompts x ``sampling_repeat_n`` samples, keep-n of repeat-n.
* ``DynamicSamplingGenerator``  - DAPO-style: drop prompt groups whose rewards are all equal (no learning signal),
  track the kept ratio with an EMA and refill up to ``max_refill_times``
  (gpatch_v4/rollout_generator/ds_generator.py; docs/source/dynamic_sampling.md:46-82).
* ``StaleRolloutQueue``         - sliding pipeline of the single-controller trainer: the batch trained at step k was
  generated with the weights of step k - s (``rollout_max_staleness = s``,
  gpatch_v4/trainer/grpo_single_ctrl_trainer.py:26-31); off-policy correction consumes ``rollout_log_probs``.
"""
from __future__ import annotations

from collections import deque
from typing import Callable, List, Optional, Sequence

import torch

from ..configs.base import import_from_path


def keep_n_of_group(samples: List[dict], repeat_n: int, keep_n: int, strategy: str = "all") -> List[dict]:
    if keep_n >= repeat_n or strategy == "all":
        return samples
    out = []
    for g0 in range(0, len(samples), repeat_n):
        grp = samples[g0:g0 + repeat_n]
        if strategy == "top":
            grp = sorted(grp, key=lambda s: -float(torch.as_tensor(s["rewards"]).sum()))[:keep_n]
        elif strategy == "extremes":
            srt = sorted(grp, key=lambda s: float(torch.as_tensor(s["rewards"]).sum()))
            grp = srt[:keep_n // 2] + srt[-(keep_n - keep_n // 2):]
        else:
            grp = grp[:keep_n]
        out.extend(grp)
    return out


def default_group_filter(group: List[dict]) -> bool:
    """Keep a prompt group only when its rewards are not all identical."""
    r = [float(torch.as_tensor(s["rewards"]).sum()) for s in group]
    return max(r) - min(r) > 1e-8


class BaseRolloutGenerator:
    def __init__(self, trainer, config):
        self.tr, self.cfg = trainer, config
        t = config.training
        self.filter_fn: Optional[Callable] = None
        if t.filter_sampling_py_path:
            self.filter_fn = import_from_path(t.filter_sampling_py_path, t.filter_sampling_fn_name or "filter_fn")

    def __call__(self, prompt_iter, step: int) -> List[dict]:
        t = self.cfg.training
        prompts = next(prompt_iter)
        samples = self.tr.score(self.tr.rollout(prompts))
        if self.filter_fn is not None and t.filter_sampling_stage == "pre":
            samples = self.filter_fn(samples)
        return keep_n_of_group(samples, t.sampling_repeat_n, t.sampling_keep_n, t.sampling_keeping_strategy)

    def state_dict(self):
        return {}

    def load_state_dict(self, sd):
        pass


class DynamicSamplingGenerator(BaseRolloutGenerator):
    def __init__(self, trainer, config, group_filter: Callable = default_group_filter):
        super().__init__(trainer, config)
        ds = config.training.dynamic_sampling
        self.ds = ds
        self.group_filter = group_filter
        if ds.filter_py_path:
            self.group_filter = import_from_path(ds.filter_py_path, ds.filter_fn_name or "filter_group")
        self.keep_ratio_ema = 1.0 / max(ds.oversampling_ratio, 1.0)
        self.stats = {"refills": 0, "kept_groups": 0, "seen_groups": 0}

    def __call__(self, prompt_iter, step: int) -> List[dict]:
        t, ds = self.cfg.training, self.ds
        n = t.sampling_repeat_n
        kept: List[dict] = []
        target_groups = None
        samples: List[dict] = []
        for _ in range(ds.max_refill_times + 1):
            prompts = next(prompt_iter)
            if target_groups is None:
                target_groups = len(prompts)
            samples = self.tr.score(self.tr.rollout(prompts))
            groups = [samples[i:i + n] for i in range(0, len(samples), n)]
            good = [g for g in groups if self.group_filter(g)]
            self.stats["seen_groups"] += len(groups)
            self.stats["kept_groups"] += len(good)
            ratio = len(good) / max(len(groups), 1)
            self.keep_ratio_ema = ds.ema_decay * self.keep_ratio_ema + (1 - ds.ema_decay) * ratio
            for g in good:
                if len(kept) < target_groups * n:
                    kept.extend(g)
            if len(kept) >= target_groups * n:
                break
            self.stats["refills"] += 1
        if not kept:  # nothing informative after all refills: fall back to the last batch so the step still runs
            kept = samples[:target_groups * n]
        for gi in range(0, len(kept), n):
            for s in kept[gi:gi + n]:
                s["group_id"] = gi // n
        return kept

    def suggested_oversampling(self) -> float:
        return min(max(1.0 / max(self.keep_ratio_ema, 1e-3), 1.0), 8.0)

    def state_dict(self):
        return {"keep_ratio_ema": self.keep_ratio_ema, "stats": dict(self.stats)}

    def load_state_dict(self, sd):
        self.keep_ratio_ema = sd.get("keep_ratio_ema", self.keep_ratio_ema)
        self.stats.update(sd.get("stats", {}))


class StaleRolloutQueue:
    """Holds ``staleness + 1`` generated batches; ``push`` after generating with the current weights, ``pop`` returns
    the oldest.  With staleness 0 this is a pass-through."""

    def __init__(self, staleness: int):
        self.s = staleness
        self.q: deque = deque()

    def primed(self) -> bool:
        return len(self.q) > self.s

    def push(self, samples: List[dict], weight_version: int):
        for x in samples:
            x["weight_version"] = weight_version
        self.q.append(samples)

    def pop(self) -> List[dict]:
        return self.q.popleft()


# ------------------------------------------------------------------------------------------------ record / replay
def _to_jsonable(s: dict) -> dict:
    out = {}
    for k, v in s.items():
        if isinstance(v, torch.Tensor):
            out[k] = {"__tensor__": v.tolist(), "dtype": str(v.dtype).replace("torch.", "")}
        elif isinstance(v, tuple):
            out[k] = {"__tuple__": list(v)}
        elif isinstance(v, (int, float, str, bool, list, dict)) or v is None:
            out[k] = v
    return out


def _from_jsonable(d: dict) -> dict:
    out = {}
    for k, v in d.items():
        if isinstance(v, dict) and "__tensor__" in v:
            out[k] = torch.tensor(v["__tensor__"], dtype=getattr(torch, v["dtype"]))
        elif isinstance(v, dict) and "__tuple__" in v:
            out[k] = tuple(v["__tuple__"])
        else:
            out[k] = v
    return out


class RecordingGenerator(BaseRolloutGenerator):
    """Wraps another generator and appends every batch it returns to a jsonl file (one line per step)."""

    def __init__(self, trainer, config, inner: BaseRolloutGenerator, path: str):
        super().__init__(trainer, config)
        self.inner, self.path = inner, path

    def __call__(self, prompt_iter, step: int) -> List[dict]:
        import json
        samples = self.inner(prompt_iter, step)
        with open(self.path, "a") as f:
            f.write(json.dumps({"step": step, "samples": [_to_jsonable(s) for s in samples]}) + "\n")
        return samples

    def state_dict(self):
        return self.inner.state_dict()

    def load_state_dict(self, sd):
        self.inner.load_state_dict(sd)


class ReplayRolloutGenerator(BaseRolloutGenerator):
    """Feeds recorded rollouts (tokens, masks, rollout log-probs, rewards) back to the trainer instead of sampling:
    reproduces a run's training phases without the rollout engine, or trains on rollouts made elsewhere
    (the reference's replay generator under ``gpatch_v4/rollout_generator/``).  Resumes at the recorded position."""

    def __init__(self, trainer, config, path: str, loop: bool = False):
        super().__init__(trainer, config)
        self.path, self.loop, self.pos = path, loop, 0
        from ..data.datasets import IndexedJsonlDataset
        self.rows = IndexedJsonlDataset(path)

    def __call__(self, prompt_iter, step: int) -> List[dict]:
        if self.pos >= len(self.rows):
            if not self.loop:
                raise StopIteration(f"replay file {self.path} has {len(self.rows)} steps")
            self.pos = 0
        row = self.rows[self.pos]
        self.pos += 1
        return [_from_jsonable(s) for s in row["samples"]]

    def state_dict(self):
        return {"pos": self.pos}

    def load_state_dict(self, sd):
        self.pos = int(sd.get("pos", 0))


class ExternalRolloutGenerator(BaseRolloutGenerator):
    """Rollouts come from a user function ``fn(prompts, step, trainer) -> samples`` (another serving stack, a tool
    loop, an agentic environment); the samples are scored and filtered like the engine's own
    (``policy.rollout_gen_py_path`` / ``policy.rollout_gen_cls`` name the function)."""

    def __init__(self, trainer, config, fn: Optional[Callable] = None):
        super().__init__(trainer, config)
        p = config.policy
        self.fn = fn or import_from_path(p.rollout_gen_py_path, p.rollout_gen_cls or "generate")

    def __call__(self, prompt_iter, step: int) -> List[dict]:
        t = self.cfg.training
        samples = self.fn(next(prompt_iter), step, self.tr)
        if samples and "rewards" not in samples[0]:
            samples = self.tr.score(samples)
        return keep_n_of_group(samples, t.sampling_repeat_n, t.sampling_keep_n, t.sampling_keeping_strategy)


def build_generator(trainer, config) -> BaseRolloutGenerator:
    """``policy.rollout_gen_type``: base | dynamic | replay | external | two_turn_reflect | agentic; ``training.dynamic_sampling.enable`` selects
    dynamic as before.  ``task.rollout.{replay_path, record_path, replay_loop, reflect_tokens, reflect_top_k}`` configure them."""
    kind = config.policy.rollout_gen_type or "base"
    opt = dict((config.task or {}).get("rollout", {}) or {})
    dbg = config.debug
    if getattr(dbg, "replay_rollout_path", None):      # debug.replay_rollout_path / dump_rollout_path: same machinery
        kind, opt["replay_path"] = "replay", dbg.replay_rollout_path
    if getattr(dbg, "dump_rollout_path", None):
        opt.setdefault("record_path", dbg.dump_rollout_path)
    if kind == "replay":
        gen: BaseRolloutGenerator = ReplayRolloutGenerator(trainer, config, opt["replay_path"],
                                                           bool(opt.get("replay_loop", False)))
    elif kind == "external":
        gen = ExternalRolloutGenerator(trainer, config)
    elif kind == "agentic":
        from ..agentic import make_env

        class _ByteTok:   # stands in when the job has no tokenizer (synthetic runs)
            def encode(self, t):
                return [b % 250 + 3 for b in t.encode("utf-8")]

            def decode(self, ids):
                return bytes((i - 3) % 250 for i in ids).decode("latin-1")

        env_name, env_kw = opt.get("env", "frozen_lake"), dict(opt.get("env_kwargs", {}) or {})
        gen = AgenticRolloutGenerator(trainer, config, lambda: make_env(env_name, **env_kw),
                                      getattr(trainer, "tokenizer", None) or _ByteTok(),
                                      int(opt.get("max_turns", 4)), opt.get("max_new_tokens"))
    elif kind == "two_turn_reflect":
        gen = TwoTurnReflectGenerator(trainer, config, opt.get("reflect_tokens", []), int(opt.get("reflect_top_k", 1)))
    elif kind == "dynamic" or config.training.dynamic_sampling.enable:
        gen = DynamicSamplingGenerator(trainer, config)
    else:
        gen = BaseRolloutGenerator(trainer, config)
    if opt.get("record_path"):
        gen = RecordingGenerator(trainer, config, gen, opt["record_path"])
    return gen


class TwoTurnReflectGenerator(BaseRolloutGenerator):
    """Second-turn reflection: after the first-turn samples of a prompt are scored, its ``top_k`` best and ``top_k``
    worst responses each get a follow-up turn - the first-turn conversation plus ``reflect_tokens`` (a user message
    asking the model to reconsider) - and the model answers again.  The batch then holds the first-turn samples and
    the second-turn samples, ``1 + 2 * top_k`` rollout batches per prompt batch, each second-turn group normalised on
    its own (the reference's two-turn reflect agent loop: ``reflect_prompt`` / ``reflect_top_k`` / ``rb_multiplier``,
    gpatch_v4/configs/training_config.py:977-986).  The first turn is context, not a target, in the second turn."""

    def __init__(self, trainer, config, reflect_tokens: Sequence[int], top_k: int = 1):
        super().__init__(trainer, config)
        self.reflect_tokens, self.top_k = list(reflect_tokens), max(int(top_k), 1)

    @property
    def rb_multiplier(self) -> int:
        return 1 + 2 * self.top_k

    def __call__(self, prompt_iter, step: int) -> List[dict]:
        t = self.cfg.training
        n = t.sampling_repeat_n
        first = self.tr.score(self.tr.rollout(next(prompt_iter)))
        groups = [first[i:i + n] for i in range(0, len(first), n)]
        follow = []   # (origin sample, kind)
        for g in groups:
            srt = sorted(g, key=lambda s: float(torch.as_tensor(s["rewards"]).sum()))
            k = min(self.top_k, len(srt) // 2 or 1)
            follow += [(s, "worst") for s in srt[:k]] + [(s, "best") for s in srt[-k:]]
        prompts2 = [torch.as_tensor(s["tokens"]).tolist() + self.reflect_tokens for s, _ in follow]
        second = self.tr.score(self.tr.rollout(prompts2)) if prompts2 else []
        base_gid = len(groups)
        for j, (origin, kind) in enumerate(follow):
            for s in second[j * n:(j + 1) * n]:
                s["group_id"] = base_gid + j
                s["turn"], s["reflect_of"], s["reflect_kind"] = 2, origin.get("unique_id"), kind
        for s in first:
            s["turn"] = 1
        return first + second


class AgenticRolloutGenerator(BaseRolloutGenerator):
    """Multi-turn environment rollouts instead of single-turn prompts: every group runs ``sampling_repeat_n``
    trajectories of one environment seed through ``agentic.TrajEnvManager`` (the policy is the trainer's rollout
    engine, one generate call per turn), and the trajectory's tokens / assistant-token mask / rollout log-probs /
    episode reward become one training sample.  With a ``teacher:`` section and
    ``advantage_type=on_policy_distill`` this is agentic distillation: the teacher scores the student's trajectories
    token by token (the reference's agent loop actors and agentic distill trainer)."""

    def __init__(self, trainer, config, env_factory: Callable, tokenizer, max_turns: int = 4,
                 max_new_tokens: Optional[int] = None):
        super().__init__(trainer, config)
        self.env_factory, self.tok, self.max_turns, self.max_new = env_factory, tokenizer, max_turns, max_new_tokens
        self.seed = 0

    def _generate(self, ctx: List[int]) -> dict:
        from ..rollout.engine import SamplingParams
        tr = self.tr
        sp = SamplingParams(**{**tr.sampling.__dict__, "seed": tr.sampling.seed + self.seed * 7919 + len(ctx),
                               "max_new_tokens": self.max_new or tr.sampling.max_new_tokens})
        r = tr.engine.generate([ctx], sp, n=1)[0]
        return {"token_ids": r.out_tokens, "logprobs": r.out_logprobs}

    def __call__(self, prompt_iter, step: int) -> List[dict]:
        from ..agentic import TrajEnvManager
        t = self.cfg.training
        groups = max(t.rollout_gbs, 1)
        self.tr.engine.wake_up(("kv_cache",))
        samples = []
        for g in range(groups):
            env_seed = step * 100003 + g
            for j in range(t.sampling_repeat_n):
                self.seed += 1
                mgr = TrajEnvManager(self.env_factory(), self.tok, self._generate, max_turns=self.max_turns,
                                     max_context_tokens=self.tr.engine.max_model_len - (self.max_new or
                                                                                        self.tr.sampling.max_new_tokens),
                                     group_id=g, traj_id=j)
                s = mgr.run(env_seed, step)
                toks = torch.as_tensor(s["tokens"], dtype=torch.int64)
                s.update(tokens=toks, sequence_length=int(toks.numel()), rewards=torch.tensor(float(s["reward"])),
                         unique_id=(step, g, j), finish_reason="env")
                if "rollout_log_probs" in s:
                    s["rollout_log_probs"] = torch.as_tensor(s["rollout_log_probs"], dtype=torch.float32)
                samples.append(s)
        self.tr.engine.sleep(("kv_cache",))
        return samples

    def state_dict(self):
        return {"seed": self.seed}

    def load_state_dict(self, sd):
        self.seed = int(sd.get("seed", 0))
