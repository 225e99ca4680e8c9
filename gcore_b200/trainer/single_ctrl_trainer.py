"""Single-controller (asynchronous) GRPO: rollout and training overlap through ``RolloutController``; the batch
trained at step k may have been generated with weights up to ``rollout_max_staleness`` steps old, and the rollout
log-probs recorded at generation time feed the off-policy correction
(gpatch_v4/trainer/grpo_single_ctrl_trainer.py:17-200, docs of the async step API in actor/grpo_train_actor.py).

In the colocated SPMD layout the sampler endpoint is this rank's own ``InferEngine`` (generation and training then
alternate on the GPU, and the controller provides the staleness / tail-batching logic); with disaggregated sampler
processes the endpoints are ``SamplerClient`` objects over HTTP and generation truly overlaps training.
"""
from __future__ import annotations

from typing import Dict, Iterator, List, Optional

from ..rollout_generator.async_rollout import RolloutController
from .grpo_trainer import GrpoTrainer


class _LocalSampler:
    """Adapts ``GrpoTrainer.rollout`` to the controller's sampler interface.  The controller hands over every prompt
    group it fires in a round at once, so the colocated engine decodes all of them in one continuous batch."""

    def __init__(self, trainer: GrpoTrainer):
        self.tr = trainer

    def generate_groups(self, prompts, repeat_n, params=None):
        return self.tr.rollout(list(prompts), n=repeat_n)

    def generate(self, prompts, params=None):
        return self.tr.rollout([prompts[0]], n=len(prompts))


class GrpoSingleCtrlTrainer:
    def __init__(self, config, prompt_iter: Iterator, model_cfg=None, reward_fn=None, samplers: Optional[List] = None):
        self.cfg = config
        self.tr = GrpoTrainer(config, model_cfg=model_cfg, reward_fn=reward_fn)
        self.prompt_iter = prompt_iter
        self._samplers = samplers
        self.controller: Optional[RolloutController] = None

    def setup(self):
        self.tr.setup()
        t = self.cfg.training
        samplers = self._samplers or [_LocalSampler(self.tr)]
        from ..core import parallel_state as ps
        groups = max(t.rollout_gbs // max(ps.get_data_parallel_world_size(), 1), 1)
        self.controller = RolloutController(self.prompt_iter, samplers, self.tr.score, t.sampling_repeat_n, groups,
                                            max_staleness=t.rollout_max_staleness,
                                            keep_stale=self.cfg.ppo.offpolicy_correction != "none",
                                            over_dispatch_ratio=t.rollout_over_dispatch_ratio,
                                            reuse_unused_prompts=t.rollout_reuse_unused_prompts)
        return self

    def step(self) -> Dict[str, float]:
        c = self.controller
        c.set_weight_version(self.tr.ppo_step)
        samples = c.collect()
        m = self.tr.train_on_samples(samples)
        m["rollout-metrics/weight_staleness"] = float(max(self.tr.ppo_step - 1 - s.get("weight_version", 0)
                                                          for s in samples))
        m.update({f"controller/{k}": float(v) for k, v in c.stats.items()})
        return m

    def run(self, steps: int) -> List[Dict[str, float]]:
        return [self.step() for _ in range(steps)]
