"""GRPO with disaggregated placement: the trainer ranks run this trainer, the rollout ranks run
``rollout/disaggregated.py::SamplerServer``.  Same step as the colocated trainer (``grpo_trainer.py``) except that the
rollout phase asks the remote engines and the weight hand-over is a bucket broadcast to them
(``placement_type: disaggregated``; the reference's trainer drives remote sampler actors the same way:
gpatch_v4/trainer/grpo_trainer.py with gpatch_v4/client/update_weight_factory.py:381-445)."""
from __future__ import annotations

from types import SimpleNamespace
from typing import List, Optional, Sequence

import torch

from ..core import parallel_state as ps
from ..rollout.disaggregated import RemoteRollout, RoleLayout
from ..rollout.engine import SamplingParams
from .grpo_trainer import GrpoTrainer, response_mask


class DisaggGrpoTrainer(GrpoTrainer):
    def __init__(self, config, layout: RoleLayout, **kw):
        super().__init__(config, **kw)
        self.layout = layout
        self.remote = RemoteRollout(layout)

    def setup(self):
        cfg = self.cfg
        self.policy.setup_model_and_get_optimizer()
        ie = cfg.sampler.infer_engine_configs[0]
        self.policy.temperature = ie.temperature
        self.lora = bool(cfg.policy.lora.enabled)
        self.release_rollout_weights = False
        self.serve_fp8 = False
        self.engine = None
        self.sampling = SamplingParams(temperature=ie.temperature, top_k=ie.top_k, top_p=ie.top_p, min_p=ie.min_p, repetition_penalty=ie.repetition_penalty,
                                       max_new_tokens=ie.generate_max_tokens, seed=ie.seed,
                                       stop_token_ids=tuple(ie.generate_params.get("stop_token_ids", ())))
        if getattr(cfg.policy, "offload_ref_model", False):
            self.policy.offload_ref_model()
        self.policy.release_grad_buffers()
        self.update_weights()          # the rollout ranks start from the trainer's initial weights
        return self

    def rollout(self, prompts: Sequence, n: Optional[int] = None, sampling: Optional[dict] = None) -> List[dict]:
        t = self.cfg.training
        n = int(n or t.sampling_repeat_n)
        sp = SamplingParams(**{**self.sampling.__dict__, **(sampling or {}),
                               "seed": self.sampling.seed + self.ppo_step * 1000003})
        res = self.remote.generate(prompts, n, sp)
        samples = []
        dp_rank = ps.get_data_parallel_rank()
        for k, r in enumerate(res):
            toks = torch.tensor(r["prompt"] + r["out_tokens"], dtype=torch.int64)
            P, S = len(r["prompt"]), len(r["prompt"]) + len(r["out_tokens"])
            lp = torch.zeros(S, dtype=torch.float32)
            lp[P - 1:S - 1] = torch.tensor(r["out_logprobs"], dtype=torch.float32)
            samples.append(dict(tokens=toks, prompt_length=P, sequence_length=S, rollout_log_probs=lp,
                                group_id=k // n, unique_id=(self.ppo_step, dp_rank, k),
                                mask=response_mask(P, S), finish_reason=r["finish_reason"]))
        return samples

    def update_weights(self):
        self.last_transfer = self.remote.update_weights(
            self.policy, self.cfg.policy.sampler_client.update_weight_max_size_mb)

    def offload_model(self):
        pass

    def onload_model(self):
        pass

    def shutdown(self):
        self.remote.stop()
