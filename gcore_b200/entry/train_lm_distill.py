"""Distillation entry point (the reference's on-policy / off-policy distill mains under ``gpatch_v4/entry/``).

``distill_mode=on_policy`` (default): the student samples, a frozen teacher (``teacher:`` section) scores the samples
and the per-token advantage is the teacher - student log-prob gap (``ppo.advantage_type=on_policy_distill``,
``ppo.loss_func=opd``).  ``distill_mode=off_policy``: the teacher generates the responses and the student is trained
on them with the SFT loss.

``torchrun ... -m gcore_b200.entry.train_lm_distill --config distill.yaml +distill_mode=off_policy``"""
import sys

import torch

from ..configs.config import RlConfig
from ..rollout.engine import InferEngine, RolloutWeights, SamplingParams
from ..trainer.grpo_trainer import GrpoTrainer
from ..trainer.rl_loop import RlLoop
from ..utils.logging_utils import get_logger
from .common import finalize, init_runtime, load


def off_policy_loop(trainer: GrpoTrainer, prompt_batches, steps: int, log):
    """Teacher rollouts -> SFT on the student.  The teacher serves from its own engine (storage shared with the
    teacher's training-layout weights)."""
    cfg = trainer.cfg
    ie = cfg.sampler.infer_engine_configs[0]
    teacher = trainer.teacher
    eng = InferEngine(teacher.model_cfg, RolloutWeights.from_model(teacher.model), tp_size=teacher.model.tp_size,
                      max_running_requests=ie.max_running_requests or cfg.training.rollout_gbs,
                      max_model_len=ie.max_model_len or (cfg.data.max_prompt_length + ie.generate_max_tokens),
                      kv_block_size=ie.kv_block_size, use_cuda_graph=not ie.disable_cuda_graph, device=teacher.device)
    sp = SamplingParams(temperature=ie.temperature, top_k=ie.top_k, top_p=ie.top_p, min_p=ie.min_p, repetition_penalty=ie.repetition_penalty,
                        max_new_tokens=ie.generate_max_tokens, seed=ie.seed)
    history = []
    for step, prompts in zip(range(steps), prompt_batches):
        reqs = eng.generate(prompts, sp, n=1)
        samples = []
        for r in reqs:
            toks = torch.tensor(r.prompt + r.out_tokens, dtype=torch.int64)
            m = torch.zeros(toks.numel())
            m[len(r.prompt) - 1:toks.numel() - 1] = 1.0
            samples.append({"tokens": toks, "loss_mask": m, "prompt_length": len(r.prompt)})
        trainer.policy.allocate_grad_buffers()
        metrics = trainer.policy.finetune_step(samples)
        trainer.update_weights()
        history.append(metrics)
        log.info(f"step {step} lm_loss {metrics['lm_loss']:.4f}")
    return history


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    mode = "on_policy"
    for a in list(argv):
        if a.lstrip("+").startswith("distill_mode="):
            mode = a.split("=", 1)[1]
            argv.remove(a)
    cfg = load(RlConfig, argv)
    init_runtime(cfg)
    log = get_logger("distill")
    loop = RlLoop(cfg).setup()
    assert loop.trainer.teacher is not None, "distillation needs a `teacher:` section"
    if mode == "on_policy":
        history = loop.run()
    else:
        total = cfg.training.exit_step or cfg.training.total_ppo_step or 0
        history = off_policy_loop(loop.trainer, loop.prompt_iter, total, log)
    finalize()
    return history


if __name__ == "__main__":
    main()
    sys.exit(0)
