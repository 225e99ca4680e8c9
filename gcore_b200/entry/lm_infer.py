"""Batch inference entry point (``gpatch_v4/entry`` infer / eval mains): loads a checkpoint (torch_dist or HF) into
the rollout engine and writes one jsonl line per prompt with the generated token ids and log-probs.

    python -m gcore_b200.entry.lm_infer --config rl.yaml +task.infer.prompts=prompts.jsonl +task.infer.out=out.jsonl
"""
import json
import sys

import torch

from ..configs.config import RlConfig
from ..trainer.grpo_trainer import GrpoTrainer
from .common import finalize, init_runtime, load


def main(argv=None):
    cfg = load(RlConfig, argv)
    init_runtime(cfg)
    tr = GrpoTrainer(cfg)
    tr.setup()
    inf = dict((cfg.task or {}).get("infer", {}) or {})
    if cfg.checkpoint.load_ckpt_path:
        from ..checkpoint.torch_dist import load_checkpoint, read_latest_step
        if read_latest_step(cfg.checkpoint.load_ckpt_path) is not None:
            load_checkpoint(tr.policy, cfg.checkpoint.load_ckpt_path, load_optim=False)
        else:
            from ..checkpoint.hf import load_hf
            load_hf(tr.policy, cfg.checkpoint.load_ckpt_path)
        tr.update_weights()
    prompts = [json.loads(l)["prompt_token_ids"] for l in open(inf["prompts"])] if inf.get("prompts") else \
        [torch.randint(100, 1000, (16,)).tolist() for _ in range(4)]
    out = tr.rollout(prompts)
    if inf.get("out"):
        with open(inf["out"], "w") as f:
            for s in out:
                f.write(json.dumps({"tokens": torch.as_tensor(s["tokens"]).tolist(),
                                    "prompt_length": int(s["prompt_length"])}) + "\n")
    finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
