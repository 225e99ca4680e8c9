"""Evaluation entry point (the reference's eval main over ``gpatch_v4/evaluate/evaluate_runner.py``): loads a
checkpoint (torch_dist or HF) into the colocated rollout engine, samples ``training.sampling_repeat_n`` responses for
``eval.batches`` batches of prompts, scores them with the job's reward function and reports mean reward, pass@k and
response length over all data-parallel ranks.

    python -m gcore_b200.entry.lm_eval --config rl.yaml +task.eval.batches=4 +task.eval.ks=[1,4] +task.eval.out=metrics.json
"""
import json
import sys

from ..configs.config import RlConfig
from ..core import parallel_state as ps
from ..evaluate.runner import EvaluateRunner
from ..trainer.rl_loop import RlLoop
from .common import finalize, init_runtime, load


def main(argv=None):
    cfg = load(RlConfig, argv)
    init_runtime(cfg)
    loop = RlLoop(cfg).setup()
    tr = loop.trainer
    ev = dict((cfg.task or {}).get("eval", {}) or {})
    ck = cfg.checkpoint.load_ckpt_path
    if ck:
        from ..checkpoint.torch_dist import read_latest_step
        if read_latest_step(ck) is None:   # not a torch_dist tree (RlLoop.setup loaded it otherwise): HF safetensors
            from ..checkpoint.hf import load_hf
            load_hf(tr.policy, ck)
        tr.update_weights()
    n = cfg.training.sampling_repeat_n
    runner = EvaluateRunner(tr.rollout, lambda s: [float(x["rewards"]) for x in tr.score(s)], n,
                            ks=tuple(ev.get("ks", (1,))), threshold=float(ev.get("threshold", 0.5)),
                            dp_group=ps.get_data_parallel_group())
    prompts = []
    for _ in range(int(ev.get("batches", 1))):
        prompts += next(loop.prompt_iter)
    metrics = runner.run(prompts)
    if ev.get("out") and ps.is_last_rank():
        json.dump(metrics, open(ev["out"], "w"))
    print(metrics)
    finalize()
    return metrics


if __name__ == "__main__":
    main()
    sys.exit(0)
