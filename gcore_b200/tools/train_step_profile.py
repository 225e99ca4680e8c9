"""Where does a training micro-batch spend its time?  Builds one model shard, runs forward / backward / optimizer on a
synthetic packed micro-batch and prints (a) CUDA-event timings per phase and (b) the torch-profiler kernel table.

``python -m gcore_b200.tools.train_step_profile --model qwen2.5-7b --layers 8 --tokens 8192 --seqlen 1280``
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--seqlen", type=int, default=1280)
    ap.add_argument("--recompute", default="full")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--profile", action="store_true")
    args = ap.parse_args()
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import get_preset
    from gcore_b200.ops import _lib
    torch.cuda.set_device(0)
    mcfg = get_preset(args.model, num_layers=args.layers)
    eng = TrainingEngine(PolicyConfig(recompute=args.recompute, without_ref=True), OptimizerConfig(),
                         TrainingConfig(), model_cfg=mcfg)
    eng.setup_model_and_get_optimizer(seed=1)
    nseq = max(args.tokens // args.seqlen, 1)
    g = torch.Generator().manual_seed(0)
    samples = [{"tokens": torch.randint(100, 150000, (args.seqlen,), generator=g), "prompt_length": 256}
               for _ in range(nseq)]
    from gcore_b200.core.packing import response_mask
    for s in samples:
        s["mask"] = response_mask(256, args.seqlen)
    mb = eng._pack(samples, list(range(nseq)))

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def one(record=None):
        eng.ddp.zero_grad_buffer()
        t0 = ev()
        hidden, _ = eng._hidden(eng.model, mb)
        t1 = ev()
        lp, _ = eng._logprob_entropy(eng.model, hidden, mb.targets, False)
        loss = -(lp * mb.loss_mask).sum() / mb.loss_mask.sum()
        t2 = ev()
        loss.backward()
        t3 = ev()
        eng.ddp.finish_grad_sync()
        eng.optimizer.step(1e-6)
        t4 = ev()
        torch.cuda.synchronize()
        if record is not None:
            record.append(dict(fwd_layers_ms=t0.elapsed_time(t1), head_fwd_ms=t1.elapsed_time(t2),
                               bwd_ms=t2.elapsed_time(t3), opt_ms=t3.elapsed_time(t4)))

    eng.model.train()
    for _ in range(2):
        one()
    rec = []
    for _ in range(args.iters):
        one(rec)
    mean = {k: round(sum(r[k] for r in rec) / len(rec), 2) for k in rec[0]}
    L, T = args.layers, mb.tokens.numel()
    per_layer = mcfg.num_parameters(include_embedding=False) / mcfg.num_layers * 2 * T
    head = 2 * T * mcfg.hidden_size * mcfg.vocab_size
    mean["fwd_layers_tflops"] = round(per_layer * L / mean["fwd_layers_ms"] / 1e9, 1)
    mean["head_fwd_tflops"] = round(head / mean["head_fwd_ms"] / 1e9, 1)
    passes = 3 if args.recompute == "full" else 2
    mean["bwd_tflops"] = round((per_layer * L * passes + head * 3) / mean["bwd_ms"] / 1e9, 1)
    print(json.dumps(mean))
    if args.profile:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            one()
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=25, max_name_column_width=60))
    _lib.check_device_errors()


if __name__ == "__main__":
    main()
