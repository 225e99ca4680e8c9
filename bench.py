"""Headline benchmark: synchronous GRPO step on a Qwen2.5-7B-shaped dense decoder, bf16, random-init weights,
synthetic prompts and rule reward (the benchmark recipe's config 2), colocated trainer + rollout engine.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W               (N > 1)

Weak scaling: 8 prompts x 8 samples per GPU (64 x 8 at N = 8), prompts of 256 tokens, responses up to 1024 tokens,
trainer TP = min(2, N), DP = N / TP, rollout engine with the same TP sharing the trainer's parameter storage.
The metric is whole-job (prompt + response) tokens pushed through one GRPO step per second of step time:
rollout, reward, previous- and reference-policy log-probs, advantages, policy update (with optimizer step) and the
weight hand-over to the rollout engine, all inside the timed region.

Prints ONE JSON line on rank 0.  ``--impl reference`` reports whether the unmodified reference can run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def reference_arm(args):
    ref = os.path.join(ROOT, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "gpatch_v4")):
        why = "baseline/_ref is empty: the offline install of the reference has not been run on this box"
    else:
        sys.path.insert(0, ref)
        try:
            import importlib
            importlib.import_module("gpatch_v4.entry.train_lm_grpo")
        except Exception as e:  # noqa: BLE001
            why = (f"reference installs (--no-deps) but its GRPO entry point cannot import: {type(e).__name__}: {e}; "
                   "hydra, omegaconf, ray, megatron.core, mbridge, transformer_engine and sglang are not in the "
                   "image and cannot be fetched offline")
    if why is None:
        why = "reference imported, but its launch needs a Ray cluster and Megatron-LM checkouts that are absent here"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")}))
    return 0


class ClockSampler:
    """Samples the SM clock and the throttle reasons while the timed region runs: one NVML query per second from a
    thread of this process (three calls per sample).  A polling ``nvidia-smi -lms 200`` per rank, the obvious way,
    slowed the timed steps by 5-10 % against the warm-up steps (driver contention with the launch path), so it is
    only the fallback when the NVML bindings are missing."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    REASONS = (("hw_slowdown", "nvmlClocksThrottleReasonHwSlowdown", 0x8),
               ("hw_thermal_slowdown", "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
               ("sw_thermal_slowdown", "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
               ("sw_power_cap", "nvmlClocksThrottleReasonSwPowerCap", 0x4))

    def __init__(self, gpu_index: int, period_s: float = 1.0):
        self.idx, self.period = gpu_index, period_s
        self.rows = []          # nvidia-smi fallback: csv rows
        self.samples = []       # NVML: (sm_mhz, max_mhz, reasons bitmask)
        self.proc = self.thread = self.nvml = self.handle = None
        self._stop = threading.Event()
        self.t_mark = 0.0       # samples older than this (taken while the sampler was starting up) are dropped

    def mark(self):
        """Start of the timed region: only samples from here on are reported."""
        self.t_mark = time.time()

    def _open_nvml(self):
        import pynvml
        import torch
        pynvml.nvmlInit()
        h = None
        try:   # the CUDA device of this rank by UUID (CUDA_VISIBLE_DEVICES may renumber the devices)
            uuid = str(torch.cuda.get_device_properties(self.idx).uuid)
            h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:  # noqa: BLE001
            h = pynvml.nvmlDeviceGetHandleByIndex(self.idx)
        self.nvml, self.handle = pynvml, h

    def _poll(self):
        n = self.nvml
        get_reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons")
        mx = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
        while not self._stop.is_set():
            try:
                self.samples.append((n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM), mx,
                                     int(get_reasons(self.handle)), time.time()))
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.period)

    def start(self):
        try:
            self._open_nvml()
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001 - no NVML bindings: fall back to the command-line tool, at a slow rate
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "1000", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")] + [time.time()])

    def stop(self):
        if self.nvml is not None:
            self._stop.set()
            self.thread.join(timeout=5)
            self.samples = [x for x in self.samples if x[3] >= self.t_mark]
            sm = [s[0] for s in self.samples]
            reasons = set()
            for _, _, bits, _ in self.samples:
                for name, const, default in self.REASONS:
                    if bits & int(getattr(self.nvml, const, default)):
                        reasons.add(name)
            return {"sm_mhz": statistics.median(sm) if sm else None,
                    "sm_max_mhz": float(self.samples[0][1]) if self.samples else None, "reasons": sorted(reasons),
                    "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if r[-1] < self.t_mark:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


# The benchmark recipes: GRPO on the 7B dense model (the headline), GRPO on the 30B-A3B MoE with expert parallelism,
# long-context SFT with context x tensor parallelism, block-fp8 GRPO with LoRA on the 12-layer DeepSeek-V3 shape.
CONFIGS = {
    "grpo7b": dict(kind="grpo", model="qwen2.5-7b", prompts_per_gpu=8, samples=8, prompt_len=256, max_response=1024),
    "moe30b": dict(kind="grpo", model="qwen3-30b-a3b", prompts_per_gpu=4, samples=16, prompt_len=256, max_response=2048,
                   mb_tokens=8192, recompute="full"),
    "longctx": dict(kind="sft", model="llama3-8b-swa", seq_len=65536, sequences=8, recompute="full"),
    "dsv3fp8": dict(kind="grpo", model="deepseek-v3-12l", prompts_per_gpu=4, samples=8, prompt_len=512,
                    max_response=1024, mb_tokens=8192, recompute="full"),
}


def parallelism(config: str, world: int):
    """(tp, cp, ep) of a recipe at ``world`` GPUs (the named layouts at 8, the closest smaller ones below)."""
    if config == "grpo7b":
        return (1 if world == 1 else 2), 1, 1
    if config in ("moe30b", "dsv3fp8"):
        return 1, 1, world
    tp = 2 if world >= 2 else 1
    return tp, max(1, min(4, world // tp)), 1


def build_config(args, world):
    from gcore_b200.configs.base import from_dict
    from gcore_b200.configs.config import RlConfig
    tp, cp, ep = parallelism(args.config, world)
    dp = world // (tp * cp)
    prompts_per_dp = args.prompts_per_gpu * tp
    n = args.samples
    dist_cfg = {"tensor_model_parallel_size": tp, "sequence_parallel": tp > 1, "context_parallel_size": cp,
                "expert_model_parallel_size": ep}
    policy = {"model_arch": args.model, "recompute": args.recompute, "recompute_num_layers": args.recompute_layers,
              "offload_ref_model": bool(args.offload_ref),
              "share_rollout_weights": True, "dist_config": dist_cfg, "dynamic_mbs_target_seqlen": args.mb_tokens}
    ppo = {"ppo_ratio_eps": 0.2, "grpo_kl_loss_beta": 0.001, "advantage_type": "grpo", "loss_func": "grpo"}
    opt = {"lr": 1e-6, "lr_decay_style": "constant", "weight_decay": 0.01, "max_grad_norm": 1.0}
    if args.config == "dsv3fp8":
        policy.update(fp8=True, lora={"rank": 64, "alpha": 128, "type": "lora",
                                      "target_modules": ["linear_q_down_proj", "linear_q_up_proj", "linear_kv_down_proj",
                                                         "linear_kv_up_proj", "linear_proj"]})
        ppo["grpo_kl_loss_beta"] = 0.0
        opt.update(lr=2e-5, weight_decay=0.0)
    if args.config == "longctx":
        cfg = from_dict(RlConfig, {
            "training": {"train_gbs": args.sequences, "train_mbs": 1, "seq_length": args.seq_len, "seed": 1234,
                         "total_ppo_step": 1000, "per_token_loss": True},
            "policy": policy, "optimizer": {"lr": 1e-5, "lr_decay_style": "constant", "weight_decay": 0.1,
                                            "max_grad_norm": 1.0}})
        return cfg, tp, dp, 0
    cfg = from_dict(RlConfig, {
        "training": {"rollout_gbs": prompts_per_dp * dp, "sampling_repeat_n": n, "train_gbs": prompts_per_dp * dp * n,
                     "train_mbs": 1, "seed": 1234, "total_ppo_step": 1000},
        "policy": policy, "optimizer": opt,
        "sampler": {"infer_engine_configs": [{"generate_max_tokens": args.max_response, "temperature": 1.0,
                                               "max_model_len": args.prompt_len + args.max_response,
                                               "kv_block_size": 16, "seed": 42,
                                               "dist_config": {"tensor_model_parallel_size": tp}}]},
        "data": {"max_prompt_length": args.prompt_len},
        "ppo": ppo,
    })
    return cfg, tp, dp, prompts_per_dp


def long_context_batch(step: int, dp_rank: int, sequences: int, seq_len: int):
    """``sequences`` packed streams of ``seq_len`` tokens, each a run of documents whose lengths are
    lognormal(mu=7, sigma=1.2) clipped to [64, 32768]; token ids uniform in [100, 128000); loss on every token.
    Returned as one sample per document (the engine packs them back into ``seq_len``-token micro-batches), in pinned
    host memory."""
    import torch
    g = torch.Generator().manual_seed(7919 * step + dp_rank)
    samples = []
    for _ in range(sequences):
        left = seq_len
        while left > 0:
            n = int(torch.empty(1).log_normal_(7.0, 1.2, generator=g).clamp_(64, 32768).item())
            n = min(n, left)
            if left - n < 64:
                n = left
            toks = torch.randint(100, 128000, (n,), generator=g, dtype=torch.int64).pin_memory()
            m = torch.ones(n, dtype=torch.float32)
            m[-1] = 0.0
            samples.append({"tokens": toks, "loss_mask": m, "prompt_length": 0})
            left -= n
    return samples


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "nccl_eager"])
    ap.add_argument("--config", default="grpo7b", choices=sorted(CONFIGS),
                    help="benchmark recipe; the headline (and the default) is grpo7b")
    ap.add_argument("--model", default=None)
    ap.add_argument("--layers", type=int, default=None, help="debug only: truncating the model invalidates the number")
    ap.add_argument("--prompts-per-gpu", type=int, default=None)
    ap.add_argument("--samples", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--max-response", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=None, help="longctx: tokens per packed sequence")
    ap.add_argument("--sequences", type=int, default=None, help="longctx: sequences per global batch")
    ap.add_argument("--mb-tokens", type=int, default=None,
                    help="token budget of a packed micro-batch; default 8192 on one GPU (activations share the GPU with "
                    "the optimizer state of the whole model), 16384 when tensor parallelism halves the state")
    ap.add_argument("--recompute", default=None, help="full | none; default: full on 1 GPU (optimizer state of the "
                    "whole 7B model shares the GPU with the activations), none when tensor parallelism halves it")
    ap.add_argument("--recompute-layers", type=int, default=None,
                    help="with --recompute full: recompute only the first N layers")
    ap.add_argument("--offload-ref", type=int, default=None,
                    help="1: the frozen reference model lives in pinned host memory outside its forward pass (its "
                    "upload runs on a side stream under the old-policy pass); default: on at 1 GPU, where the whole "
                    "model's optimizer state shares the GPU with the activations")
    args = ap.parse_args()
    for k, v in CONFIGS[args.config].items():
        if k != "kind" and getattr(args, k, None) is None:
            setattr(args, k, v)
    args.kind = CONFIGS[args.config]["kind"]
    if args.kind == "sft":
        args.mb_tokens = args.mb_tokens or args.seq_len
    if args.mb_tokens is None:
        args.mb_tokens = 8192 if args.gpus == 1 else 16384
    if args.recompute is None:
        args.recompute = "full" if args.gpus == 1 else "none"
        if args.gpus == 1 and args.recompute_layers is None and args.layers is None and args.model == "qwen2.5-7b":
            # 152 GB of weights, reference model, fp32 gradients and AdamW state leave room for the activations of
            # 16 of the 28 layers at 8192 tokens per micro-batch (peak 164 GB of 180); the other 12 are recomputed
            args.recompute_layers = 12
    if args.offload_ref is None:
        args.offload_ref = 0
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    from gcore_b200.core import parallel_state as ps
    from gcore_b200.models.config import get_preset
    from gcore_b200.ops import _lib
    from gcore_b200.trainer.grpo_trainer import GrpoTrainer, synthetic_reward

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    torch.cuda.set_device(local)
    if world > 1:
        ps.init_distributed("nccl")
    cfg, tp, dp, prompts_per_dp = build_config(args, world)
    _, cp, ep = parallelism(args.config, world)
    if world > 1:
        ps.initialize_model_parallel(tp=tp, cp=cp, ep=ep)
    if args.impl == "nccl_eager":
        # library build of the same step: cuBLAS GEMMs, the library's fused attention, PyTorch elementwise ops, NCCL
        # collectives at the call sites of the fused kernels, a CUDA-graph decode loop over library ops, and a weight
        # resync that copies every tensor through a staging bucket into a separate rollout copy (freed after rollout)
        cfg.training.training_backend = "nccl_eager"
        cfg.policy.share_rollout_weights = False
        cfg.policy.release_rollout_weights = True
        os.environ["GCORE_B200_FORCE_EAGER"] = "1"
        for k in ("GCORE_FUSED_TP", "GCORE_FUSED_DP", "GCORE_FUSED_EP", "GCORE_FUSED_CP", "GCORE_PEER_ALLREDUCE"):
            os.environ[k] = "0"
    over = {"num_layers": args.layers} if args.layers else {}
    mcfg = get_preset(args.model, **over)
    total_steps = args.warmup + args.steps
    from gcore_b200.utils import io_counters
    if args.kind == "sft":
        from gcore_b200.engine import get_training_engine
        cfg.policy.without_ref = True
        engine = get_training_engine(cfg.policy, cfg.optimizer, cfg.training, None, model_cfg=mcfg, total_steps=1000)
        engine.setup_model_and_get_optimizer()
        dp_rank = ps.get_data_parallel_rank()
        per_dp = max(args.sequences // dp, 1)
        # every step's documents are generated ahead of the timed region, in pinned host memory
        batches = [long_context_batch(i, dp_rank, per_dp, args.seq_len) for i in range(total_steps)]
        trainer = None

        def run_step(i):
            t0 = time.perf_counter()
            m = engine.finetune_step(batches[i])          # uploads the tokens, returns the loss to the host
            dt = time.perf_counter() - t0
            m.update({"time_perf/step": dt, "time_perf/train_step": dt,
                      "rollout-metrics/total_tokens": float(per_dp * dp * args.seq_len)})
            return m
    else:
        trainer = GrpoTrainer(cfg, model_cfg=mcfg, reward_fn=synthetic_reward).setup()
        dp_rank = ps.get_data_parallel_rank()
        # synthetic prompts live in pinned host memory; every step copies its prompts to the device inside the timed
        # region
        g = torch.Generator().manual_seed(1000 + dp_rank)
        # token ids uniform in [100, 150000) as the recipe says, capped by the model's vocabulary (129 280 for the
        # DeepSeek-V3 shape: ids beyond it would index outside the embedding table)
        hi = min(150000, mcfg.vocab_size)
        host_prompts = torch.randint(100, hi, (total_steps, prompts_per_dp, args.prompt_len), generator=g,
                                     dtype=torch.int64).pin_memory()

        def run_step(i):
            # the engine uploads the prompt tokens (pinned host -> device) when it prefills them
            return trainer.step(host_prompts[i])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    for i in range(args.warmup):
        if i == args.warmup - 1:
            # the sampler comes up during the last untimed step, so that whatever its start costs (NVML attach, or the
            # fork of the fallback tool) is not inside the timed region; only samples taken after `mark()` are reported
            sampler.start()
        m = run_step(i)
        if rank == 0:
            print(f"[warmup {i}] step {m['time_perf/step']:.2f}s rollout {m.get('time_perf/rollout', 0.0):.2f}s "
                  f"logps {m.get('time_perf/compute_logps', 0.0):.2f}s train {m['time_perf/train_step']:.2f}s "
                  f"tokens {m['rollout-metrics/total_tokens']:.0f}", file=sys.stderr, flush=True)
    _lib.check_device_errors()
    # the model, engine and optimizer objects built so far are permanent: keep the cyclic collector from walking them
    # every time the per-token Python objects of a rollout trigger a full collection
    import gc
    gc.collect()
    gc.freeze()
    io_counters.reset()
    launches0 = trainer_launches(trainer)
    if args.warmup == 0:
        sampler.start()
    barrier()
    sampler.mark()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    tokens = 0.0
    phase = {}
    for i in range(args.warmup, total_steps):
        m = run_step(i)
        tokens += m["rollout-metrics/total_tokens"]
        for k, v in m.items():
            if k.startswith("time_perf/"):
                phase[k] = phase.get(k, 0.0) + v / args.steps
        if rank == 0 and "time_perf/step" in m:
            print(f"[step {i}] step {m['time_perf/step']:.2f}s rollout {m.get('time_perf/rollout', 0.0):.2f}s "
                  f"logps {m.get('time_perf/compute_logps', 0.0):.2f}s train {m.get('time_perf/train_step', 0.0):.2f}s",
                  file=sys.stderr, flush=True)
    ev1.record()
    barrier()
    wall = time.perf_counter() - t0
    dev_s = ev0.elapsed_time(ev1) / 1e3
    clocks = sampler.stop()
    _lib.check_device_errors()
    t = torch.tensor([dev_s, wall], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_s, wall = float(t[0]), float(t[1])
    launches = trainer_launches(trainer) - launches0
    h2d, d2h = io_counters.get()
    if rank == 0:
        value = tokens / dev_s
        out = {
            "metric": ("grpo_rollout_plus_train_tokens_per_s" if args.kind == "grpo" else "sft_train_tokens_per_s"),
            "value": round(value, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_s / args.steps * 1e3, 1),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": vs_baseline(args, world, value),
            "dtype": "bf16 (frozen base projections block-scaled e4m3)" if args.config == "dsv3fp8" else "bf16",
            "data": "synthetic", "recipe": args.config,
            "impl": args.impl,
            "config": bench_config_record(args, cfg, tp, cp, ep, dp),
            "clocks": clocks,
            "e2e": {"value": round(tokens / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d / args.steps),
                    "d2h_bytes_per_step": int(d2h / args.steps)},
            "gpu_launches": int(launches),
            "phases_s": {k.split("/")[1]: round(v, 3) for k, v in phase.items()},
            "resync_ms": round(phase.get("time_perf/update_weights", 0.0) * 1e3, 3),
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1),
            "peak_reserved_gb": round(torch.cuda.max_memory_reserved() / 2**30, 1),
            "alloc_retries": int(torch.cuda.memory_stats().get("num_alloc_retries", 0)),
            **({"reward_mean": round(m["rollout-rewards/mean"], 4)} if args.kind == "grpo"
               else {"lm_loss": round(float(m["lm_loss"]), 4)}),
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def bench_config_record(args, cfg, tp, cp, ep, dp):
    par = f"tp{tp}" + (f"cp{cp}" if cp > 1 else "") + (f"ep{ep}" if ep > 1 else "") + f"dp{dp}"
    rec = {"model": args.model + (f"-{args.layers}layers-DEBUG" if args.layers else ""), "parallelism": par,
           "weights": "random-init", "recompute": args.recompute, "recompute_layers": args.recompute_layers,
           "micro_batch_tokens": args.mb_tokens, "l2": "inputs (weights of every pass) are larger than L2",
           "reference_model": "pinned host memory outside its forward pass" if args.offload_ref else "resident"}
    if args.kind == "sft":
        rec.update(global_batch=int(args.sequences), seq_len=int(args.seq_len),
                   documents="lognormal(7, 1.2) clipped to [64, 32768], packed")
        return rec
    rec.update(global_batch=int(cfg.training.rollout_gbs * args.samples), seq_len=args.prompt_len + args.max_response,
               prompts=int(cfg.training.rollout_gbs), samples_per_prompt=args.samples,
               resync=("zero-copy shared parameter storage (trainer and rollout engine, same layout)"
                       if cfg.policy.share_rollout_weights else
                       "bucketed copy into a separate rollout copy (rebuilt every step, freed after rollout)"))
    return rec


def vs_baseline(args, world, value):
    """value / the library (``nccl_eager``) build's measured value of the same config at the same GPU count, from the
    committed ``baseline/measured_baselines.json``; None when that row has not been measured.  (The reference
    publishes no number for this metric, and cannot run here: the library build is its stand-in.)"""
    if args.impl != "native" or args.layers or args.config != "grpo7b":
        return None
    try:
        rows = json.load(open(os.path.join(ROOT, "baseline", "measured_baselines.json")))["nccl_eager"]
        base = rows[args.model][str(world)]["value"]
        return round(value / base, 3) if base else None
    except Exception:  # noqa: BLE001
        return None


def trainer_launches(trainer) -> int:
    from gcore_b200.ops import attention, fused, gemm, optim, rl, vocab
    from gcore_b200.ops import router
    from gcore_b200.parallel import ep_fused, symm
    eager = sum(sum(m.LAUNCHES.values()) for m in (attention, fused, gemm, optim, rl, vocab, router, ep_fused, symm))
    if trainer is None:
        return eager
    eng = trainer.engine
    return eager + eng.stats["graph_replays"] * getattr(eng, "graph_launches", 0)


if __name__ == "__main__":
    sys.exit(main())
