"""Black-box rollout baseline: the same rollout batch as ``bench.py`` served by vLLM (the engine the reference
wraps: gpatch_v4/generation_backend/vllm_engine.py:40, infer_engine.py:393-768), random-init weights of the same
architecture, prompts given as token ids, every response forced to ``max_tokens`` (random-init models do not emit EOS,
and the native engine generates all of them too), the log-prob of each sampled token returned as the reference asks
its engines for ``rollout_log_probs``.

    python baseline/vllm_rollout.py --model qwen2.5-7b --prompts 8 --samples 8 --prompt-len 256 --max-response 1024 \
        --tp 1 --iters 3 --out baseline/vllm_rollout_n1.json

Prints (and writes) one JSON line: wall seconds per rollout (best and median of ``--iters`` after one warm-up
iteration), decode tokens/s, and prompt + response tokens/s.  Only timings are taken from vLLM; nothing of it is
used by the framework.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def hf_config_dict(name: str) -> dict:
    from gcore_b200.models.config import get_preset
    c = get_preset(name)
    if getattr(c, "num_experts", 0):
        return {
            "architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe", "hidden_size": c.hidden_size,
            "intermediate_size": c.ffn_hidden_size, "moe_intermediate_size": c.moe_ffn_hidden_size,
            "num_hidden_layers": c.num_layers, "num_attention_heads": c.num_attention_heads,
            "num_key_value_heads": c.num_kv_heads, "head_dim": c.head_dim, "num_experts": c.num_experts,
            "num_experts_per_tok": c.moe_top_k, "norm_topk_prob": True, "decoder_sparse_step": 1, "mlp_only_layers": [],
            "vocab_size": c.vocab_size, "rope_theta": c.rope_theta, "rms_norm_eps": c.rms_norm_eps,
            "max_position_embeddings": 32768, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
            "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
        }
    return {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": c.hidden_size,
        "intermediate_size": c.ffn_hidden_size, "num_hidden_layers": c.num_layers,
        "num_attention_heads": c.num_attention_heads, "num_key_value_heads": c.num_kv_heads,
        "vocab_size": c.vocab_size, "rope_theta": c.rope_theta, "rms_norm_eps": c.rms_norm_eps,
        "max_position_embeddings": 32768, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
        "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2, "use_sliding_window": False,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--samples", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--max-response", type=int, default=1024)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.7)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    result = {"impl": "vllm", "model": args.model, "prompts": args.prompts, "samples": args.samples,
              "prompt_len": args.prompt_len, "max_response": args.max_response, "tp": args.tp}
    try:
        import torch
        import vllm
        from vllm import LLM, SamplingParams
        result["vllm"] = vllm.__version__
        d = tempfile.mkdtemp(prefix="vllm_cfg_")
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(hf_config_dict(args.model), f)
        llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16",
                  tensor_parallel_size=args.tp, max_model_len=args.prompt_len + args.max_response,
                  gpu_memory_utilization=args.gpu_memory_utilization, max_num_seqs=args.prompts * args.samples,
                  enable_prefix_caching=True, seed=0)
        sp = SamplingParams(n=args.samples, temperature=1.0, max_tokens=args.max_response, ignore_eos=True,
                            logprobs=0, detokenize=False)
        g = torch.Generator().manual_seed(1000)
        times = []
        for it in range(args.iters + 1):
            toks = torch.randint(100, 150000, (args.prompts, args.prompt_len), generator=g).tolist()
            prompts = [{"prompt_token_ids": t} for t in toks]
            t0 = time.perf_counter()
            outs = llm.generate(prompts, sp, use_tqdm=False)
            dt = time.perf_counter() - t0
            n_out = sum(len(o.token_ids) for r in outs for o in r.outputs)
            if it > 0:
                times.append(dt)
            print(f"[vllm iter {it}] {dt:.3f}s generated {n_out}", file=sys.stderr, flush=True)
        nseq = args.prompts * args.samples
        best, med = min(times), statistics.median(times)
        result.update({"rollout_s_best": round(best, 3), "rollout_s_median": round(med, 3),
                       "generated_tokens": n_out,
                       "decode_tokens_per_s": round(n_out / med, 1),
                       "prompt_plus_response_tokens_per_s": round(nseq * (args.prompt_len + args.max_response) / med, 1)})
    except Exception as e:  # noqa: BLE001 - the baseline is optional: report why it did not run
        result["unavailable"] = f"{type(e).__name__}: {str(e)[:300]}"
    line = json.dumps(result)
    print(line, flush=True)
    if args.out:
        with open(args.out, "w") as f:
            f.write(line + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
