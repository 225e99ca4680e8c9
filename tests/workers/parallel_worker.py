"""gloo worker for the parallelism parity tests: mode = tp | tp_value | tp_mla | tp_mla_lora | tp_lora | tp_lora_moe | tp_mtp | tp_moe | tp2ep2 | ep2dp4 | ep | ep_rollout | ep_grpo | cp | cp_mla | cp_mtp | dpo_cp | dpo_dp | dpo_tp | rm_cp | pp_value | pp | pp_moe | tp_nosp | vpp | fsdp |
ep_dynmbs | aux_dp | tp_topk | nodistopt | dyncp | dp_grpo_balance | pg_offload."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig  # noqa: E402
from gcore_b200.core import parallel_state as ps  # noqa: E402
from gcore_b200.engine.train_engine import TrainingEngine  # noqa: E402
from gcore_b200.models.config import ModelConfig, get_preset  # noqa: E402


NOSP_CFG = get_preset("tiny_llama", dtype="float32", qk_layernorm=True, mtp_num_layers=1,
                      mtp_loss_scaling_factor=0.3)


def samples(n, seed, L=48, vocab=1024):
    g = torch.Generator().manual_seed(seed)
    out = []
    for i in range(n):
        ln = int(torch.randint(L // 2, L + 1, (1,), generator=g))
        t = torch.randint(3, vocab, (ln,), generator=g)
        m = torch.zeros(ln)
        m[ln // 3:ln - 1] = 1
        out.append({"tokens": t, "loss_mask": m})
    return out


MOE_CFG = ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=128, num_attention_heads=4, num_kv_heads=2,
                      ffn_hidden_size=256, vocab_size=512, num_experts=8, moe_top_k=2, moe_ffn_hidden_size=64,
                      moe_aux_loss_coef=1e-2, dtype="float32", qk_layernorm=True)


MLA_CFG = ModelConfig(arch="deepseek_v3", num_layers=2, hidden_size=128, num_attention_heads=4, num_kv_heads=4,
                      ffn_hidden_size=256, vocab_size=512, use_mla=True, q_lora_rank=64, kv_lora_rank=32,
                      qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, head_dim=24, dtype="float32")


def engine(mcfg, tp, sp=True, lr=1e-3, vpp=None):
    pc = PolicyConfig(recompute="none", without_ref=True)
    pc.dist_config.tensor_model_parallel_size = tp
    pc.dist_config.virtual_pipeline_model_parallel_size = vpp
    pc.dist_config.sequence_parallel = sp and tp > 1
    oc = OptimizerConfig(lr=lr, lr_decay_style="constant", weight_decay=0.0, max_grad_norm=1.0)
    tc = TrainingConfig(train_mbs=2, train_gbs=8)
    e = TrainingEngine(pc, oc, tc, model_cfg=mcfg)
    e.setup_model_and_get_optimizer(seed=11)
    return e


def value_engine(tp):
    from gcore_b200.configs.config import PpoConfig
    pc = PolicyConfig(recompute="none", without_ref=True)
    pc.dist_config.tensor_model_parallel_size = tp
    pc.dist_config.sequence_parallel = tp > 1
    oc = OptimizerConfig(lr=1e-3, lr_decay_style="constant", weight_decay=0.0, max_grad_norm=1.0)
    e = TrainingEngine(pc, oc, TrainingConfig(train_mbs=2, train_gbs=8), ppo_cfg=PpoConfig(),
                       model_cfg=get_preset("tiny_llama", dtype="float32", qkv_bias=True), value_head=True)
    e.setup_model_and_get_optimizer(seed=11)
    return e


def value_samples():
    smp = samples(8, 60)
    g = torch.Generator().manual_seed(9)
    for s in smp:
        n = s["tokens"].numel()
        s["mask"] = s["loss_mask"]
        s["returns"], s["values"] = torch.randn(n, generator=g), torch.randn(n, generator=g)
    return smp


def value_run():
    e = value_engine(1)
    out = e.rl_train_value(value_samples())
    smp = value_samples()
    for s in smp:
        s.pop("values")
    e.compute_values(smp)
    return {"loss": out["value/loss"], "grad_norm": out["value/grad_norm"],
            "values_sum": float(sum(s["values"].double().sum() for s in smp)), "value_3_5": float(smp[3]["values"][5])}


def preference_run():
    """Two reward-model steps and one contrastive step per pooling mode: (loss, gradient norm) of each."""
    from gcore_b200.trainer.preference_trainers import embedding_step, rm_step
    e = value_engine(1)
    out = []
    for s in range(2):
        o = rm_step(e, samples(4, 200 + s), samples(4, 300 + s))
        out.append([o["rm/loss"], float(e.optimizer.last_grad_norm)])
    e2 = engine(get_preset("tiny_llama", dtype="float32", qkv_bias=True), 1)
    for pooling in ("last", "mean"):
        o = embedding_step(e2, samples(4, 400), samples(4, 500), pooling=pooling)
        out.append([o["embedding/loss"], o["grad_norm"]])
    return {"runs": out}


def lora_engine(mcfg, tp, targets=None):
    """Engine with rank-8 adapters whose two halves are both non-zero and drawn from the full (unsharded) tensors, so
    that a TP = 2 run and a single-process run hold the same effective adapters."""
    import zlib
    pc = PolicyConfig(recompute="none", without_ref=True)
    pc.dist_config.tensor_model_parallel_size = tp
    pc.dist_config.sequence_parallel = tp > 1
    pc.lora.rank, pc.lora.alpha = 8, 16
    if targets:
        pc.lora.target_modules = list(targets)
    oc = OptimizerConfig(lr=1e-3, lr_decay_style="constant", weight_decay=0.0, max_grad_norm=1.0)
    e = TrainingEngine(pc, oc, TrainingConfig(train_mbs=2, train_gbs=8), model_cfg=mcfg)
    e.setup_model_and_get_optimizer(seed=11)
    r = ps.get_tensor_model_parallel_rank() if tp > 1 else 0
    with torch.no_grad():
        for n, p in sorted(e.model.named_parameters()):
            if not getattr(p, "is_lora", False):
                continue
            mode = getattr(p, "tp_mode", "none")
            shape = list(p.shape)
            if tp > 1 and mode == "column":
                shape[0] *= tp
            if tp > 1 and mode == "row":
                shape[-1] *= tp
            g = torch.Generator().manual_seed(zlib.crc32(n.encode()) & 0x7FFFFFFF)
            full = torch.randn(*shape, generator=g) * 0.05
            if tp > 1 and mode == "column":
                full = full.chunk(tp, 0)[r]
            if tp > 1 and mode == "row":
                full = full.chunk(tp, -1)[r]
            p.copy_(full)
    return e


def main():
    mode, out = sys.argv[1], sys.argv[2]
    ps.init_distributed(os.environ.get("GCORE_TEST_BACKEND", "gloo"))  # nccl: the same parity check on GPUs
    world, rank = dist.get_world_size(), dist.get_rank()
    res = {}
    if mode == "tp":
        ps.initialize_model_parallel(tp=2)
        mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
        e = engine(mcfg, 2)
        losses = []
        for s in range(4):
            losses.append(e.finetune_step(samples(8, 50 + s))["lm_loss"])  # TP ranks see the same data
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm)}
        if len(sys.argv) > 3:
            from gcore_b200.checkpoint.hf import save_hf
            from gcore_b200.checkpoint.torch_dist import save_checkpoint
            save_checkpoint(e, os.path.join(sys.argv[3], "ckpt"), 4)
            save_hf(e, os.path.join(sys.argv[3], "hf"))
    elif mode == "tp_value":
        # critic under tensor parallelism: the scalar head is replicated, every rank back-propagates the whole loss
        from gcore_b200.configs.config import PpoConfig
        ps.initialize_model_parallel(tp=2)
        e = value_engine(2)
        res = e.rl_train_value(value_samples())
    elif mode in ("tp_mla", "tp_mla_lora"):
        # latent attention under tensor parallelism: replicated down-projections in front of sharded heads
        ps.initialize_model_parallel(tp=2)
        if mode == "tp_mla":
            e = engine(MLA_CFG, 2)
        else:
            e = lora_engine(MLA_CFG, 2, ["linear_q_down_proj", "linear_q_up_proj", "linear_kv_down_proj",
                                         "linear_kv_up_proj", "linear_proj"])
        losses = [e.finetune_step(samples(8, 50 + s, vocab=512))["lm_loss"] for s in range(3)]
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm)}
    elif mode in ("tp_lora", "tp_lora_moe"):
        # adapters under tensor + sequence parallelism: the replicated half of an adapter on a sharded projection gets
        # partial gradients per rank, router / shared-expert adapters see one token shard per rank
        import dataclasses
        ps.initialize_model_parallel(tp=2)
        if mode == "tp_lora":
            e = lora_engine(get_preset("tiny_llama", dtype="float32", qkv_bias=True), 2)
            vocab = 1024
        else:
            e = lora_engine(dataclasses.replace(MOE_CFG, moe_aux_loss_coef=0.0), 2,
                            ["linear_qkv", "linear_proj", "linear_fc1", "linear_fc2", "router"])
            vocab = 512
        losses = [e.finetune_step(samples(8, 50 + s, vocab=vocab))["lm_loss"] for s in range(3)]
        from gcore_b200.models.lora import verify_lora_weight_consistency
        same = verify_lora_weight_consistency({k: v for k, v in e.adapters.items() if hasattr(v, "lora_B")
                                               and isinstance(v.lora_B, torch.nn.ParameterList)},
                                              ps.get_tensor_model_parallel_group())
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm), "replicated_halves_equal": bool(same)}
    elif mode == "tp_mtp":
        # multi-token-prediction blocks under tensor + sequence parallelism: their branch re-shards the gathered trunk
        # output, whose backward must hand back each rank's own share only
        import dataclasses
        ps.initialize_model_parallel(tp=2)
        mcfg = dataclasses.replace(get_preset("tiny_llama", dtype="float32", qkv_bias=True), mtp_num_layers=2,
                                   mtp_loss_scaling_factor=0.3)
        e = engine(mcfg, 2)
        outs = [e.finetune_step(samples(8, 50 + s)) for s in range(3)]
        res = {"losses": [o["lm_loss"] for o in outs], "mtp": [o["mtp_loss"] for o in outs],
               "grad_norm": float(e.optimizer.last_grad_norm)}
    elif mode == "tp_moe":
        # tensor parallel 2 with an MoE model whose experts are not split (expert parallel 1): every TP rank routes the
        # tokens of its own sequence-parallel shard through whole experts, so the expert gradients of the two ranks
        # have to be summed - the TP ranks are data-parallel replicas as far as the experts are concerned
        ps.initialize_model_parallel(tp=2)
        e = engine(MOE_CFG, 2)
        losses = [e.finetune_step(samples(8, 70 + s, vocab=512))["lm_loss"] for s in range(4)]
        w = e.model.decoder.layers[1].mlp.experts.linear_fc1.weight.detach()
        parts = [torch.empty_like(w) for _ in range(world)]
        dist.all_gather(parts, w.contiguous())
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm),
               "expert_weights_equal": bool(torch.equal(parts[0], parts[1])),
               "fc1_sum": float(w.double().sum())}
    elif mode in ("tp2ep2", "ep2dp4"):
        # four ranks: tensor parallel 2 x data parallel 2 with the experts split 2 ways and replicated 2 ways, or pure
        # data parallel 4 with the experts split 2 ways and replicated 2 ways
        if mode == "tp2ep2":
            ps.initialize_model_parallel(tp=2, ep=2, etp=1)
            e = engine(MOE_CFG, 2)
        else:
            ps.initialize_model_parallel(tp=1, ep=2)
            e = engine(MOE_CFG, 1)
        dpr, dpw = ps.get_data_parallel_rank(), ps.get_data_parallel_world_size()
        losses = [e.finetune_step(samples(8, 70 + s, vocab=512)[dpr::dpw])["lm_loss"] for s in range(2)]
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm),
               "edp": dist.get_world_size(ps.get_expert_data_parallel_group())}
    elif mode == "ep":
        ps.initialize_model_parallel(tp=1, ep=2)
        mcfg = ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=128, num_attention_heads=4, num_kv_heads=2,
                           ffn_hidden_size=256, vocab_size=512, num_experts=8, moe_top_k=2, moe_ffn_hidden_size=64,
                           moe_aux_loss_coef=1e-2, dtype="float32", qk_layernorm=True)
        e = engine(mcfg, 1)
        losses = []
        for s in range(3):
            batch = samples(8, 70 + s, vocab=512)
            losses.append(e.finetune_step(batch[rank::world])["lm_loss"])  # EP ranks are also DP ranks
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm)}
    elif mode == "ep_rollout":
        # two engines whose experts are split over both ranks serve different workloads (3 prompts x 9 tokens against
        # 1 prompt x 3 tokens): the engine that finishes first has to keep its experts in the others' all-to-alls
        from gcore_b200.models.gpt import GPTModel
        from gcore_b200.rollout.engine import InferEngine, RolloutWeights, SamplingParams
        ps.initialize_model_parallel(tp=1, ep=2)
        mcfg = ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=128, num_attention_heads=4, num_kv_heads=2,
                           ffn_hidden_size=256, vocab_size=512, num_experts=8, moe_top_k=2, moe_ffn_hidden_size=64,
                           dtype="float32", qk_layernorm=True)
        torch.manual_seed(0)
        model = GPTModel(mcfg, ep_size=2, recompute="none")
        model.reset_parameters(21)
        model.eval()
        eng = InferEngine(mcfg, RolloutWeights.from_model(model), max_running_requests=2, max_model_len=48,
                          kv_block_size=4, sync_interval=2, use_cuda_graph=False)
        assert eng.ep_group is not None
        g = torch.Generator().manual_seed(100 + rank)
        n_prompts, n_new = (3, 9) if rank == 0 else (1, 3)
        prompts = [torch.randint(3, 512, (5 + 2 * i,), generator=g).tolist() for i in range(n_prompts)]
        reqs = eng.generate(prompts, SamplingParams(max_new_tokens=n_new, greedy=True))
        json.dump({"prompts": prompts, "tokens": [r.out_tokens for r in reqs],
                   "logprobs": [r.out_logprobs for r in reqs]}, open(f"{out}.{rank}", "w"))
    elif mode == "ep_grpo":
        # whole GRPO steps with experts split over both ranks, in the trainer and in the colocated rollout engine
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        from test_grpo_cpu import make_cfg, reward_has_small_token
        from gcore_b200.trainer.grpo_trainer import GrpoTrainer
        ps.initialize_model_parallel(tp=1, ep=2)
        dt = "bfloat16" if torch.cuda.is_available() else "float32"
        mcfg = ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=256, num_attention_heads=2, num_kv_heads=1,
                           head_dim=128, ffn_hidden_size=512, vocab_size=1024, num_experts=8, moe_top_k=2,
                           moe_ffn_hidden_size=128, moe_aux_loss_coef=1e-3, dtype=dt, qk_layernorm=True)
        cfg = make_cfg()
        cfg.policy.dist_config.expert_model_parallel_size = 2
        cfg.training.rollout_gbs, cfg.training.train_gbs = 8, 32   # 4 prompts x 4 samples per rank
        cfg.sampler.infer_engine_configs[0].generate_params = {"stop_token_ids": [7 + rank]}
        torch.manual_seed(0)
        tr = GrpoTrainer(cfg, model_cfg=mcfg, reward_fn=reward_has_small_token).setup()
        assert tr.engine.ep_group is not None and tr.policy.model.ep_size == 2
        g = torch.Generator().manual_seed(5 + rank)
        prompts = [torch.randint(3, 1024, (6 + i,), generator=g).tolist() for i in range(4)]
        ms = [tr.step(prompts) for _ in range(2)]
        smp = tr.last_samples[0]
        P, S = smp["prompt_length"], smp["sequence_length"]
        gap = float((smp["logprobs"][P - 1:S - 1] - smp["rollout_log_probs"][P - 1:S - 1]).abs().max())
        res = {"grad_norm": [m["policy/grad_norm"] for m in ms], "ratio": [m["ppo-metrics/ratio"] for m in ms],
               "logprob_gap": gap, "dtype": dt}
        allres = [None, None]
        dist.all_gather_object(allres, res)
        res = {"ranks": allres}
    elif mode == "cp":
        ps.initialize_model_parallel(tp=1, cp=2)
        mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True, sliding_window=16,
                          sliding_window_pattern=[0, 1], attention_sinks=True)
        e = engine(mcfg, 1)
        losses = []
        for s in range(4):
            losses.append(e.finetune_step(samples(8, 90 + s))["lm_loss"])  # CP ranks see the same data
        lp = e.compute_log_probs(samples(3, 99))
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm),
               "logprobs": [x["logprobs"].tolist() for x in lp]}
    elif mode == "cp_mla":
        # latent attention under context parallelism: the compressed latent crosses the ranks, not the expanded heads
        ps.initialize_model_parallel(tp=1, cp=2)
        e = engine(MLA_CFG, 1)
        losses = [e.finetune_step(samples(8, 170 + s, vocab=512))["lm_loss"] for s in range(3)]
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm)}
    elif mode == "cp_mtp":
        # multi-token prediction on context-parallel shards: the look-ahead of a chunk's last positions is its halo
        ps.initialize_model_parallel(tp=1, cp=2)
        e = engine(NOSP_CFG, 1)
        losses = [e.finetune_step(samples(8, 180 + s))["lm_loss"] for s in range(3)]
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm)}
    elif mode in ("dpo_cp", "dpo_dp", "dpo_tp"):
        # preference pairs: sequence log-probs cross context-parallel ranks; the token-mean SFT term is global
        from gcore_b200.trainer.preference_trainers import dpo_step
        ps.initialize_model_parallel(tp=2 if mode == "dpo_tp" else 1, cp=2 if mode == "dpo_cp" else 1)
        e = engine(get_preset("tiny_llama", dtype="float32", qkv_bias=True), 2 if mode == "dpo_tp" else 1)
        dpr, dpw = ps.get_data_parallel_rank(), ps.get_data_parallel_world_size()
        outs = []
        for s in range(2):
            ch, rj = samples(4, 200 + s), samples(4, 300 + s)
            outs.append(dpo_step(e, ch[dpr::dpw], rj[dpr::dpw], beta=0.5, reference_free=True, sft_coef=0.1))
        res = {"losses": [o["dpo/loss"] for o in outs], "grad_norms": [o["grad_norm"] for o in outs]}
    elif mode == "rm_cp":
        # sequence-end scores and pooled embeddings index the whole stream, which lives on two context-parallel ranks
        from gcore_b200.trainer.preference_trainers import embedding_step, rm_step
        ps.initialize_model_parallel(tp=1, cp=2)
        res = preference_run()
    elif mode == "pp_value":
        # a critic split over two pipeline stages trains and scores through the same schedule as the policy
        ps.initialize_model_parallel(tp=1, pp=2)
        res = value_run()
    elif mode == "tp_nosp":
        # tensor parallelism without the sequence-parallel token shard: per-head q/k gains, multi-token prediction
        import dataclasses
        ps.initialize_model_parallel(tp=2)
        e = engine(NOSP_CFG, 2, sp=False)
        assert not e.model.sequence_parallel
        losses = [e.finetune_step(samples(8, 150 + s))["lm_loss"] for s in range(3)]
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm)}
    elif mode == "pp_moe":
        # MoE layers on both pipeline stages: the first stage back-propagates its own load-balance loss
        import dataclasses
        ps.initialize_model_parallel(tp=1, pp=2)
        e = engine(dataclasses.replace(MOE_CFG, num_layers=4), 1)
        losses = [e.finetune_step(samples(8, 130 + s, vocab=512))["lm_loss"] for s in range(3)]
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm)}
    elif mode in ("pp", "vpp"):
        ps.initialize_model_parallel(tp=1, pp=2)
        mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True, num_layers=4)
        e = engine(mcfg, 1, vpp=2 if mode == "vpp" else None)
        assert len(e.model.decoder.layers) == 2
        if mode == "vpp":  # interleaved: stage 0 holds layers 0 and 2, stage 1 holds 1 and 3
            assert e.model.global_layer_ids == [rank, rank + 2] and len(e.model.chunk_bounds) == 2
        losses, norms = [], []
        for s in range(4):
            losses.append(e.finetune_step(samples(8, 130 + s))["lm_loss"])  # pipeline ranks see the same data
            norms.append(float(e.optimizer.last_grad_norm))
        lp = e.compute_log_probs(samples(3, 199))
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm), "grad_norms": norms,
               "logprobs": [x["logprobs"].tolist() for x in lp]}
        if len(sys.argv) > 3:
            from gcore_b200.checkpoint.torch_dist import load_checkpoint, save_checkpoint
            save_checkpoint(e, os.path.join(sys.argv[3], "ckpt"), 4)
            # a fresh two-stage engine (other seed) resumes from it and takes the same next step
            e2 = engine(mcfg, 1, vpp=2 if mode == "vpp" else None)
            e2.setup_model_and_get_optimizer(seed=77)
            assert load_checkpoint(e2, os.path.join(sys.argv[3], "ckpt")) == 4
            res["next_loss"] = [x.finetune_step(samples(8, 140))["lm_loss"] for x in (e, e2)]
    elif mode == "fsdp":
        from gcore_b200.engine.fsdp2_engine import Fsdp2Engine
        ps.initialize_model_parallel(tp=1)
        mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
        pc = PolicyConfig(recompute="none", without_ref=True)
        oc = OptimizerConfig(lr=1e-3, lr_decay_style="constant", weight_decay=0.0, max_grad_norm=1.0)
        e = Fsdp2Engine(pc, oc, TrainingConfig(train_mbs=2, train_gbs=8), model_cfg=mcfg)
        e.setup_model_and_get_optimizer(seed=11)
        losses = []
        for s in range(4):
            batch = samples(8, 150 + s)
            losses.append(e.finetune_step(batch[rank::world])["lm_loss"])
        local = sum(p.to_local().numel() if hasattr(p, "to_local") else p.numel() for p in e.model.parameters())
        total = sum(p.numel() for p in e.model.parameters())
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm), "local_frac": local / total}
        if len(sys.argv) > 3:
            e.save_checkpoint(sys.argv[3], 4)
            e2 = Fsdp2Engine(pc, oc, TrainingConfig(train_mbs=2, train_gbs=8), model_cfg=mcfg)
            e2.setup_model_and_get_optimizer(seed=99)
            assert e2.load_checkpoint(sys.argv[3]) == 4
            res["next_loss"] = [x.finetune_step(samples(8, 160)[rank::world])["lm_loss"] for x in (e, e2)]
    elif mode == "ep_dynmbs":
        # expert-parallel ranks whose samples pack into different numbers of micro-batches (rank 0: six long samples,
        # rank 1: two short ones) under a token budget: every rank must still run the same number of all-to-alls
        ps.initialize_model_parallel(tp=1, ep=2)
        e = engine(MOE_CFG, 1)
        e.policy_cfg.dynamic_mbs_target_seqlen = 64
        losses, counts = [], []
        for s in range(2):
            batch = samples(8, 170 + s, vocab=512)
            batch.sort(key=lambda x: -len(x["tokens"]))
            mine = batch[:6] if rank == 0 else batch[6:]
            counts.append(len(e._microbatches(mine)))
            losses.append(e.finetune_step(mine)["lm_loss"])
        lp = e.compute_log_probs(samples(3 if rank == 0 else 1, 180 + rank, vocab=512))
        allc = [None, None]
        dist.all_gather_object(allc, counts)
        res = {"losses": losses, "counts": allc, "n_logprobs": len(lp)}
    elif mode == "aux_dp":
        # only the MoE auxiliary loss has a gradient (loss masks are zero): two data-parallel ranks with two
        # micro-batches each must produce the gradient of one rank running the same four micro-batches
        ps.initialize_model_parallel(tp=1)
        e = engine(MOE_CFG, 1)
        batch = samples(8, 190, vocab=512)
        for b in batch:
            b["loss_mask"] = torch.zeros_like(b["loss_mask"])
        m = e.finetune_step(batch[rank * 4:(rank + 1) * 4])
        res = {"grad_norm": m["grad_norm"]}
    elif mode == "dyncp":
        # data-parallel pool of two ranks; sequences longer than the per-rank budget run on both ranks (CP 2), the
        # others on one: the step must equal a single process training on the union of the two ranks' samples
        ps.initialize_model_parallel(tp=1)
        mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
        pc = PolicyConfig(recompute="none", without_ref=True)
        pc.dist_config.dynamic_context_parallel = True
        pc.dist_config.max_seqlen_per_dp_cp_rank = 40
        oc = OptimizerConfig(lr=1e-3, lr_decay_style="constant", weight_decay=0.0, max_grad_norm=1.0)
        e = TrainingEngine(pc, oc, TrainingConfig(train_mbs=2, train_gbs=8), model_cfg=mcfg)
        e.setup_model_and_get_optimizer(seed=11)
        assert e._dcp is not None
        losses = [e.finetune_step(samples(8, 210 + s, L=72)[rank::world])["lm_loss"] for s in range(3)]
        mine = samples(6, 219, L=72)[rank::world]
        lp = e.compute_log_probs(mine)
        allp = [None, None]
        dist.all_gather_object(allp, [x["logprobs"].tolist() for x in lp])
        res = {"losses": losses, "grad_norm": float(e.optimizer.last_grad_norm), "logprobs": allp}
    elif mode == "dp_grpo_balance":
        # GRPO on two data-parallel ranks whose responses differ in length (different stop tokens): with
        # policy.balance_dp_seqlen the update runs on evened-out token counts; smart-pad groups similar lengths
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        from test_grpo_cpu import make_cfg, reward_has_small_token
        from gcore_b200.trainer.grpo_trainer import GrpoTrainer
        ps.initialize_model_parallel(tp=1)
        cfg = make_cfg()
        cfg.policy.balance_dp_seqlen = True
        cfg.policy.smart_pad_train = True
        cfg.training.rollout_gbs, cfg.training.train_gbs = 8, 32   # 4 prompts x 4 samples per rank
        cfg.sampler.infer_engine_configs[0].generate_max_tokens = 4 if rank == 0 else 24
        torch.manual_seed(0)
        tr = GrpoTrainer(cfg, model_cfg=get_preset("tiny_llama", dtype="float32", qkv_bias=True),
                         reward_fn=reward_has_small_token).setup()
        g = torch.Generator().manual_seed(5 + rank)
        prompts = [torch.randint(3, 1024, (6 + i,), generator=g).tolist() for i in range(4)]
        m = tr.step(prompts)
        res = {"before": m["rollout-metrics/dp_balance_tokens_before"],
               "after": m["rollout-metrics/dp_balance_tokens_after"], "grad_norm": m["policy/grad_norm"]}
        allres = [None, None]
        dist.all_gather_object(allres, res)
        res = {"ranks": allres}
    elif mode == "pg_offload":
        # data-parallel SFT steps with the communicators destroyed and re-created in between (what a rollout phase
        # does under policy.offload_process_group): the run equals one without the cycle
        ps.initialize_model_parallel(tp=1)
        mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
        e = engine(mcfg, 1)
        losses = []
        for s_ in range(3):
            losses.append(e.finetune_step(samples(8, 230 + s_)[rank::world])["lm_loss"])
            if s_ == 0:
                n = e.offload_process_groups()
                assert n >= 1 and ps.get_data_parallel_group() is None
                assert e.reload_process_groups() >= 1 and ps.get_data_parallel_group() is not None
        res = {"losses": losses}
    elif mode == "nodistopt":
        ps.initialize_model_parallel(tp=1)
        mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
        norms = []
        for dist_opt in (True, False):
            pc = PolicyConfig(recompute="none", without_ref=True)
            oc = OptimizerConfig(lr=1e-3, lr_decay_style="constant", weight_decay=0.0, max_grad_norm=1.0,
                                 use_distributed_optimizer=dist_opt)
            e = TrainingEngine(pc, oc, TrainingConfig(train_mbs=2, train_gbs=8), model_cfg=mcfg)
            e.setup_model_and_get_optimizer(seed=11)
            norms.append(e.finetune_step(samples(8, 200)[rank::world])["grad_norm"])
        res = {"norms": norms}
    elif mode == "tp_topk":
        # vocabulary-sharded head with top-k / top-p / min-p: the filter must act on the whole vocabulary
        from gcore_b200.models.gpt import GPTModel
        from gcore_b200.rollout.engine import InferEngine, RolloutWeights, SamplingParams
        ps.initialize_model_parallel(tp=2)
        mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
        model = GPTModel(mcfg, tp_size=2, recompute="none")
        model.reset_parameters(21)
        model.eval()
        eng = InferEngine(mcfg, RolloutWeights.from_model(model), tp_size=2,
                          tp_group=ps.get_tensor_model_parallel_group(), max_running_requests=4, max_model_len=48,
                          kv_block_size=4, sync_interval=2, use_cuda_graph=False)
        g = torch.Generator().manual_seed(100)
        prompts = [torch.randint(3, 1024, (5 + 2 * i,), generator=g).tolist() for i in range(2)]
        out_all = {}
        for name, kw in (("top_k", dict(top_k=3)), ("top_p", dict(top_p=0.3)), ("min_p", dict(min_p=0.2))):
            reqs = eng.generate(prompts, SamplingParams(max_new_tokens=6, temperature=1.5, seed=5, **kw), n=2)
            out_all[name] = {"tokens": [r.out_tokens for r in reqs], "logprobs": [r.out_logprobs for r in reqs]}
        res = {"prompts": prompts, "out": out_all}
    if rank == 0:
        json.dump(res, open(out, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
