"""Every entry point runs in-process on a tiny CPU model from a YAML file plus dotted overrides."""
import json
import os

import pytest
import torch
import yaml

TINY = {"model_arch": "tiny_llama", "model_config": {"dtype": "float32"}, "recompute": "none"}


def _rl_yaml(tmp_path, **extra):
    cfg = {"training": {"rollout_gbs": 4, "sampling_repeat_n": 2, "train_gbs": 8, "train_mbs": 4, "total_ppo_step": 2,
                        "seed": 3},
           "policy": dict(TINY), "optimizer": {"lr": 1e-3, "lr_decay_style": "constant", "weight_decay": 0.0},
           "sampler": {"infer_engine_configs": [{"generate_max_tokens": 8, "max_model_len": 40, "kv_block_size": 4,
                                                  "disable_cuda_graph": True}]},
           "data": {"max_prompt_length": 16, "synthetic": {"num_samples": 32, "prompt_len": 8, "lo": 3, "hi": 1000}},
           "report": {"log_dir": str(tmp_path / "logs")}}
    cfg.update(extra)
    p = tmp_path / "rl.yaml"
    p.write_text(yaml.safe_dump(cfg))
    return str(p)


def _sft_yaml(tmp_path):
    cfg = {"training": {"train_gbs": 4, "train_mbs": 2, "exit_step": 3, "seq_length": 32, "calc_mfu_freq": 0},
           "policy": dict(TINY), "optimizer": {"lr": 1e-3, "lr_decay_style": "constant"},
           "data": {"synthetic": {"num_samples": 64, "seq_len": 32, "loss_tokens": 16}},
           "report": {"log_dir": str(tmp_path / "logs")}}
    p = tmp_path / "sft.yaml"
    p.write_text(yaml.safe_dump(cfg))
    return str(p)


def test_rl_and_preference_entries(tmp_path):
    from gcore_b200.entry import (train_lm_dpo, train_lm_grpo, train_lm_grpo_single_ctrl, train_lm_reward_model)
    y = _rl_yaml(tmp_path)
    assert train_lm_grpo.main(["--config", y]) == 0
    assert train_lm_grpo_single_ctrl.main(["--config", y, "training.single_controller=true"]) == 0
    small = ["training.train_gbs=4", "training.rollout_gbs=4"]
    assert train_lm_dpo.main(["--config", y] + small) == 0
    assert train_lm_dpo.main(["--config", y, "dpo_beta=0.3", "dpo_label_smoothing=0.1", "dpo_sft_loss_coef=0.5",
                              "reference_free=true"] + small) == 0
    assert train_lm_reward_model.main(["--config", y, "rm_margin=0.5"] + small) == 0


def test_distillation_entry_on_and_off_policy(tmp_path):
    from gcore_b200.configs.base import ConfigError
    from gcore_b200.entry import train_lm_distill
    y = _rl_yaml(tmp_path, teacher=dict(TINY), ppo={"advantage_type": "on_policy_distill", "loss_func": "opd"})
    hist = train_lm_distill.main(["--config", y])
    assert len(hist) == 2 and all(m["policy/grad_norm"] > 0 for m in hist)
    hist = train_lm_distill.main(["--config", y, "+distill_mode=off_policy", "training.total_ppo_step=3"])
    assert len(hist) == 3 and all(torch.isfinite(torch.tensor(m["lm_loss"])) for m in hist)
    with pytest.raises(ConfigError):   # the distillation advantage without a teacher is a configuration error
        train_lm_distill.main(["--config", y, "~teacher"])


def test_on_policy_distillation_moves_the_student_towards_the_teacher():
    """The per-token advantage is the teacher - student log-prob gap: after some steps the student assigns its own
    samples a likelihood closer to the teacher's."""
    from test_grpo_cpu import make_cfg
    from gcore_b200.configs.config import PolicyConfig
    from gcore_b200.models.config import get_preset
    from gcore_b200.trainer.grpo_trainer import GrpoTrainer
    torch.manual_seed(0)
    cfg = make_cfg()
    cfg.teacher = PolicyConfig(recompute="none", without_ref=True)
    cfg.ppo.advantage_type, cfg.ppo.loss_func = "on_policy_distill", "opd"
    cfg.optimizer.lr = 5e-3
    # a small vocabulary (the student's samples cover it) and a sharpened teacher (x10 output weights) make the
    # signal visible within a few dozen steps
    tr = GrpoTrainer(cfg, model_cfg=get_preset("tiny_llama", dtype="float32", vocab_size=32)).setup()
    assert tr.teacher is not None and tr.teacher.optimizer is None
    with torch.no_grad():
        tr.teacher.model.output_weight().mul_(10.0)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 32, (8,), generator=g).tolist() for _ in range(4)]

    def gap():
        tot, n = 0.0, 0.0
        for s in tr.last_samples:
            m = torch.as_tensor(s["mask"]).float()
            tot += float(((s["teacher_logprobs"] - s["logprobs"]) * m).sum())
            n += float(m.sum())
        return tot / n

    gaps = []
    for _ in range(28):
        tr.step(prompts)
        gaps.append(gap())
    # the gap is -KL(student || teacher) estimated on the student's samples: it rises towards zero
    assert sum(gaps[-4:]) / 4 > sum(gaps[:2]) / 2 + 0.8, gaps


def test_pretrain_entry_reads_a_token_stream_and_dataloader_verifies(tmp_path):
    from gcore_b200.data.datasets import IndexedJsonlDataset, PretrainTokenDataset
    from gcore_b200.entry import train_lm_pretrain, verify_dataloader
    docs = [[(i * 7 + j) % 500 + 3 for j in range(11 + i % 5)] for i in range(40)]
    f = tmp_path / "pre.jsonl"
    f.write_text("\n".join(json.dumps({"tokens": d}) for d in docs) + "\n")
    ds = PretrainTokenDataset(IndexedJsonlDataset(str(f)), None, 32, eod_id=1)
    stream = [t for d in docs for t in d + [1]]
    assert len(ds) == len(stream) // 32
    for r in (0, 3, len(ds) - 1):       # rows are exact slices of the concatenated documents, loss on every token
        assert ds[r]["tokens"].tolist() == stream[r * 32:(r + 1) * 32] and ds[r]["prompt_length"] == 0
    y = _sft_yaml(tmp_path)
    hist = train_lm_pretrain.main(["--config", y, f"data.train_data_path={f}"])
    assert len(hist) == 3
    rep = verify_dataloader.main(["--config", y, "+verify.batches=6", "+verify.dp_size=2"])
    assert rep["resume_ok"] and rep["disjoint_ok"] and rep["tokens"] == 6 * 2 * 2 * 32


def test_eval_infer_embedding_and_vlm_entries(tmp_path):
    from gcore_b200.entry import lm_eval, lm_infer, train_lm_embedding, train_vlm
    y = _rl_yaml(tmp_path)
    out = tmp_path / "metrics.json"
    m = lm_eval.main(["--config", y, "+task.eval.batches=2", "+task.eval.ks=[1,2]", f"+task.eval.out={out}"])
    assert m["eval/num_samples"] == 16 and "eval/pass@2" in m and json.load(open(out)) == m
    gen = tmp_path / "gen.jsonl"
    assert lm_infer.main(["--config", y, f"+task.infer.out={gen}"]) == 0
    assert len(open(gen).read().splitlines()) == 8
    hist = train_lm_embedding.main(["--config", _sft_yaml(tmp_path), "training.exit_step=4", "training.train_gbs=8",
                                    "training.train_mbs=16"])
    assert len(hist) == 4 and all(0.0 <= h["embedding/acc"] <= 1.0 for h in hist)
    vlm = ["policy.image_token_id=5", "+policy.vision_config.patch_size=2", "+policy.vision_config.hidden_size=64",
           "+policy.vision_config.num_layers=1", "+policy.vision_config.num_heads=2",
           "+policy.vision_config.ffn_hidden_size=128", "+policy.vision_config.max_grid=8"]
    hist = train_vlm.main(["--config", y, "training.total_ppo_step=4"] + vlm)
    assert len(hist) == 4 and hist[-1]["lm_loss"] < hist[0]["lm_loss"]
    hist = train_vlm.main(["--config", y, "+task.vlm.mode=grpo"] + vlm)
    assert len(hist) == 2 and "rollout-rewards/mean" in hist[0]


def test_record_replay_and_external_rollout_generators(tmp_path):
    """A GRPO run records its rollouts; a second run replays them without sampling and takes the same training steps;
    an external generate function can stand in for the engine."""
    from gcore_b200.entry import train_lm_grpo
    from gcore_b200.trainer.rl_loop import RlLoop
    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import RlConfig
    y = _rl_yaml(tmp_path)
    rec = tmp_path / "rollouts.jsonl"
    a = RlLoop(load_config(RlConfig, y, [f"+task.rollout.record_path={rec}"])).setup()
    ha = a.run()
    assert len(open(rec).read().splitlines()) == 2
    b = RlLoop(load_config(RlConfig, y, ["policy.rollout_gen_type=replay", f"+task.rollout.replay_path={rec}"])).setup()
    calls = []
    b.trainer.rollout = lambda prompts: calls.append(1)   # the engine must not be asked
    hb = b.run()
    assert not calls and len(hb) == 2
    for ma, mb in zip(ha, hb):
        assert abs(ma["policy/grad_norm"] - mb["policy/grad_norm"]) < 1e-5
        assert abs(ma["ppo-metrics/pg_loss"] - mb["ppo-metrics/pg_loss"]) < 1e-6
    # external generator: a plug-in function produces the samples (here: it delegates to the trainer's engine)
    plug = tmp_path / "my_gen.py"
    plug.write_text("CALLS = []\n\n\ndef generate(prompts, step, trainer):\n    CALLS.append(step)\n"
                    "    return trainer.rollout(prompts)\n")
    c = RlLoop(load_config(RlConfig, y, ["policy.rollout_gen_type=external",
                                         f"policy.rollout_gen_py_path={plug}"])).setup()
    hc = c.run()
    assert len(hc) == 2 and c.generator.fn.__module__.startswith("_gcore_plugin_")
    assert abs(hc[0]["policy/grad_norm"] - ha[0]["policy/grad_norm"]) < 1e-5


def test_agentic_rollouts_train_with_grpo_and_with_a_teacher():
    """Multi-turn FrozenLake trajectories produced by the trainer's own engine (one generate call per turn): the
    assistant tokens of all turns are the training targets, rollout log-probs line up with the trainer's, and the
    same generator feeds on-policy distillation (teacher scores on the student's trajectories)."""
    from test_grpo_cpu import make_cfg
    from gcore_b200.agentic import FrozenLakeEnv
    from gcore_b200.configs.config import PolicyConfig
    from gcore_b200.models.config import get_preset
    from gcore_b200.rollout_generator.generators import AgenticRolloutGenerator
    from gcore_b200.trainer.grpo_trainer import GrpoTrainer

    class Tok:   # byte-ish tokenizer inside the tiny vocabulary
        def encode(self, t):
            return [ord(c) % 250 + 3 for c in t]

        def decode(self, ids):
            return "".join(chr((i - 3) % 250) for i in ids)

    for distill in (False, True):
        torch.manual_seed(0)
        cfg = make_cfg()
        cfg.training.rollout_gbs, cfg.training.sampling_repeat_n, cfg.training.train_gbs = 2, 2, 4
        cfg.sampler.infer_engine_configs[0].generate_max_tokens = 6
        cfg.sampler.infer_engine_configs[0].max_model_len = 640
        if distill:
            cfg.teacher = PolicyConfig(recompute="none", without_ref=True)
            cfg.ppo.advantage_type, cfg.ppo.loss_func = "on_policy_distill", "opd"
        tr = GrpoTrainer(cfg, model_cfg=get_preset("tiny_llama", dtype="float32")).setup()
        gen = AgenticRolloutGenerator(tr, cfg, lambda: FrozenLakeEnv(size=3), Tok(), max_turns=2, max_new_tokens=6)
        samples = gen(iter([]), 0)
        assert len(samples) == 4 and all(1 <= s["num_turns"] <= 2 for s in samples)
        s = samples[0]
        n_assist = int(s["mask"].sum())
        assert n_assist == 6 * s["num_turns"] and s["tokens"].numel() > s["prompt_length"] + n_assist - 1
        if not distill:
            for x in samples:
                x["rewards"] = torch.tensor(float(x["num_turns"]))   # any signal: longer episodes score higher
        m = tr.train_on_samples(samples)
        assert m["policy/grad_norm"] >= 0 and "ppo-metrics/pg_loss" in m
        keep = s["mask"] > 0
        assert torch.allclose(s["logprobs"][keep], s["rollout_log_probs"][keep], atol=2e-3)
        if distill:
            assert "teacher_logprobs" in s and float(s["advantages"][~keep].abs().sum()) == 0.0


def test_agentic_generator_from_config(tmp_path):
    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import RlConfig
    from gcore_b200.rollout_generator.generators import AgenticRolloutGenerator
    from gcore_b200.trainer.rl_loop import RlLoop
    y = _rl_yaml(tmp_path)
    loop = RlLoop(load_config(RlConfig, y, [
        "policy.rollout_gen_type=agentic", "+task.rollout.env=frozen_lake", "+task.rollout.env_kwargs.size=3",
        "+task.rollout.max_turns=2", "+task.rollout.max_new_tokens=4", "training.rollout_gbs=2",
        "training.sampling_repeat_n=2", "training.train_gbs=4", "training.total_ppo_step=1",
        "sampler.infer_engine_configs.0.max_model_len=640"])).setup()
    assert isinstance(loop.generator, AgenticRolloutGenerator)
    hist = loop.run()
    assert len(hist) == 1 and "rollout-rewards/mean" in hist[0]


def test_per_token_dumps_and_debug_rollout_paths(tmp_path):
    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import RlConfig
    from gcore_b200.trainer.rl_loop import RlLoop
    y = _rl_yaml(tmp_path)
    rec = tmp_path / "dbg_rollouts.jsonl"
    loop = RlLoop(load_config(RlConfig, y, ["training.ppo_dump_metrics_interval=1",
                                            f"debug.dump_rollout_path={rec}"])).setup()
    loop.run()
    d = tmp_path / "logs" / "token_dumps"
    files = sorted(os.listdir(d))
    assert files == ["step0000000_rank0.jsonl", "step0000001_rank0.jsonl"]
    rows = [json.loads(l) for l in open(d / files[0])]
    assert len(rows) == 8
    r = rows[0]
    n = len(r["tokens"])
    assert len(r["logprobs"]) == n and len(r["advantages"]) == n and len(r["mask"]) == n and "reward" in r
    assert all(a == 0.0 for a in r["advantages"][:r["prompt_length"] - 1])       # nothing to learn on the prompt
    assert len(open(rec).read().splitlines()) == 2
    replay = RlLoop(load_config(RlConfig, y, [f"debug.replay_rollout_path={rec}"])).setup()
    replay.trainer.rollout = None      # would raise if the engine were asked
    assert len(replay.run()) == 2


def test_debug_flags_are_honoured(tmp_path):
    """debug.debug_update_weight verifies the hand-over, check_rollout_batches validates the samples, and
    trace_python_calls writes a call trace of the package."""
    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import RlConfig
    from gcore_b200.trainer.rl_loop import RlLoop
    y = _rl_yaml(tmp_path)
    loop = RlLoop(load_config(RlConfig, y, ["debug.debug_update_weight=true", "debug.trace_python_calls=true",
                                            "training.total_ppo_step=1", "policy.share_rollout_weights=false"])).setup()
    loop.run()     # separate rollout copy: the verification really compares two sets of tensors
    trace = open(tmp_path / "logs" / "python_calls_rank0.log").read()
    assert "train_on_samples" in trace and "rollout" in trace
    # a malformed sample is caught before any compute
    bad = [{"tokens": torch.tensor([1, 2, 3]), "prompt_length": 5, "rewards": torch.tensor(0.0), "group_id": 0}]
    with pytest.raises(AssertionError, match="prompt_length"):
        loop.trainer.train_on_samples(bad)
    # a rollout copy that went out of sync is reported
    with torch.no_grad():
        loop.trainer.engine.w.layers[0].o_w.add_(1.0)
    from gcore_b200.rollout.weight_sync import verify
    assert verify(loop.trainer.policy, loop.trainer.engine)


def test_step_profiler_from_config(tmp_path):
    """report.profile.enable: the configured steps are traced with torch.profiler, a Chrome trace lands in the export
    directory and the communication / compute split joins the step's metrics."""
    from gcore_b200.entry import train_lm_finetune
    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import FinetuneConfig
    from gcore_b200.trainer.finetune_trainer import FinetuneTrainer
    y = _sft_yaml(tmp_path)
    cfg = load_config(FinetuneConfig, y, ["report.profile.enable=true", "report.profile.profile_start_step=1",
                                          "report.profile.profile_end_step=1",
                                          f"report.profile.export_dir={tmp_path / 'prof'}"])
    tr = FinetuneTrainer(cfg).setup()
    hist = tr.train_loop()
    assert len(hist) == 3 and "profile/comm_frac" in hist[1] and "profile/comm_frac" not in hist[0]
    files = os.listdir(tmp_path / "prof")
    assert files == ["trace_rank0_step1-1.json"] and os.path.getsize(tmp_path / "prof" / files[0]) > 1000


def test_periodic_evaluation_inside_the_rl_loop(tmp_path):
    """``training.eval_interval`` with a held-out prompt set: the loop evaluates with the evaluation sampling
    parameters (greedy, shorter) and its own samples-per-prompt, and keeps training afterwards."""
    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import RlConfig
    from gcore_b200.trainer.rl_loop import RlLoop
    y = _rl_yaml(tmp_path)
    cfg = load_config(RlConfig, y, ["training.eval_interval=2", "training.total_ppo_step=4",
                                    "+data.synthetic.eval_num_samples=8", "+task.eval.repeat_n=1",
                                    "+task.eval.ks=[1]", "+task.eval.threshold=-1.0",
                                    "+sampler.infer_engine_configs.0.eval_generate_params.greedy=true",
                                    "+sampler.infer_engine_configs.0.eval_generate_params.max_tokens=4"])
    loop = RlLoop(cfg).setup()
    seen = []
    orig = loop.trainer.rollout

    def spy(prompts, n=None, sampling=None):
        out = orig(prompts, n=n, sampling=sampling)
        if sampling is not None:
            seen.append((len(prompts), n, dict(sampling), max(s["sequence_length"] - s["prompt_length"] for s in out)))
        return out
    loop.trainer.rollout = spy
    hist = loop.run()
    assert len(hist) == 4 and [e["step"] for e in loop.eval_history] == [2, 4]
    e = loop.eval_history[0]
    assert e["eval/num_samples"] == 8.0 and e["eval/pass@1"] == 1.0 and e["eval/response_length"] <= 4.0
    assert seen[0][:2] == (8, 1) and seen[0][2] == {"greedy": True, "max_new_tokens": 4} and seen[0][3] <= 4
    # greedy decoding of a fixed prompt set: the two evaluations differ only through the weight updates in between
    assert loop.eval_history[0].keys() == loop.eval_history[1].keys()


def test_finetune_length_from_epochs_and_manual_gc(tmp_path):
    """Without a step count the job runs ``num_train_epoches`` passes over the data, the decay of the learning rate
    spans the same steps, and ``manual_gc`` keeps the collector off inside the loop and restores it afterwards."""
    import gc
    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import FinetuneConfig
    from gcore_b200.trainer.finetune_trainer import FinetuneTrainer
    y = _sft_yaml(tmp_path)
    cfg = load_config(FinetuneConfig, y, ["~training.exit_step", "training.num_train_epoches=2",
                                          "data.synthetic.num_samples=16", "training.manual_gc=true",
                                          "optimizer.lr_decay_style=linear", "optimizer.min_lr=0.0"])
    tr = FinetuneTrainer(cfg).setup()
    assert tr.total_steps == 8 and tr.engine.optimizer.total_steps == 8     # 16 samples / batch 4 x 2 epochs
    state = []
    orig = tr.train_one_step

    def spy():
        state.append(gc.isenabled())
        return orig()
    tr.train_one_step = spy
    hist = tr.train_loop()
    assert len(hist) == 8 and state == [False] * 8 and gc.isenabled()
    lrs = [m["lr"] for m in hist]
    assert lrs[0] > lrs[-1] and lrs[-1] <= 0.3 * lrs[0]


def test_fsdp2_backend_is_selected_from_config_and_resumes(tmp_path):
    """``training.training_backend=fsdp2`` builds the ZeRO-3 engine, trains through the ordinary SFT trainer, saves a
    torch.distributed.checkpoint tree at the save interval and resumes from it."""
    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import FinetuneConfig
    from gcore_b200.engine.fsdp2_engine import Fsdp2Engine
    from gcore_b200.trainer.finetune_trainer import FinetuneTrainer
    y = _sft_yaml(tmp_path)
    over = ["training.training_backend=fsdp2", "training.save_interval=3",
            f"checkpoint.save_ckpt_path={tmp_path / 'ck'}"]
    tr = FinetuneTrainer(load_config(FinetuneConfig, y, over)).setup()
    assert isinstance(tr.engine, Fsdp2Engine)
    hist = tr.train_loop()
    assert len(hist) == 3 and hist[-1]["lm_loss"] < hist[0]["lm_loss"] + 0.5
    tr2 = FinetuneTrainer(load_config(FinetuneConfig, y, over + ["training.auto_load_from_save_ckpt=true",
                                                                  "training.exit_step=4"])).setup()
    assert tr2.step == 3
    for (n, p), (_, q) in zip(tr.engine.model.named_parameters(), tr2.engine.model.named_parameters()):
        assert torch.equal(p, q), n
    assert len(tr2.train_loop()) == 1
