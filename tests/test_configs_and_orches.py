import os
import subprocess
import sys
import time

import pytest
import torch
import yaml

from gcore_b200.configs.base import ConfigError, apply_overrides, from_dict, load_config
from gcore_b200.configs.config import FinetuneConfig, RlConfig
from gcore_b200.core.parallel_state import plan_groups
from gcore_b200.orches.failure import (FailureEvent, FailureType, FaultInjector, Heartbeat, InjectedFault,
                                       MockNodeReplacer, check_liveness, run_with_recovery)
from gcore_b200.orches.resource_allocator import allocation_from_config, expected_nnodes, sort_bundles

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_yaml_overrides_and_validation(tmp_path):
    y = tmp_path / "rl.yaml"
    y.write_text(yaml.safe_dump({"training": {"rollout_gbs": 16, "sampling_repeat_n": 4, "train_gbs": 64},
                                 "policy": {"dist_config": {"tensor_model_parallel_size": 2}},
                                 "ppo": {"ppo_ratio_eps": 0.3}}))
    cfg = load_config(RlConfig, str(y), ["optimizer.lr=3e-6", "+task.name=demo", "ppo.ppo_clip_ratio_high=0.4",
                                         "sampler.infer_engine_configs.0.temperature=0.7"])
    assert cfg.optimizer.lr == 3e-6 and cfg.task["name"] == "demo"
    assert cfg.ppo.clip_low == 0.3 and cfg.ppo.clip_high == 0.4
    assert cfg.sampler.infer_engine_configs[0].temperature == 0.7
    assert cfg["policy"]["dist_config"].sequence_parallel is True
    assert cfg.training.sampling_keep_n == 4  # defaults to repeat_n
    with pytest.raises(ConfigError):
        from_dict(RlConfig, {"ppo": {"loss_func": "gspo"}})  # gspo forbids per-token loss
    with pytest.raises(ConfigError):
        from_dict(RlConfig, {"ppo": {"advantage_type": "ppo"}})  # needs critic
    with pytest.raises(ConfigError):
        from_dict(RlConfig, {"training": {"rollout_max_staleness": 2}})
    with pytest.raises(ConfigError):
        from_dict(RlConfig, {"trainnig": {}})
    assert apply_overrides({"a": {"b": 1}}, ["~a.b", "a.c=[1,2]"]) == {"a": {"c": [1, 2]}}
    ft = from_dict(FinetuneConfig, {"policy": {"dist_config": {"tensor_model_parallel_size": 1}}})
    assert ft.policy.dist_config.sequence_parallel is False


def test_plan_groups_rank_order_and_expert_groups():
    fam, dense, expert = plan_groups(16, tp=2, pp=2, cp=2, ep=4, etp=1)
    assert dense["dp"] == 2 and expert["edp"] == 2
    assert fam["tp"][0] == [0, 1] and fam["cp"][0] == [0, 2] and fam["dp"][0] == [0, 4] and fam["pp"][0] == [0, 8]
    assert fam["dp_cp"][0] == [0, 2, 4, 6]
    assert fam["ep"][0] == [0, 1, 2, 3] and fam["edp"][0] == [0, 4]
    # every family partitions the world
    for name, lists in fam.items():
        flat = sorted(r for g in lists for r in g)
        assert flat == list(range(16)), name
    with pytest.raises(ValueError):
        plan_groups(6, tp=4)


def test_allocation_modes():
    base = {"training": {"rollout_gbs": 8, "sampling_repeat_n": 8, "train_gbs": 64},
            "policy": {"dist_config": {"tensor_model_parallel_size": 2, "nnodes": 1}},
            "sampler": {"infer_engine_configs": [{"dist_config": {"tensor_model_parallel_size": 2}}]}}
    a = allocation_from_config(from_dict(RlConfig, base))
    assert a.roles["train"].gpus == list(range(8)) and a.roles["sampler"].gpus == list(range(8))
    assert a.roles["train"].dp == 4 and len(a.roles["sampler"].engines()) == 4
    d = dict(base, placement_type="disaggregated")
    a = allocation_from_config(from_dict(RlConfig, d), role_gpus={"train": 4, "sampler": 4})
    assert a.roles["train"].gpus == [0, 1, 2, 3] and a.roles["sampler"].gpus == [4, 5, 6, 7]
    with pytest.raises(ValueError):
        allocation_from_config(from_dict(RlConfig, d), role_gpus={"train": 3, "sampler": 5})
    assert expected_nnodes(17, 8) == 3
    assert sort_bundles([("10.0.0.2", 1), ("10.0.0.1", 3), ("10.0.0.1", 0)]) == [2, 1, 0]


def test_failure_primitives(tmp_path):
    hb = Heartbeat(str(tmp_path), 0)
    hb.stamp(3)
    Heartbeat(str(tmp_path), 1).stamp(3)
    assert check_liveness(str(tmp_path), 2, max_wait_s=60) is None
    ev = check_liveness(str(tmp_path), 2, max_wait_s=60, now=time.time() + 120)
    assert ev is not None and ev.type == FailureType.HANG
    inj = FaultInjector({"raise_at_step": 2, "rank": 1, "only_attempt": 0}, rank=1, attempt=0)
    inj.at_step(1)
    with pytest.raises(InjectedFault):
        inj.at_step(2)
    FaultInjector({"raise_at_step": 2, "rank": 1, "only_attempt": 0}, rank=1, attempt=1).at_step(2)
    calls = []

    def attempt(i):
        calls.append(i)
        return FailureEvent(FailureType.CRASH, rank=0) if i == 0 else None

    rep = MockNodeReplacer()
    events = run_with_recovery(attempt, max_restart_attempts=2, node_replacer=rep)
    assert calls == [0, 1] and len(events) == 1 and len(rep.evicted) == 1 and rep.provisioned == 1
    with pytest.raises(RuntimeError):
        run_with_recovery(lambda i: FailureEvent(FailureType.HANG), max_restart_attempts=1)


def test_crash_is_detected_and_job_resumes_from_checkpoint(tmp_path):
    """Two gloo ranks run SFT; rank 1 raises at step 3 of the first attempt.  The launcher reports a CRASH, the
    recovery loop relaunches, the second attempt resumes from the step-2 checkpoint and finishes."""
    from gcore_b200.orches.launcher import LocalLauncher
    ckpt = tmp_path / "ckpt"
    cfg = {"training": {"train_gbs": 4, "train_mbs": 2, "exit_step": 5, "save_interval": 2, "seq_length": 64,
                        "calc_mfu_freq": 0},
           "policy": {"model_arch": "tiny_llama", "model_config": {"dtype": "float32"}, "recompute": "none"},
           "optimizer": {"lr": 1e-3, "lr_decay_style": "constant"},
           "data": {"synthetic": {"num_samples": 64, "seq_len": 64, "loss_tokens": 32}},
           "checkpoint": {"save_ckpt_path": str(ckpt)},
           "report": {"log_dir": str(tmp_path / "logs")},
           "debug": {"fault_injection": {"raise_at_step": 3, "rank": 1, "only_attempt": 0}}}
    y = tmp_path / "sft.yaml"
    y.write_text(yaml.safe_dump(cfg))
    launcher = LocalLauncher(2, heartbeat_dir=str(tmp_path / "hb"), max_wait_s=600, poll_s=0.2,
                             extra_env={"PYTHONPATH": ROOT, "OMP_NUM_THREADS": "2"})

    def attempt(i):
        launcher.launch(["-m", "gcore_b200.entry.train_lm_finetune", "--config", str(y)], attempt=i)
        return launcher.wait()

    events = run_with_recovery(attempt, max_restart_attempts=1, node_replacer=MockNodeReplacer())
    assert len(events) == 1 and events[0].type == FailureType.CRASH
    from gcore_b200.checkpoint.torch_dist import read_latest_step
    assert read_latest_step(str(ckpt)) == 5
    assert sorted(os.listdir(ckpt))[:3] == ["iter_0000002", "iter_0000004", "iter_0000005"]


def test_every_recipe_yaml_loads_and_names_a_known_model():
    import glob
    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import FinetuneConfig, RlConfig
    from gcore_b200.models.config import PRESETS
    from gcore_b200.configs.base import load_yaml
    files = sorted(glob.glob(os.path.join(ROOT, "tasks", "math_rl", "yaml", "*.yaml")))
    assert len(files) >= 35
    for f in files:
        raw = load_yaml(f)                    # variants name a ``base:`` recipe and spell only what they change
        cfg = load_config(RlConfig if "sampler" in raw else FinetuneConfig, f, [])
        assert cfg.policy.model_arch in PRESETS, f
        if "teacher" in raw:
            assert cfg.teacher.model_arch in PRESETS and cfg.ppo.advantage_type == "on_policy_distill"
        if raw["policy"].get("fp8"):
            assert cfg.policy.fp8 and cfg.policy.lora.enabled and "linear_kv_up_proj" in cfg.policy.lora.target_modules


def test_recipe_variants_change_what_they_say_and_plug_ins_resolve():
    from gcore_b200.configs.base import ConfigError, import_from_path, load_config, load_yaml
    from gcore_b200.configs.config import FinetuneConfig, RlConfig
    y = lambda n: os.path.join(ROOT, "tasks", "math_rl", "yaml", n)
    base = load_config(RlConfig, y("grpo_qwen2.5_7b.yaml"), [])
    want = {"rl_cispo.yaml": lambda c: c.ppo.loss_func == "cispo" and c.ppo.ppo_clip_ratio_high == 0.28,
            "rl_gspo.yaml": lambda c: c.ppo.loss_func == "gspo" and not c.ppo.per_token_loss,
            "rl_icepop.yaml": lambda c: c.ppo.offpolicy_correction == "icepop" and c.ppo.offpolicy_correction_lower == 0.5,
            "rl_clip_cov.yaml": lambda c: c.ppo.entropy_regularization_type == "clip-cov",
            "rl_dynamic_sampling.yaml": lambda c: c.training.dynamic_sampling.enable and c.policy.without_ref,
            "rl_async.yaml": lambda c: c.training.async_rollout and c.training.rollout_max_staleness == 1,
            "rl_online_mtp.yaml": lambda c: c.training.online_mtp_sft and c.policy.model_config["mtp_num_layers"] == 1,
            "rl_disaggregated.yaml": lambda c: c.placement_type == "disaggregated" and c.disaggregated_train_gpus == 4,
            "rl_sampling_filters.yaml": lambda c: c.sampler.infer_engine_configs[0].repetition_penalty == 1.1,
            "rl_dynamic_cp.yaml": lambda c: c.policy.dist_config.dynamic_context_parallel
            and c.policy.dist_config.context_parallel_size == 4,
            "rl_gdpo.yaml": lambda c: c.ppo.advantage_type == "gdpo" and c.ppo.gdpo_reward_weights["format"] == 0.2}
    for name, check in want.items():
        c = load_config(RlConfig, y(name), [])
        assert check(c), name
        # everything the variant does not mention is the base recipe's
        assert c.policy.model_arch == base.policy.model_arch and c.training.rollout_gbs == base.training.rollout_gbs
        assert c.report.run_name == name[:-5]
    s = load_config(FinetuneConfig, y("sft_fsdp2.yaml"), [])
    assert s.training.training_backend == "fsdp2" and s.policy.dist_config.tensor_model_parallel_size == 1
    assert load_config(FinetuneConfig, y("sft_with_mtp.yaml"), []).policy.model_config["mtp_num_layers"] == 1
    assert load_config(FinetuneConfig, y("sft_muon.yaml"), []).optimizer.optimizer_type == "muon"
    c = load_config(RlConfig, y("rl_custom_advantage.yaml"), [])
    fn = import_from_path(os.path.join(ROOT, c.ppo.advantage_py_path), c.ppo.advantage_fn_name)
    import torch
    smp = [{"group_id": 0, "rewards": torch.tensor(r), "mask": torch.tensor([0.0, 1.0, 1.0])} for r in (1.0, 0.0, 0.0)]
    out = fn(smp, c.ppo)
    assert out[0]["advantages"].tolist() == [0.0, 1.0, 1.0] and out[1]["advantages"].tolist() == [0.0, -0.5, -0.5]
    # policy-loss plug-in: uncertain tokens with a positive advantage get the wider upper clip
    from gcore_b200.loss.policy_loss import LossInput
    c = load_config(RlConfig, y("rl_custom_loss.yaml"), [])
    loss = import_from_path(os.path.join(ROOT, c.ppo.loss_func_py_path), c.ppo.loss_func_fn_name)
    lp = torch.tensor([-3.0, -0.5, -3.0], requires_grad=True)
    lo = loss(c.ppo, LossInput(lp, torch.tensor([-3.5, -0.9, -3.5]), None, None, torch.tensor([1.0, 1.0, -1.0]),
                               torch.ones(3), torch.zeros(3, dtype=torch.int32), 1))
    assert torch.allclose(lo.token_loss, torch.tensor([-1.4, -1.2, 1.6487]), atol=1e-4)
    assert lo.metrics["widened_clip_frac"].tolist() == [1.0, 3.0]
    gen = import_from_path(os.path.join(ROOT, "tasks", "math_rl", "gen_rm_reward.py"), "parse_verdict")
    prompt = import_from_path(os.path.join(ROOT, "tasks", "math_rl", "gen_rm_reward.py"), "build_grader_prompt")
    assert gen("Verdict: wrong. On reflection, Verdict: Correct") == 1.0 and gen("unsure") == 0.0
    assert "Reference answer: 42" in prompt({"prompt_text": "6 x 7?", "response_text": "42", "answer": "42"})


def test_preference_recipes_load():
    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import DpoConfig, RewardTrainConfig
    y = lambda n: os.path.join(ROOT, "tasks", "preference", "yaml", n)
    d = load_config(DpoConfig, y("dpo_qwen2.5_7b.yaml"), [])
    assert d.dpo_beta == 0.1 and d.dpo_sft_loss_coef == 0.05 and not d.reference_free
    r = load_config(DpoConfig, y("dpo_reference_free_lora.yaml"), [])
    assert r.reference_free and r.policy.lora.rank == 32 and r.policy.model_arch == d.policy.model_arch
    m = load_config(RewardTrainConfig, y("reward_model_bt.yaml"), [])
    assert m.rm_loss == "bt" and m.policy.without_ref


def test_recipe_includes_merge_in_order_and_reject_cycles(tmp_path):
    from gcore_b200.configs.base import ConfigError, load_yaml
    (tmp_path / "a.yaml").write_text("x: {p: 1, q: 2}\ny: 1\n")
    (tmp_path / "b.yaml").write_text("base: a.yaml\nx: {q: 3}\nz: 5\n")
    (tmp_path / "c.yaml").write_text("base: [a.yaml, b.yaml]\ny: 9\n")
    assert load_yaml(str(tmp_path / "b.yaml")) == {"x": {"p": 1, "q": 3}, "y": 1, "z": 5}
    assert load_yaml(str(tmp_path / "c.yaml")) == {"x": {"p": 1, "q": 3}, "y": 9, "z": 5}
    (tmp_path / "d.yaml").write_text("base: e.yaml\n")
    (tmp_path / "e.yaml").write_text("base: d.yaml\n")
    with pytest.raises(ConfigError):
        load_yaml(str(tmp_path / "d.yaml"))


def test_image_generation_and_vision_language_recipes_load():
    import glob
    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import FinetuneConfig, T2iConfig
    from gcore_b200.models.dit import DiTConfig
    files = sorted(glob.glob(os.path.join(ROOT, "tasks", "t2i", "yaml", "*.yaml")))
    assert len(files) >= 4
    for f in files:
        cfg = load_config(T2iConfig, f, [])
        assert cfg.model.pipeline in ("flux", "qwen_image_edit", "flux_kontext", "bagel")
        if cfg.model.transformer:
            DiTConfig(**cfg.model.transformer)          # rotary axes sum to the head size, etc.
    cfg = load_config(FinetuneConfig, os.path.join(ROOT, "tasks", "vlm_sft", "yaml", "sft_vlm_images.yaml"), [])
    assert cfg.policy.vision_config["patch_size"] == 14 and cfg.data.py_path.endswith("dataset.py")


def test_reference_spellings_of_ppo_fields_are_accepted():
    from gcore_b200.configs.base import ConfigError, from_dict
    from gcore_b200.configs.config import PpoConfig
    c = from_dict(PpoConfig, {"ppo_entropy_regularization_type": "kl-cov", "ppo_kl_cov_ratio": 0.01,
                              "off_policy_correction_mode": "icepop", "off_policy_correction_upper_bound": 3.0,
                              "custom_advantage_py_path": "/x/adv.py", "custom_advantage_py_name": "fn",
                              "vespo_c1_neg": 2.0})
    assert c.entropy_regularization_type == "kl-cov" and c.kl_cov_ratio == 0.01 and c.offpolicy_correction == "icepop"
    assert c.offpolicy_correction_upper == 3.0 and c.advantage_py_path == "/x/adv.py" and c.advantage_fn_name == "fn"
    assert c.vespo_c1_neg == 2.0
    import pytest
    with pytest.raises(ConfigError):
        from_dict(PpoConfig, {"ppo_kl_cov_ratio": 0.01, "kl_cov_ratio": 0.02})


def test_dpo_config_options_and_alias():
    import pytest
    from gcore_b200.configs.base import ConfigError, from_dict
    from gcore_b200.configs.config import DpoConfig
    c = from_dict(DpoConfig, {"dpo_beta": 0.2, "dpo_ftx_gamma": 0.3})
    assert c.dpo_beta == 0.2 and c.dpo_sft_loss_coef == 0.3 and c.dpo_loss_type == "sigmoid"
    with pytest.raises(ConfigError):
        from_dict(DpoConfig, {"dpo_loss_type": "ipo"})
