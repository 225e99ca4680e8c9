"""Disaggregated placement on CPU (gloo): trainer ranks and rollout ranks as separate processes; weights travel as a
bucket broadcast, prompts and samples as objects; after the run the rollout ranks hold the trainer's weights."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(tmp_path, world, n_train, train_tp, sampler_tp, port):
    out = tmp_path / "disagg.json"
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT=port, OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "workers", "disagg_worker.py"), str(out),
                               str(n_train), str(train_tp), str(sampler_tp)],
                              env=dict(env, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r)))
             for r in range(world)]
    for p in procs:
        assert p.wait(timeout=240) == 0
    return json.load(open(out))


def test_two_trainers_one_rollout_rank(tmp_path):
    res = _run(tmp_path, 3, 2, 1, 1, "29581")
    train = [r for r in res if r["role"] == "train"]
    samp = [r for r in res if r["role"] == "sampler"]
    assert len(train) == 2 and len(samp) == 1
    # 4 prompts x 4 samples per trainer rank were generated remotely, both steps; the update ran
    assert all(t > 0 for r in train for t in r["tokens"]) and all(g > 0 for r in train for g in r["grad_norm"])
    assert train[0]["transfer"]["buckets"] > 1
    # initial hand-over + one per step
    assert samp[0]["stats"] == {"weight_updates": 3, "generate_calls": 2}
    # data-parallel trainers hold the same weights, and the rollout rank holds exactly those
    assert train[0]["digest"] == train[1]["digest"]
    for name, dg in samp[0]["digest"].items():
        assert train[0]["digest"][name] == dg, name


def test_tensor_parallel_trainer_to_tensor_parallel_rollout(tmp_path):
    """TP2 trainer -> TP2 rollout engine: tensors are made whole on the trainer side and re-cut on the rollout side;
    every rollout rank ends with the shard the trainer rank of the same tensor-parallel index holds."""
    res = _run(tmp_path, 4, 2, 2, 2, "29583")
    train = {r["tp_rank"]: r for r in res if r["role"] == "train"}
    samp = {r["tp_rank"]: r for r in res if r["role"] == "sampler"}
    assert set(train) == set(samp) == {0, 1}
    for tpr in (0, 1):
        for name, dg in samp[tpr]["digest"].items():
            assert train[tpr]["digest"][name] == dg, (tpr, name)
    assert samp[0]["stats"]["generate_calls"] == 2


def test_grpo_entry_point_runs_disaggregated(tmp_path):
    """``placement_type: disaggregated`` through the ordinary entry point: one trainer rank, one rollout rank."""
    import yaml
    cfg = {"placement_type": "disaggregated", "disaggregated_train_gpus": 1,
           "training": {"rollout_gbs": 4, "sampling_repeat_n": 2, "train_gbs": 8, "train_mbs": 4, "total_ppo_step": 2,
                        "seed": 3},
           "policy": {"model_arch": "tiny_llama", "model_config": {"dtype": "float32"}, "recompute": "none"},
           "optimizer": {"lr": 1e-3, "lr_decay_style": "constant", "weight_decay": 0.0},
           "sampler": {"infer_engine_configs": [{"generate_max_tokens": 8, "max_model_len": 40, "kv_block_size": 4,
                                                  "disable_cuda_graph": True}]},
           "data": {"max_prompt_length": 16, "synthetic": {"num_samples": 32, "prompt_len": 8, "lo": 3, "hi": 1000}},
           "report": {"log_dir": str(tmp_path / "logs")}}
    y = tmp_path / "rl.yaml"
    y.write_text(yaml.safe_dump(cfg))
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29585", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, "-m", "gcore_b200.entry.train_lm_grpo", "--config", str(y)],
                              env=dict(env, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r)), cwd=ROOT)
             for r in range(2)]
    for p in procs:
        assert p.wait(timeout=240) == 0
