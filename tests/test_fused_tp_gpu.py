"""Fused tensor-parallel GEMM + collective kernels on >= 2 GPUs (peer stores + flags), checked against NCCL."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_ag_gemm_and_gemm_rs_two_ranks(tmp_path):
    out = tmp_path / "fused.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29571", os.path.join(ROOT, "tests", "workers", "fused_tp_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    for k, v in res.items():
        for name, ok in v.items():
            if isinstance(ok, bool):
                assert ok, (k, name, res)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_zero1_peer_memory_step_matches_nccl_path(tmp_path):
    out = tmp_path / "zero1.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29573", os.path.join(ROOT, "tests", "workers", "zero1_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    for k, v in res.items():
        for name, ok in v.items():
            if isinstance(ok, bool):
                assert ok, (k, name, res)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_ep_dispatch_combine_matches_nccl_path(tmp_path):
    out = tmp_path / "ep.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29575", os.path.join(ROOT, "tests", "workers", "fused_ep_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    for k, v in res.items():
        for name, ok in v.items():
            if isinstance(ok, bool):
                assert ok, (k, name, res)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_context_parallel_attention_over_peer_memory(tmp_path):
    out = tmp_path / "cp.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29577", os.path.join(ROOT, "tests", "workers", "cp_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    for k, v in res.items():
        for name, ok in v.items():
            if isinstance(ok, bool):
                assert ok, (k, name, res)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_weight_resync_over_peer_memory_tp2_to_tp1(tmp_path):
    out = tmp_path / "ws.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29579", os.path.join(ROOT, "tests", "workers", "weight_sync_worker.py"),
           str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    for k, v in res.items():
        for name, ok in v.items():
            if isinstance(ok, bool):
                assert ok, (k, name, res)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["pp", "vpp"])
def test_pipeline_stages_over_nccl_p2p(tmp_path, mode):
    """1F1B and interleaved 1F1B with activations and gradients on NCCL send / recv (two communicators): losses and
    log-probs equal the single-GPU run, and the two-stage checkpoint resumes."""
    sys.path.insert(0, os.path.join(ROOT, "tests", "workers"))
    import parallel_worker as pw
    from gcore_b200.models.config import get_preset
    out = tmp_path / "pp.json"
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29591", GCORE_TEST_BACKEND="nccl",
               NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "workers", "parallel_worker.py"), mode,
                               str(out), str(tmp_path)], env=dict(env, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r)))
             for r in range(2)]
    for p in procs:
        assert p.wait(timeout=150) == 0
    got = json.load(open(out))
    mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True, num_layers=4)
    e = pw.engine(mcfg, 1)
    ref, norms = [], []
    for s in range(4):
        ref.append(e.finetune_step(pw.samples(8, 130 + s))["lm_loss"])
        norms.append(float(e.optimizer.last_grad_norm))
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 2e-3, (ref, got["losses"], norms, got["grad_norms"])
    lp = e.compute_log_probs(pw.samples(3, 199))
    for a, b in zip(lp, got["logprobs"]):
        assert torch.allclose(a["logprobs"].cpu(), torch.tensor(b), atol=2e-3)
    assert abs(got["next_loss"][0] - got["next_loss"][1]) < 1e-4, got["next_loss"]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_grpo_steps_with_experts_split_over_two_gpus(tmp_path):
    """Two GRPO steps of a small MoE policy in bf16 with the experts split over both GPUs, in the trainer (peer-memory
    dispatch / combine) and in the colocated rollout engines (lockstep passes, different stop tokens per rank)."""
    out = tmp_path / "ep_grpo.json"
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29593", GCORE_TEST_BACKEND="nccl",
               NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "workers", "parallel_worker.py"), "ep_grpo",
                               str(out)], env=dict(env, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r)))
             for r in range(2)]
    for p in procs:
        assert p.wait(timeout=150) == 0
    got = json.load(open(out))["ranks"]
    for r in got:
        assert r["dtype"] == "bfloat16"
        assert all(g > 0 for g in r["grad_norm"]) and all(abs(x - 1.0) < 2e-2 for x in r["ratio"]), got
        assert r["logprob_gap"] < 0.15, got
