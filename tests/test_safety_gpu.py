"""Safety nets that stand in for a sanitizer: a device wait whose peer never shows up runs out and reports through
the error word (the context stays usable), kernels declared deterministic give bit-identical results twice, and
kernels do not write outside their output (canary-padded buffers)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def test_peer_wait_runs_out_and_reports_instead_of_hanging():
    from gcore_b200.ops import _lib
    from gcore_b200.ops.gemm import gemm
    lib = _lib.kernels()
    dev = torch.device("cuda", torch.cuda.current_device())
    # a "group" of two ranks whose second member does not exist: both flag arrays are local, nobody answers
    flags = torch.zeros(2, 64 * 8, dtype=torch.int32, device=dev)
    ptrs = torch.tensor([flags[0].data_ptr(), flags[1].data_ptr()], dtype=torch.int64, device=dev)
    err = _lib.err_flag(dev)
    err.zero_()
    lib.gk_set_peer_wait_budget(200_000_000)  # ~0.1 s
    try:
        rc = lib.gk_peer_barrier(_lib.ptr(ptrs), 0, 2, 0, 1, _lib.ptr(err), _lib.stream_ptr())
        assert rc == 0
        torch.cuda.synchronize()
        assert int(err.item()) == 6  # the wait gave up and said so
        with pytest.raises(RuntimeError, match="timed-out wait"):
            _lib.check_device_errors()
    finally:
        lib.gk_set_peer_wait_budget(0)
    assert int(err.item()) == 0  # check_device_errors cleared the word
    # the published flag reached the "peer" and the context still computes
    assert int(flags[1][0]) == 1
    a, b = _rand(128, 256), _rand(192, 256)
    assert torch.allclose(gemm(a, b).float(), a.float() @ b.float().t(), rtol=2e-2, atol=2e-2)


def test_deterministic_kernels_are_bitwise_repeatable():
    from gcore_b200.ops.attention import flash_attn_varlen
    from gcore_b200.ops.gemm import gemm, linear_forward
    torch.manual_seed(0)
    # split-K decode GEMM (semaphore / cluster reduction), attention forward + backward (no atomics)
    x, w = _rand(64, 3584, scale=0.5), _rand(4608, 3584, scale=0.05)
    assert torch.equal(linear_forward(x, w), linear_forward(x, w))
    a, b = _rand(1000, 512), _rand(777, 512, scale=0.05)
    assert torch.equal(gemm(a, b), gemm(a, b))
    cu = torch.tensor([0, 300, 301, 900, 1024], dtype=torch.int32, device="cuda")
    outs = []
    for _ in range(2):
        torch.manual_seed(1)
        qq, kk, vv = (torch.randn(1024, h, 128, device="cuda").mul(0.5).bfloat16().requires_grad_(True)
                      for h in (8, 2, 2))
        o = flash_attn_varlen(qq, kk, vv, cu, cu, 600, 600, causal=True)
        o.backward(torch.ones_like(o))
        outs.append((o.detach().clone(), qq.grad.clone(), kk.grad.clone(), vv.grad.clone()))
    for t0, t1 in zip(*outs):
        assert torch.equal(t0, t1)


@pytest.mark.parametrize("M,N,K", [(130, 70, 96), (1, 257, 64), (257, 8, 40)])
def test_gemm_writes_only_its_output(M, N, K):
    from gcore_b200.ops.gemm import gemm
    torch.manual_seed(2)
    a, b = _rand(M, K), _rand(N, K, scale=0.1)
    pad = 64
    buf = torch.full((M + 2 * pad, N + 2 * 8), 1234.0, dtype=torch.bfloat16, device="cuda")
    out = buf[pad:pad + M, 8:8 + N]
    assert out.data_ptr() % 16 == 0
    gemm(a, b, out=out)
    assert torch.allclose(out.float(), a.float() @ b.float().t(), rtol=2e-2, atol=2e-2)
    canary = buf.clone()
    canary[pad:pad + M, 8:8 + N] = 1234.0
    assert bool((canary == 1234.0).all()), "a store landed outside the output view"


def test_rmsnorm_and_swiglu_write_only_their_output():
    from gcore_b200.ops import fused
    x = _rand(37, 512)
    g = torch.ones(512, device="cuda").bfloat16()
    y, _ = fused.rmsnorm(x, g, 1e-6)
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2)
    gu = _rand(37, 2 * 256)
    s = fused.swiglu(gu)
    assert s.shape == (37, 256)
    assert torch.allclose(s.float(), torch.nn.functional.silu(gu[:, :256].float()) * gu[:, 256:].float(), rtol=2e-2,
                          atol=2e-2)


def _parity_model(kind, dtype):
    from gcore_b200.models.config import ModelConfig, get_preset
    if kind == "dense":
        return get_preset("tiny_llama", dtype=dtype, qkv_bias=True, num_layers=4)
    if kind == "moe":
        return ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=256, num_attention_heads=2, num_kv_heads=1,
                           head_dim=128, ffn_hidden_size=512, vocab_size=1024, num_experts=8, moe_top_k=2,
                           moe_ffn_hidden_size=128, moe_aux_loss_coef=1e-2, dtype=dtype, qk_layernorm=True)
    return ModelConfig(arch="deepseek_v3", num_layers=2, hidden_size=256, num_attention_heads=4, num_kv_heads=4,
                       ffn_hidden_size=512, vocab_size=1024, use_mla=True, q_lora_rank=128, kv_lora_rank=128,
                       qk_nope_head_dim=64, qk_rope_head_dim=32, v_head_dim=64, head_dim=96, num_experts=8,
                       moe_top_k=2, moe_ffn_hidden_size=128, moe_shared_expert_ffn=128,
                       moe_router_type="sigmoid_group", moe_n_group=4, moe_topk_group=2, first_k_dense=1,
                       moe_routed_scaling_factor=2.5, moe_router_bias=True, rope_interleaved=True, dtype=dtype)


@pytest.mark.parametrize("kind,dtype,tol", [("dense", "float32", 1e-3), ("dense", "bfloat16", 3e-3),
                                            ("moe", "bfloat16", 5e-3), ("mla_moe", "bfloat16", 5e-3)])
def test_training_steps_match_the_eager_backend(kind, dtype, tol, monkeypatch):
    """Four optimisation steps of a small decoder through the engine: native kernels against the PyTorch definitions
    of the same ops (losses and gradient norms).  fp32 models included: the fused Adam kernel only writes bf16
    parameters, other dtypes are refreshed from the master weights."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "workers"))
    import parallel_worker as pw

    def run(eager):
        monkeypatch.setenv("GCORE_B200_FORCE_EAGER", "1" if eager else "0")
        e = pw.engine(_parity_model(kind, dtype), 1)
        out = []
        for s in range(4):
            loss = e.finetune_step(pw.samples(8, 130 + s))["lm_loss"]
            out.append((float(loss), float(e.optimizer.last_grad_norm)))
        return out

    native, eager = run(False), run(True)
    for (l0, n0), (l1, n1) in zip(native, eager):
        assert abs(l0 - l1) < tol and abs(n0 - n1) < 10 * tol * max(1.0, n1), (native, eager)


@pytest.mark.parametrize("flag", ["fp8", "fp8_qat", "fp4_qat"])
def test_low_precision_training_matches_the_eager_backend(flag, monkeypatch):
    """policy.fp8 (block-scaled e4m3 GEMM with on-the-fly activation quantisation) and the QAT modes through the
    engine on the GPU: native quantisers / fp8 GEMM against their PyTorch definitions."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "workers"))
    import parallel_worker as pw
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import get_preset
    mcfg = get_preset("tiny_llama", dtype="bfloat16", qkv_bias=True, ffn_hidden_size=512)

    def run(eager):
        monkeypatch.setenv("GCORE_B200_FORCE_EAGER", "1" if eager else "0")
        pc = PolicyConfig(recompute="none", without_ref=True, **{flag: True})
        e = TrainingEngine(pc, OptimizerConfig(lr=1e-3, lr_decay_style="constant", weight_decay=0.0, max_grad_norm=1.0),
                           TrainingConfig(train_mbs=2, train_gbs=8), model_cfg=mcfg)
        e.setup_model_and_get_optimizer(seed=11)
        assert len(e.lowp_modules) == 4 * mcfg.num_layers
        return [float(e.finetune_step(pw.samples(8, 50 + s))["lm_loss"]) for s in range(3)]

    native, eager = run(False), run(True)
    assert all(abs(a - b) < 8e-3 for a, b in zip(native, eager)), (native, eager)
