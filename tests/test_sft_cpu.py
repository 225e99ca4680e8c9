"""BASELINE config 1: tiny Llama SFT in fp32 on CPU, single process vs gloo world_size=2 (DP=2)."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_samples(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        t = torch.randint(3, 1024, (512,), generator=g)
        m = torch.zeros(512)
        m[255:511] = 1.0  # loss on the second 256 tokens (log-prob axis)
        out.append({"tokens": t, "loss_mask": m})
    return out


def build_engine(lr=1e-4):
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import get_preset
    pc = PolicyConfig(recompute="none", without_ref=True)
    oc = OptimizerConfig(lr=lr, lr_decay_style="constant", weight_decay=0.0, max_grad_norm=0.0)
    tc = TrainingConfig(train_mbs=4, train_gbs=8)
    eng = TrainingEngine(pc, oc, tc, model_cfg=get_preset("tiny_llama", dtype="float32"))
    eng.setup_model_and_get_optimizer(seed=7)
    return eng


def run_steps(eng, rank, world, steps=20, fixed=False):
    losses = []
    for s in range(steps):
        batch = make_samples(8, seed=100 if fixed else 100 + s)
        mine = batch[rank::world]
        losses.append(eng.finetune_step(mine)["lm_loss"])
    return losses


def test_single_process_loss_decreases():
    torch.manual_seed(0)
    eng = build_engine(lr=1e-3)
    losses = run_steps(eng, 0, 1, steps=8, fixed=True)
    assert losses[0] > 6.5  # ~ln(1024)
    assert losses[-1] < losses[0] - 0.5


def test_world2_gloo_matches_single_process(tmp_path):
    out = tmp_path / "res"
    out.mkdir()
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29533", OMP_NUM_THREADS="2")
    procs = []
    for r in range(2):
        e = dict(env, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r))
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "workers", "sft_worker.py"),
                                       str(out)], env=e))
    for p in procs:
        assert p.wait(timeout=900) == 0
    ref = run_steps(build_engine(), 0, 1, steps=20)
    got = torch.load(out / "losses_0.pt")
    assert len(got) == 20
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-4, (ref, got)
    # the reloaded checkpoint reproduces the parameters bit for bit
    assert torch.load(out / "reload_ok_0.pt") is True


def test_async_checkpoint_save_snapshots_the_step_and_publishes_later(tmp_path):
    """An asynchronous save copies the tensors before returning (training continues and changes the weights), the
    checkpoint appears under ``latest`` only once it is complete, and it holds the weights of its own step."""
    import sys
    import os
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "workers"))
    import parallel_worker as pw
    from gcore_b200.checkpoint import torch_dist as td
    from gcore_b200.models.config import get_preset
    mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
    e = pw.engine(mcfg, 1)
    e.finetune_step(pw.samples(8, 1))
    at_save = [p.detach().clone() for p in e.model.parameters()]
    root = str(tmp_path / "ck")
    td.save_checkpoint(e, root, 1, async_save=True)
    assert td.read_latest_step(root) is None and len(td._PENDING) == 1     # not published yet
    e.finetune_step(pw.samples(8, 2))                                      # weights move on while the file is written
    td.save_checkpoint(e, root, 2, async_save=True)                        # publishes step 1, starts step 2
    assert td.read_latest_step(root) == 1
    td.wait_for_async_save()
    assert td.read_latest_step(root) == 2 and not td._PENDING
    assert not [f for f in os.listdir(os.path.join(root, "iter_0000001")) if f.startswith(".part_")]
    e2 = pw.engine(mcfg, 1)
    e2.setup_model_and_get_optimizer(seed=3)
    assert td.load_checkpoint(e2, root, step=1) == 1
    for a, b in zip(at_save, e2.model.parameters()):
        assert torch.equal(a, b)
    assert td.load_checkpoint(e2, root) == 2
    for a, b in zip(e.model.parameters(), e2.model.parameters()):
        assert torch.equal(a, b)


def test_checkpoint_stage_converters(tmp_path):
    """hf <-> torch_dist round trip, policy -> critic (decoder copied, value head new, no vocabulary projection) and
    strip (weights only) with the conversion tool."""
    import json
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "workers"))
    import parallel_worker as pw
    from gcore_b200.checkpoint.torch_dist import CheckpointReader, save_checkpoint
    from gcore_b200.models.config import get_preset
    from gcore_b200.tools import ckpt_convert as cc
    mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
    cfg_json = tmp_path / "model.json"
    cfg_json.write_text(json.dumps(mcfg.to_dict()))
    e = pw.engine(mcfg, 1)
    e.finetune_step(pw.samples(8, 1))
    save_checkpoint(e, str(tmp_path / "rl"), 7, extra_state={"consumed_batches": 7})
    cc.main(["strip", "--model", str(cfg_json), "--src", str(tmp_path / "rl"), "--dst", str(tmp_path / "pol"),
             "--dtype", "float32"])
    keys = set(CheckpointReader(str(tmp_path / "pol" / "iter_0000000")).keys())
    assert not any(k.startswith("optimizer.") for k in keys) and "output_layer.weight" in keys
    cc.main(["policy2critic", "--model", str(cfg_json), "--src", str(tmp_path / "pol"), "--dst", str(tmp_path / "crit"),
             "--dtype", "float32"])
    rd = CheckpointReader(str(tmp_path / "crit" / "iter_0000000"))
    assert tuple(rd.full_tensor("output_layer.weight").shape) == (1, mcfg.hidden_size)
    src = CheckpointReader(str(tmp_path / "pol" / "iter_0000000"))
    k = "decoder.layers.mlp.linear_fc2.weight"
    assert torch.equal(rd.full_tensor(k), src.full_tensor(k))
    cc.main(["mcore2hf", "--model", str(cfg_json), "--src", str(tmp_path / "pol"), "--dst", str(tmp_path / "hf"),
             "--dtype", "float32"])
    cc.main(["hf2mcore", "--model", str(cfg_json), "--src", str(tmp_path / "hf"), "--dst", str(tmp_path / "back"),
             "--dtype", "float32"])
    back = CheckpointReader(str(tmp_path / "back" / "iter_0000000"))
    for key in ("embedding.word_embeddings.weight", "decoder.layers.self_attention.linear_qkv.weight", k):
        assert torch.equal(back.full_tensor(key), src.full_tensor(key)), key


def test_square_averaging_cross_entropy_weights_and_gradient():
    """``training.loss_func: square_averaging_cross_entropy``: the gradient equals that of
    sum_i sum_t nll_it / sqrt(N_i) / sum_i sqrt(N_i), whatever the micro-batching."""
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.loss import policy_loss as PL
    from gcore_b200.models.config import get_preset
    mask = torch.tensor([1.0, 1, 1, 1, 0, 1, 0, 0])
    seq = torch.tensor([0, 0, 0, 0, 0, 1, 1, 2], dtype=torch.int32)
    w = PL.square_averaging_weights(mask, seq, 3, denom=3.0)          # sqrt(4) + sqrt(1) = 3
    assert torch.allclose(w, torch.tensor([1 / 6, 1 / 6, 1 / 6, 1 / 6, 0, 1 / 3, 0, 0]))
    g = torch.Generator().manual_seed(0)
    samples = []
    for n_ans in (4, 64, 16, 1):
        t = torch.randint(3, 1024, (80,), generator=g)
        m = torch.zeros(80)
        m[10:10 + n_ans] = 1.0
        samples.append({"tokens": t, "loss_mask": m})
    grads = []
    for mbs in (4, 1):
        pc = PolicyConfig(recompute="none", without_ref=True)
        oc = OptimizerConfig(lr=0.0, lr_decay_style="constant", weight_decay=0.0, max_grad_norm=0.0)
        tc = TrainingConfig(train_mbs=mbs, train_gbs=4, loss_func="square_averaging_cross_entropy")
        eng = TrainingEngine(pc, oc, tc, model_cfg=get_preset("tiny_llama", dtype="float32"))
        eng.setup_model_and_get_optimizer(seed=7)
        eng.finetune_step([dict(s) for s in samples])
        grads.append(dict((n, p.main_grad.clone()) for n, p in eng.model.named_parameters()))
        model = eng.model
    name = "decoder.layers.0.mlp.linear_fc1.weight"
    assert torch.allclose(grads[0][name], grads[1][name], atol=1e-6)
    # direct definition on the same (unchanged, lr = 0) model
    eng.ddp.zero_grad_buffer()      # autograd hooks route every gradient into the fp32 main_grad buffers
    total, norm = 0.0, sum(float(s["loss_mask"].sum()) ** 0.5 for s in samples)
    for s in samples:
        n = s["tokens"].numel()
        h, _ = model(s["tokens"], torch.arange(n, dtype=torch.int32), torch.tensor([0, n], dtype=torch.int32), n)
        lp = torch.log_softmax(model.logits(h).float(), -1)[:-1].gather(-1, s["tokens"][1:, None]).squeeze(-1)
        m = s["loss_mask"][:-1]
        total = total - (lp * m).sum() / m.sum().sqrt() / norm
    total.backward()
    ref = dict(model.named_parameters())[name].main_grad
    assert torch.allclose(grads[0][name], ref, atol=2e-5), float((grads[0][name] - ref).abs().max())
