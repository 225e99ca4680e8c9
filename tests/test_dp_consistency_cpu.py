"""Properties that must not depend on how a batch is spread over data-parallel ranks or packed into micro-batches
(gloo, world 2): equal micro-batch counts under expert parallelism with a token budget, the weight of the MoE
auxiliary loss, the gradient norm without a sharded optimizer, and top-k / top-p / min-p sampling with a
vocabulary-sharded head."""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "workers"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

from test_parallel_cpu import _spawn  # noqa: E402


def test_ep_ranks_run_equal_microbatch_counts_under_a_token_budget(tmp_path):
    out = tmp_path / "dyn.json"
    _spawn("ep_dynmbs", out, port="29571")
    got = json.load(open(out))
    for step in range(2):
        assert got["counts"][0][step] == got["counts"][1][step] > 1, got["counts"]
    assert all(l == l and l > 0 for l in got["losses"])
    assert got["n_logprobs"] == 3


def test_moe_aux_loss_weight_is_independent_of_dp_and_microbatching(tmp_path):
    import parallel_worker as pw
    out = tmp_path / "aux.json"
    _spawn("aux_dp", out, port="29563")
    got = json.load(open(out))
    e = pw.engine(pw.MOE_CFG, 1)
    batch = pw.samples(8, 190, vocab=512)
    for b in batch:
        b["loss_mask"] = torch.zeros_like(b["loss_mask"])
    ref = e.finetune_step(batch)["grad_norm"]   # one rank, the same four micro-batches of two samples
    assert ref > 0
    assert abs(ref - got["grad_norm"]) < 1e-5 * max(ref, 1.0) + 1e-7, (ref, got)


def test_grad_norm_without_sharded_optimizer_counts_each_bucket_once(tmp_path):
    out = tmp_path / "norm.json"
    _spawn("nodistopt", out, port="29565")
    a, b = json.load(open(out))["norms"]
    assert abs(a - b) < 1e-4 * max(a, 1.0), (a, b)


def test_tp2_filtered_sampling_equals_single_rank(tmp_path):
    from gcore_b200.models.config import get_preset
    from gcore_b200.models.gpt import GPTModel
    from gcore_b200.rollout.engine import InferEngine, RolloutWeights, SamplingParams
    out = tmp_path / "topk.json"
    _spawn("tp_topk", out, port="29567")
    got = json.load(open(out))
    mcfg = get_preset("tiny_llama", dtype="float32", qkv_bias=True)
    model = GPTModel(mcfg, recompute="none")
    model.reset_parameters(21)
    model.eval()
    eng = InferEngine(mcfg, RolloutWeights.from_model(model), max_running_requests=4, max_model_len=48,
                      kv_block_size=4, sync_interval=2, use_cuda_graph=False)
    for name, kw in (("top_k", dict(top_k=3)), ("top_p", dict(top_p=0.3)), ("min_p", dict(min_p=0.2))):
        reqs = eng.generate(got["prompts"], SamplingParams(max_new_tokens=6, temperature=1.5, seed=5, **kw), n=2)
        assert [r.out_tokens for r in reqs] == got["out"][name]["tokens"], name
        for a, b in zip(reqs, got["out"][name]["logprobs"]):
            assert max(abs(x - y) for x, y in zip(a.out_logprobs, b)) < 1e-4, name


def test_dynamic_context_parallel_step_equals_single_process(tmp_path):
    import parallel_worker as pw
    from gcore_b200.models.config import get_preset
    out = tmp_path / "dcp.json"
    _spawn("dyncp", out, port="29569")
    got = json.load(open(out))
    e = pw.engine(get_preset("tiny_llama", dtype="float32", qkv_bias=True), 1)
    ref = [e.finetune_step(pw.samples(8, 210 + s, L=72))["lm_loss"] for s in range(3)]
    for a, b in zip(ref, got["losses"]):
        assert abs(a - b) < 5e-4, (ref, got["losses"])
    assert abs(float(e.optimizer.last_grad_norm) - got["grad_norm"]) < 5e-3
    full = e.compute_log_probs(pw.samples(6, 219, L=72))
    for r in range(2):
        for mine, theirs in zip(full[r::2], got["logprobs"][r]):
            assert torch.allclose(mine["logprobs"], torch.tensor(theirs), atol=2e-4)


def test_grpo_update_runs_on_balanced_token_counts(tmp_path):
    out = tmp_path / "bal.json"
    _spawn("dp_grpo_balance", out, port="29573")
    r0, r1 = json.load(open(out))["ranks"]
    assert abs(r0["before"] - r1["before"]) > abs(r0["after"] - r1["after"]), (r0, r1)
    assert r0["before"] + r1["before"] == r0["after"] + r1["after"]
    assert r0["grad_norm"] == r1["grad_norm"] and r0["grad_norm"] > 0


def test_training_continues_after_process_groups_are_offloaded_and_reloaded(tmp_path):
    import parallel_worker as pw
    from gcore_b200.models.config import get_preset
    out = tmp_path / "pg.json"
    _spawn("pg_offload", out, port="29575")
    got = json.load(open(out))["losses"]
    e = pw.engine(get_preset("tiny_llama", dtype="float32", qkv_bias=True), 1)
    ref = [e.finetune_step(pw.samples(8, 230 + s))["lm_loss"] for s in range(3)]
    for a, b in zip(ref, got):
        assert abs(a - b) < 5e-4, (ref, got)
