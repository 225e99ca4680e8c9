"""CPU tests of the algorithm-core and service modules: registry, Muon, feature store, adaptive entropy, filter
sampling, DP balancing (gloo, 2 ranks), agentic envs and trajectory masks, RPC clients, transfer queue."""
import os
import types

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_registry_resolves_eager_on_cpu_and_accepts_overrides():
    from gcore_b200.ops import registry
    assert "gemm" in registry.available() and "rmsnorm" in registry.available()
    fn = registry.resolve("rmsnorm")
    assert fn.__name__.endswith("_ref")
    registry.register_fn("rmsnorm", lambda *a, **k: "mine", "override")
    assert registry.resolve("rmsnorm")() == "mine"
    registry._REGISTRY["rmsnorm"].pop("override")
    with pytest.raises(KeyError):
        registry.resolve("no_such_op")


def test_newton_schulz_orthogonalises_and_muon_descends():
    from gcore_b200.core.muon import Muon, newton_schulz5
    torch.manual_seed(0)
    for shape in ((64, 128), (128, 48)):
        X = newton_schulz5(torch.randn(*shape)).float()
        sv = torch.linalg.svdvals(X)
        assert sv.min() > 0.4 and sv.max() < 1.6  # singular values pushed into the quintic's band around 1
    w = torch.nn.Parameter(torch.randn(32, 16))
    b = torch.nn.Parameter(torch.zeros(32))
    x, y = torch.randn(256, 16), torch.randn(256, 32)
    opt = Muon([w], [b], lr=0.1, wd=0.0)
    first = None
    for _ in range(40):
        loss = ((x @ w.t() + b - y) ** 2).mean()
        first = first if first is not None else loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert loss.item() < 0.8 * first


def test_feature_store_intervals_persistence_and_adaptive_entropy(tmp_path):
    from gcore_b200.core import ppo_feature_store as fs
    fs.reset_ppo_feature_store()
    st = fs.get_ppo_feature_store()
    st.configure("entropy", "mean")
    st.configure("peak", "max")
    with fs.ppo_step_interval(3) as iv:
        st.record_weighted_sum("entropy", 6.0, 4.0)
        st.record_weighted_sum("entropy", 2.0, 4.0)
        st.record_weighted_sum("peak", 5.0, 1.0)
        st.record_weighted_sum("peak", 9.0, 1.0)
    assert iv.results == {"entropy": 1.0, "peak": 9.0}
    assert st.get_history_mean("entropy") == 1.0 and st.list_pending_features() == []
    cfg = types.SimpleNamespace(use_adaptive_entropy=True, ppo_entropy_bonus=0.01, entropy_target=0.5,
                                entropy_coef_delta=0.005, entropy_coef_min=0.0, entropy_coef_max=0.02)
    assert fs.get_entropy_bonus_coef(cfg) == 0.0           # no measurement yet: entropy treated as high
    m = fs.update_adaptive_entropy(cfg, 0.3)               # below target -> coefficient rises, bonus switches on
    assert abs(m["policy/entropy_coef"] - 0.015) < 1e-9 and abs(fs.get_entropy_bonus_coef(cfg) - 0.015) < 1e-9
    fs.update_adaptive_entropy(cfg, 0.3)
    fs.update_adaptive_entropy(cfg, 0.3)
    assert abs(st.get(fs.ENTROPY_COEF_KEY) - 0.02) < 1e-9    # clamped at the maximum
    fs.update_adaptive_entropy(cfg, 0.9)                   # above target -> falls, and the bonus is gated off
    assert abs(st.get(fs.ENTROPY_COEF_KEY) - 0.015) < 1e-9 and fs.get_entropy_bonus_coef(cfg) == 0.0
    st.save_to_ckpt(str(tmp_path), 3)
    fs.reset_ppo_feature_store()
    st2 = fs.get_ppo_feature_store()
    assert st2.load_from_ckpt(str(tmp_path), 3) and abs(st2.get(fs.ENTROPY_COEF_KEY) - 0.015) < 1e-9
    with pytest.raises(ValueError):
        st2.load_from_ckpt(str(tmp_path), 4)


def test_filter_sampling_strategies():
    from gcore_b200.core import filter_samplings as F
    groups = [[{"rewards": torch.tensor([r])} for r in (0.1, 0.9, 0.5, 0.0)]]
    bw = F.get_group_filter("best-and-worst")(None, groups, 4, 2)
    assert [float(s["rewards"]) for s in bw[0]] == pytest.approx([0.9, 0.0])
    assert len(F.get_group_filter("test")(None, groups, 4, 3)[0]) == 3
    flat = [{"group_id": g, "reward": r, "sample_mask": m} for g, r, m in
            ((0, 1.0, 1), (0, 0.0, 1), (0, 0.5, 0), (1, 1.0, 1))]
    out = F.filter_rollout_samples(None, flat, ["sample-mask", "valid_group", "best-and-worst"])
    assert [(s["group_id"], s["reward"]) for s in out] == [(0, 0.0), (0, 1.0)]


def _balance_worker(rank, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    from gcore_b200.core.dp_balancing import rebalance_across_dp_ranks, restore_original_order
    g = dist.group.WORLD
    lens = [400, 390, 380, 370] if rank == 0 else [10, 10, 10, 10]
    samples = [{"tokens": torch.full((n,), rank * 100 + i), "uid": (rank, i)} for i, n in enumerate(lens)]
    mine, restore = rebalance_across_dp_ranks(samples, g)
    load = sum(len(s["tokens"]) for s in mine)
    for s in mine:
        s["logprobs"] = s["tokens"].float() * 2
    back = restore_original_order(mine, restore, g, keys=("logprobs", "uid"))
    ok = all(b["uid"] == (rank, i) and torch.equal(b["logprobs"], samples[i]["tokens"].float() * 2)
             for i, b in enumerate(back))
    q.put((rank, load, ok))
    dist.barrier()
    dist.destroy_process_group()


def test_dp_rebalance_evens_tokens_and_restores_order():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_balance_worker, args=(r, 29561, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    loads = [r[1] for r in res]
    assert all(r[2] for r in res)
    assert sum(loads) == 1580 and max(loads) - min(loads) <= 20, loads  # was 1540 vs 40 before balancing


def test_smart_pad_buckets_cut_padding():
    from gcore_b200.core.dp_balancing import padding_waste, smart_pad_buckets
    lens = [5, 100, 7, 90, 50, 49]
    naive = [[0, 1], [2, 3], [4, 5]]
    buckets, inv = smart_pad_buckets(lens, 2)
    assert padding_waste(lens, buckets) < padding_waste(lens, naive)
    flat = [i for b in buckets for i in b]
    assert [flat[inv[i]] for i in range(len(lens))] == list(range(len(lens)))


def test_envs_parsers_and_trajectory_mask():
    from gcore_b200.agentic import (FrozenLakeEnv, SokobanEnv, ToolReasonEnvWrapper, ToolRegistry, TrajEnvManager,
                                    make_env, parse_tool_calls, split_reasoning)
    env = FrozenLakeEnv(size=4)
    obs, info = env.reset(seed=3)
    assert obs.count("P") == 1 and obs.count("G") == 1 and "instructions" in info
    # a scripted shortest path exists (the generator guarantees one): BFS over the rendered board
    from collections import deque
    grid = env.map
    prev, dq = {(0, 0): None}, deque([(0, 0)])
    while dq:
        r, c = dq.popleft()
        for name, (dr, dc) in (("Left", (0, -1)), ("Down", (1, 0)), ("Right", (0, 1)), ("Up", (-1, 0))):
            n = (r + dr, c + dc)
            if 0 <= n[0] < 4 and 0 <= n[1] < 4 and grid[n[0]][n[1]] != "H" and n not in prev:
                prev[n] = ((r, c), name)
                dq.append(n)
    path, cur = [], (3, 3)
    while prev[cur] is not None:
        cur, name = prev[cur][0], prev[cur][1]
        path.append(name)
    reward = done = None
    for name in reversed(path):
        _, reward, done, _, info = env.step(f"thinking... <answer>{name}</answer>")
    assert done and reward == 1.0 and info["success"]
    assert env.step("gibberish")[4]["action_is_valid"] is False
    sk = SokobanEnv()
    board, _ = sk.reset(seed=5)
    assert board.count("P") + board.count("S") == 1 and sk.boxes != sk.targets
    assert split_reasoning("<think>plan</think> go") == ("plan", "go")
    text, calls = parse_tool_calls('x <tool_call>{"name": "add", "arguments": {"a": 1, "b": 2}}</tool_call>')
    assert calls[0].name == "add" and text == "x"
    tools = ToolRegistry()
    tools.register("add", lambda a, b: a + b)
    wrapped = ToolReasonEnvWrapper(make_env("simple"), tools)
    wrapped.reset()
    obs, r, done, _, info = wrapped.step('<tool_call>{"name": "add", "arguments": {"a": 1, "b": 2}}</tool_call>')
    assert '"result": 3' in obs and not done and info["tool_calls"] == 1

    class Tok:
        def encode(self, t):
            return [ord(c) % 250 + 3 for c in t]

        def decode(self, ids):
            return "<answer>1</answer>"

    m = TrajEnvManager(make_env("simple", max_steps=2), Tok(), lambda ctx: {"token_ids": [5, 6, 7],
                                                                            "logprobs": [-0.1, -0.2, -0.3]})
    s = m.run(seed=0)
    assert s["num_turns"] == 2 and s["reward"] == 1.0  # only the first answer "1" is right
    assert int(s["mask"].sum()) == 6                    # 2 assistant turns x 3 generated tokens
    pos = torch.nonzero(s["mask"]).flatten()
    assert all(int(s["tokens"][p + 1]) in (5, 6, 7) for p in pos)
    assert torch.allclose(s["rollout_log_probs"][pos[:3]], torch.tensor([-0.1, -0.2, -0.3]))


def test_rpc_clients_and_transfer_queue():
    from gcore_b200.client import HttpRpcClient, KvStore, KvStoreClient, LocalRpcClient, pick_endpoint_idx, serve
    from gcore_b200.transfer import TransferQueue, make_key
    assert [pick_endpoint_idx(r, 4, 2) for r in range(4)] == [0, 0, 1, 1]
    assert [pick_endpoint_idx(r, 2, 4, 1) for r in range(2)] == [1, 3]
    srv, url = serve(KvStore())
    try:
        c = KvStoreClient(HttpRpcClient([url]))
        c.put("w", torch.arange(4))
        assert torch.equal(c.get("w"), torch.arange(4)) and c.get("missing", 7) == 7
    finally:
        srv.shutdown()
    a, b = KvStore(), KvStore()
    a.put("k", 1), a.put("k2", 2)
    lc = LocalRpcClient([a, b], dp_rank=0, dp_size=2, load_aware=True)
    assert lc.pick() == 1  # the emptier endpoint wins
    tq = TransferQueue()
    tq.put_batch(3, range(4), [{"tokens": torch.ones(2) * i} for i in range(4)])
    tq.storage.put(make_key(3, 1), {"advantages": torch.zeros(2)})
    assert tq.ready(3, ["tokens", "advantages"]) == ["step3:1"]
    r0 = tq.get_batch(3, ["tokens"], 8, dp_rank=0, dp_size=2)
    r1 = tq.get_batch(3, ["tokens"], 8, dp_rank=1, dp_size=2)
    assert len(r0) + len(r1) == 4 and not set(x["_key"] for x in r0) & set(x["_key"] for x in r1)
    assert tq.get_batch(3, ["tokens"], 8, dp_rank=0, dp_size=1) == []  # everything was consumed once
    tq.clear_step(3)
    assert len(tq.storage) == 0


def test_async_rollout_controller_staleness_tail_and_dp_split():
    import time

    from gcore_b200.rollout_generator.async_rollout import RolloutController

    class Sampler:
        def __init__(self, delay):
            self.delay = delay

        def generate(self, prompts, params=None):
            time.sleep(self.delay)
            return [{"tokens": list(p) + [7, 8]} for p in prompts]

    def prompts():
        i = 0
        while True:
            yield [[i * 10 + j] for j in range(4)]
            i += 1

    def score(samples):
        for s in samples:
            s["rewards"] = float(len(s["tokens"]))
        return samples

    c = RolloutController(prompts(), [Sampler(0.002), Sampler(0.004)], score, repeat_n=3, groups_per_batch=4,
                          max_staleness=1)
    c.set_weight_version(0)
    b0 = c.collect(timeout_s=30)
    assert len(b0) == 12 and all(s["weight_version"] == 0 for s in b0)
    assert len({s["group_id"] for s in b0}) == 4 and all(s["prompt_length"] == 1 for s in b0)
    # two versions later the groups still queued from version 0 are too stale and must be dropped
    time.sleep(0.05)
    c.set_weight_version(2)
    b1 = c.collect(timeout_s=30)
    assert all(2 - s["weight_version"] <= 1 for s in b1) and c.stats["dropped_stale"] > 0
    parts = RolloutController.split_for_dp(b1, 2, 3)
    assert [len(p) for p in parts] == [6, 6]
    assert not {s["group_id"] for s in parts[0]} & {s["group_id"] for s in parts[1]}
    c.shutdown()
    # tail batching: a straggling sampler does not hold the batch back for ever
    c2 = RolloutController(prompts(), [Sampler(0.001), Sampler(1.5)], score, repeat_n=2, groups_per_batch=6,
                           max_staleness=0, max_inflight=6, tail_wait_s=0.2)
    t0 = time.time()
    b = c2.collect(timeout_s=30)
    assert 0 < len(b) < 12 and time.time() - t0 < 1.4 and c2.stats["tail_batches"] == 1
    c2.shutdown()


def test_dynamic_cp_schedule_invariants():
    from gcore_b200.parallel.dynamic_cp import cp_size_for, imbalance, schedule
    assert [cp_size_for(n, 1000, 8) for n in (10, 1000, 1001, 3500, 8000)] == [1, 1, 2, 4, 8]
    with pytest.raises(ValueError):
        cp_size_for(9000, 1000, 8)
    g = torch.Generator().manual_seed(0)
    lens = torch.exp(torch.randn(64, generator=g) * 1.2 + 6).clamp(16, 7000).long().tolist()
    plan = schedule(lens, 8, 1000)
    assert sorted(a.gid for a in plan) == list(range(64))
    for a in plan:
        assert a.block_start % a.cp_size == 0 and a.block_start + a.cp_size <= 8
        assert -(-lens[a.gid] // a.cp_size) <= 1000
    # per micro-step and rank the token budget holds
    load = {}
    for a in plan:
        for r in range(a.block_start, a.block_start + a.cp_size):
            load[(a.step, r)] = load.get((a.step, r), 0) + -(-lens[a.gid] // a.cp_size)
    assert max(load.values()) <= 1000
    assert imbalance(plan, lens, 8) < 1.35


def _dyncp_worker(rank, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=4)
    from gcore_b200.parallel import dynamic_cp as D
    g = dist.group.WORLD
    groups = D.build_block_groups(g)
    lens = {0: [900, 30], 1: [40, 2100], 2: [50], 3: [3900, 20, 10]}[rank]
    samples = [{"tokens": torch.full((n,), rank * 10 + i)} for i, n in enumerate(lens)]
    all_lens, offsets = D.gather_lengths(samples, g)
    plan = D.schedule(all_lens, 4, 1000)
    steps = D.reroute_samples(samples, plan, offsets, g)
    mine = [s for st in steps for s in st]
    ok_blocks = all(s["_block"][0] <= rank < s["_block"][0] + s["_block"][1] for s in mine)
    for s in mine:
        s["logprobs"] = s["tokens"].float() + 0.5
    back = D.reverse_reroute(mine, len(samples), g)
    ok_back = all(torch.equal(b["logprobs"], samples[i]["tokens"].float() + 0.5) for i, b in enumerate(back))
    q.put((rank, ok_blocks, ok_back, sorted(groups), len(mine)))
    dist.barrier()
    dist.destroy_process_group()


def test_dynamic_cp_reroute_round_trip():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_dyncp_worker, args=(r, 29563, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(4))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert all(r[1] and r[2] for r in res)
    assert res[0][3] == [(0, 2), (0, 4), (2, 2)]
    # the 3900-token sample needs all four ranks, the 2100-token one a block of four too (3 -> 4): everyone sees them
    assert all(r[4] >= 2 for r in res)


def test_task_recipes_load_and_small_packages(tmp_path):
    import glob

    from gcore_b200.configs.base import load_config
    from gcore_b200.configs.config import RlConfig
    from gcore_b200.custom import load_custom_module, register_custom_module
    from gcore_b200.evaluate import EvaluateRunner, pass_at_k
    from gcore_b200.gdebug import check_rollout_batches, find_risky_settings
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    yamls = sorted(glob.glob(os.path.join(root, "tasks", "math_rl", "yaml", "*.yaml")))
    assert len(yamls) >= 4
    for y in yamls:
        cfg = load_config(RlConfig, y)
        assert cfg.policy.model_arch
    cfg = load_config(RlConfig, os.path.join(root, "tasks", "math_rl", "yaml", "grpo_qwen2.5_7b.yaml"),
                      ["ppo.skip_prev_logps=true", "training.train_gbs=256"])
    assert any("skip_prev_logps" in r for r in find_risky_settings(cfg))
    # rule reward of the recipe
    import importlib.util
    spec = importlib.util.spec_from_file_location("math_reward_mod", os.path.join(root, "tasks", "math_rl", "reward.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    r = mod.math_reward([{"response_text": "thus \\boxed{ 42 }.", "answer": "42"},
                         {"response_text": "\\boxed{41}", "answer": "42"}, {"response_text": "no box", "answer": "1"}])
    assert r.tolist() == [1.0, 0.0, 0.0]
    # custom module registry
    p = tmp_path / "my_mod.py"
    p.write_text("VALUE = 7\n")
    os.environ.pop("GCORE_CUSTOM_MODULE_REGISTRY_PATH", None)
    register_custom_module("my_custom_mod", str(p))
    assert load_custom_module("my_custom_mod").VALUE == 7
    with pytest.raises(ValueError):
        register_custom_module("my_custom_mod", str(tmp_path / "other.py"))
    # evaluation
    assert pass_at_k(4, 0, 1) == 0.0 and pass_at_k(4, 4, 1) == 1.0 and abs(pass_at_k(4, 1, 2) - 0.5) < 1e-12
    gen = lambda prompts: [{"tokens": p + [1, 2], "prompt_length": len(p), "ok": (i % 2 == 0)}  # noqa: E731
                           for p in prompts for i in range(4)]
    ev = EvaluateRunner(gen, lambda ss: torch.tensor([1.0 if s["ok"] else 0.0 for s in ss]), n=4, ks=(1, 2))
    m = ev.run([[5, 6], [7]])
    assert m["eval/reward_mean"] == 0.5 and abs(m["eval/pass@1"] - 0.5) < 1e-9 and m["eval/pass@2"] > 0.8
    # sample format check
    good = {"tokens": torch.arange(6), "prompt_length": 2, "mask": torch.tensor([0, 1, 1, 1, 1, 0.0])}
    check_rollout_batches([good])
    with pytest.raises(AssertionError):
        check_rollout_batches([dict(good, mask=torch.tensor([1, 1, 1, 1, 1, 0.0]))])


def test_streaming_dataset_shards_shuffles_and_resumes(tmp_path):
    import json
    from gcore_b200.data.datasets import StreamingJsonlDataset
    paths = []
    for s in range(3):
        p = tmp_path / f"shard{s}.jsonl"
        p.write_text("\n".join(json.dumps({"id": s * 100 + i}) for i in range(17 + s)) + "\n")
        paths.append(str(p))
    total = 17 + 18 + 19
    # data-parallel ranks partition the records
    parts = [[r["id"] for r in StreamingJsonlDataset(paths, rank, 2)] for rank in range(2)]
    assert sorted(parts[0] + parts[1]) == sorted(s * 100 + i for s in range(3) for i in range(17 + s))
    assert abs(len(parts[0]) - len(parts[1])) <= 1 and len(parts[0]) + len(parts[1]) == total
    # the shuffle buffer permutes (seeded, repeatable) without losing records
    a = [r["id"] for r in StreamingJsonlDataset(paths, 0, 2, shuffle_buffer=8, seed=3)]
    b = [r["id"] for r in StreamingJsonlDataset(paths, 0, 2, shuffle_buffer=8, seed=3)]
    assert a == b and sorted(a) != a and len(a) in (total // 2, total - total // 2)
    # resume: a fresh dataset that loads the consumed count continues with exactly the rest of the stream
    ds = StreamingJsonlDataset(paths, 1, 2, shuffle_buffer=8, seed=3, transform=lambda r: r["id"])
    it = iter(ds)
    head = [next(it) for _ in range(10)]
    ds2 = StreamingJsonlDataset(paths, 1, 2, shuffle_buffer=8, seed=3, transform=lambda r: r["id"])
    ds2.load_state_dict(ds.state_dict())
    full = list(StreamingJsonlDataset(paths, 1, 2, shuffle_buffer=8, seed=3, transform=lambda r: r["id"]))
    assert head == full[:10] and list(ds2) == full[10:] and ds2.consumed == len(full)
    # loader workers split a rank's records between them
    dl = torch.utils.data.DataLoader(StreamingJsonlDataset(paths, 0, 1, transform=lambda r: r["id"]), batch_size=None,
                                     num_workers=2)
    assert sorted(int(x) for x in dl) == sorted(s * 100 + i for s in range(3) for i in range(17 + s))


def test_external_async_reward_streams_retries_and_falls_back():
    import threading
    import time
    from gcore_b200.reward.rewards import ExternalAsyncReward

    class Judge(ExternalAsyncReward):
        def __init__(self):
            super().__init__(max_workers=4, micro_batch=2, timeout_s=5.0, retries=1, fallback=-1.0)
            self.seen, self.lock, self.flaky = [], threading.Lock(), set()

        def score_one(self, s):
            with self.lock:
                self.seen.append(s["id"])
            time.sleep(0.02)
            if s["id"] == 3 and s["id"] not in self.flaky:   # fails once, succeeds on the retry
                self.flaky.add(3)
                raise RuntimeError("service hiccup")
            if s["id"] == 6:
                raise RuntimeError("always down")
            return float(s["id"]) * 0.5, {"latency": 0.02}

    j = Judge()
    first, second = [{"id": i} for i in range(4)], [{"id": i} for i in range(4, 8)]
    j.submit(first)            # scoring starts while the caller produces the next samples
    time.sleep(0.05)
    assert len(j.seen) > 0
    j.submit(second)
    r, per_tok, extra = j.collect()
    exp = [0.0, 0.5, 1.0, 1.5, 2.0, 2.5, -1.0, -1.0]   # ids 6 and 7 share the failing micro-batch: fallback for both
    assert r.tolist() == exp and per_tok is None
    assert j.stats["retries"] >= 1 and j.stats["failures"] == 1 and j.stats["requests"] == 4
    r2, _, _ = j([{"id": 1}, {"id": 2}])
    assert r2.tolist() == [0.5, 1.0]
    j.close()


def test_reward_redistribution_by_lcs_alignment():
    import random
    from gcore_b200.utils.reward_redist import (_lcs_python, lcs_match, redistribute_rewards,
                                                redistribute_rewards_batch)
    rng = random.Random(0)
    # native Myers alignment = quadratic oracle (same LCS length, valid strictly increasing matches)
    for trial in range(40):
        a = [rng.randrange(12) for _ in range(rng.randrange(0, 60))]
        b = list(a)
        for _ in range(rng.randrange(0, 8)):       # a few edits, like tokenizer drift
            if b and rng.random() < 0.5:
                del b[rng.randrange(len(b))]
            else:
                b.insert(rng.randrange(len(b) + 1), rng.randrange(12))
        ia, ib = lcs_match(a, b)
        ref = _lcs_python(a, b)
        assert len(ia) == len(ref[0])
        assert all(a[i] == b[j] for i, j in zip(ia, ib))
        assert all(x < y for x, y in zip(ia, ia[1:])) and all(x < y for x, y in zip(ib, ib[1:]))
    assert lcs_match([1, 2, 3, 4], [9, 8, 7, 6], max_d=2) is None
    # identical sequences: rewards pass through
    r = redistribute_rewards([5, 6, 7], [5, 6, 7], [0.1, 0.2, 0.3])
    assert torch.allclose(r, torch.tensor([0.1, 0.2, 0.3]))
    # one original token re-encoded as two: it gets the mean of their rewards; neighbours keep theirs
    r = redistribute_rewards([5, 60, 7], [5, 61, 62, 7], [1.0, 2.0, 4.0, 8.0])
    assert torch.allclose(r, torch.tensor([1.0, 3.0, 8.0]))
    # two original tokens merged into nothing on the other side: the gap takes the mean of its neighbours
    r = redistribute_rewards([5, 60, 61, 7], [5, 7], [1.0, 3.0])
    assert torch.allclose(r, torch.tensor([1.0, 2.0, 2.0, 3.0]))
    # python fallback gives the same answer; the batch version equals the loop
    a, b = [3, 4, 5, 9, 9, 6], [3, 5, 8, 6]
    rw = [0.5, 1.0, 2.0, 4.0]
    assert torch.allclose(redistribute_rewards(a, b, rw), redistribute_rewards(a, b, rw, native=False))
    outs = redistribute_rewards_batch([a, [1, 2]], [b, [1, 2]], [rw, [0.0, 1.0]], workers=2)
    assert torch.allclose(outs[0], redistribute_rewards(a, b, rw)) and outs[1].tolist() == [0.0, 1.0]


def test_moe_load_recorder_and_tensor_ipc(tmp_path):
    import json
    from gcore_b200.models.config import ModelConfig
    from gcore_b200.models.gpt import GPTModel
    from gcore_b200.utils.debug_moe import MoeLoadRecorder
    cfg = ModelConfig(arch="qwen3_moe", num_layers=2, hidden_size=64, num_attention_heads=2, num_kv_heads=2,
                      ffn_hidden_size=128, vocab_size=128, num_experts=4, moe_top_k=2, moe_ffn_hidden_size=32,
                      dtype="float32")
    torch.manual_seed(0)
    model = GPTModel(cfg, recompute="none")
    rec = MoeLoadRecorder(model)
    t = torch.randint(3, 128, (10,))
    with torch.no_grad():
        model(t, torch.arange(10, dtype=torch.int32), torch.tensor([0, 10], dtype=torch.int32), 10)
    s = rec.summary()
    assert sorted(s) == [0, 1] and all(v["tokens"] == 20 and sum(v["counts"]) == 20 for v in s.values())
    assert all(0 < v["entropy_frac"] <= 1.0 and v["max_over_mean"] >= 1.0 for v in s.values())
    rec.dump(str(tmp_path / "moe.jsonl"), step=3)
    row = json.loads(open(tmp_path / "moe.jsonl").read())
    assert row["step"] == 3 and set(row["layers"]) == {"0", "1"} and rec.summary() == {}
    rec.close()
    # a host tensor handed to another process by handle: the child's in-place update is visible here
    import torch.multiprocessing as mp
    from gcore_b200.utils.tensor_ipc import _child, export_handle
    x = torch.arange(6, dtype=torch.float32)
    ctx = mp.get_context("spawn")
    a, b = ctx.Pipe()
    p = ctx.Process(target=_child, args=(b,))
    p.start()
    a.send(export_handle(x))
    assert a.recv() == 21.0
    p.join(30)
    assert x.tolist() == [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]


def test_data_convert_tools(tmp_path):
    import json
    from gcore_b200.data.datasets import IndexedJsonlDataset, PretrainTokenDataset, SftDataset
    from gcore_b200.tools import data_convert, gpu_check
    chat = tmp_path / "chat.jsonl"
    chat.write_text(json.dumps({"messages": [{"role": "user", "content": "2+2?"},
                                             {"role": "assistant", "content": "4"}]}) + "\n" +
                    json.dumps({"prompt": "hi", "response": "there"}) + "\n")
    assert data_convert.main(["sft", "--src", str(chat), "--dst", str(tmp_path / "sft.jsonl")]) == 2
    ds = IndexedJsonlDataset(str(tmp_path / "sft.jsonl"))
    assert ds[1]["prompt"] == [ord(c) + 3 for c in "hi"] and bytes(t - 3 for t in ds[0]["response"]) == b"4"
    item = SftDataset(ds, None, 64, "prompt", "response")[0]
    assert item["prompt_length"] == len(ds[0]["prompt"]) and item["sequence_length"] == len(ds[0]["prompt"]) + 1
    text = tmp_path / "text.jsonl"
    text.write_text("\n".join(json.dumps({"text": "abcdefgh" * (i + 1)}) for i in range(5)) + "\n")
    assert data_convert.main(["pretrain", "--src", str(text), "--dst", str(tmp_path / "tok.jsonl")]) == 5
    rows = PretrainTokenDataset(IndexedJsonlDataset(str(tmp_path / "tok.jsonl")), None, 16)
    assert len(rows) == (8 * 15) // 16 and rows[0]["tokens"].tolist() == [ord(c) + 3 for c in "abcdefgh" * 2]
    q = tmp_path / "q.jsonl"
    q.write_text(json.dumps({"question": "1+1", "answer": "2"}) + "\n")
    assert data_convert.main(["prompts", "--src", str(q), "--dst", str(tmp_path / "p.jsonl")]) == 1
    assert IndexedJsonlDataset(str(tmp_path / "p.jsonl"))[0]["answer"] == "2"
    # LLaMA-Factory layouts: ShareGPT conversations, Alpaca instructions (with history), and preference pairs
    lf = tmp_path / "lf.jsonl"
    lf.write_text(
        json.dumps({"system": "be brief", "conversations": [{"from": "human", "value": "2+2?"},
                                                             {"from": "gpt", "value": "4"},
                                                             {"from": "human", "value": "and 3+3?"},
                                                             {"from": "gpt", "value": "6"}]}) + "\n" +
        json.dumps({"instruction": "Add.", "input": "1 1", "output": "2", "history": [["Add. 0 0", "0"]]}) + "\n")
    assert data_convert.main(["sft", "--src", str(lf), "--dst", str(tmp_path / "lf_sft.jsonl")]) == 2
    ds = IndexedJsonlDataset(str(tmp_path / "lf_sft.jsonl"))
    dec = lambda ids: bytes(t - 3 for t in ids).decode()
    assert dec(ds[0]["response"]) == "6" and dec(ds[0]["prompt"]).startswith("<|system|>\nbe brief\n<|user|>\n2+2?")
    assert dec(ds[0]["prompt"]).endswith("<|user|>\nand 3+3?\n<|assistant|>\n")
    assert dec(ds[1]["response"]) == "2" and "<|assistant|>\n0\n<|user|>\nAdd.\n1 1\n" in dec(ds[1]["prompt"])
    pref = tmp_path / "pref.jsonl"
    pref.write_text(
        json.dumps({"conversations": [{"from": "human", "value": "capital of France?"}],
                    "chosen": {"from": "gpt", "value": "Paris"}, "rejected": {"from": "gpt", "value": "Rome"}}) + "\n" +
        json.dumps({"instruction": "Say hi", "output": ["hi", "bye"]}) + "\n" +
        json.dumps({"prompt": "x", "chosen": "good", "rejected": "bad"}) + "\n")
    assert data_convert.main(["dpo", "--src", str(pref), "--dst", str(tmp_path / "dpo.jsonl")]) == 3
    dp = IndexedJsonlDataset(str(tmp_path / "dpo.jsonl"))
    assert [dec(dp[i]["chosen"]) for i in range(3)] == ["Paris", "hi", "good"]
    assert [dec(dp[i]["rejected"]) for i in range(3)] == ["Rome", "bye", "bad"]
    assert dec(dp[1]["prompt"]) == "<|user|>\nSay hi\n<|assistant|>\n" and dec(dp[2]["prompt"]) == "x"
    rep = gpu_check.main([])       # no GPU here: the report says so instead of failing
    assert rep["cuda_available"] is False and rep["ok"] is False


def test_over_dispatch_prompt_reuse_and_two_turn_reflect():
    import time
    from gcore_b200.rollout_generator.async_rollout import RolloutController
    from gcore_b200.rollout_generator.generators import TwoTurnReflectGenerator

    class Sampler:
        def generate(self, prompts, params=None):
            time.sleep(0.001)
            return [{"tokens": list(p) + [7]} for p in prompts]

    def prompts():
        i = 0
        while True:
            yield [[i * 10 + j] for j in range(4)]
            i += 1

    def score(samples):
        for s in samples:
            s["rewards"] = 1.0
        return samples

    c = RolloutController(prompts(), [Sampler()], score, repeat_n=2, groups_per_batch=2, max_staleness=0,
                          over_dispatch_ratio=3.0, reuse_unused_prompts=True)
    assert c.max_inflight == 6                      # 3x more groups in flight than one batch needs
    c.set_weight_version(0)
    b0 = c.collect(timeout_s=30)
    used = {tuple(s["tokens"][:1]) for s in b0}
    time.sleep(0.05)                                # the over-dispatched groups finish with version-0 weights
    c.set_weight_version(1)
    b1 = c.collect(timeout_s=30)
    assert c.stats["dropped_stale"] >= 1 and c.stats["reused_prompts"] == c.stats["dropped_stale"]
    assert all(s["weight_version"] == 1 for s in b1)
    # a prompt whose stale group was dropped is generated again instead of being lost
    time.sleep(0.05)
    c.set_weight_version(1)
    seen = {tuple(s["tokens"][:1]) for s in b1} | used
    b2 = c.collect(timeout_s=30)
    assert {tuple(s["tokens"][:1]) for s in b2} <= {(i,) for i in range(100)} and len(seen) >= 3
    c.shutdown()

    class FakeTrainer:
        def __init__(self):
            self.calls = []

        def rollout(self, prompts):
            self.calls.append([list(p) for p in prompts])
            out = []
            for gi, p in enumerate(prompts):
                for j in range(3):
                    out.append({"tokens": torch.tensor(list(p) + [100 + j]), "prompt_length": len(p),
                                "group_id": gi, "unique_id": (len(self.calls), gi, j)})
            return out

        def score(self, samples):
            for s in samples:
                s["rewards"] = torch.tensor(float(s["tokens"][-1]))     # last token = quality
            return samples

    class Cfg:
        class training:
            sampling_repeat_n, sampling_keep_n, sampling_keeping_strategy = 3, 3, "all"
            filter_sampling_py_path = None

    tr = FakeTrainer()
    gen = TwoTurnReflectGenerator(tr, Cfg, reflect_tokens=[9, 9], top_k=1)
    assert gen.rb_multiplier == 3
    batch = gen(iter([[[1, 2], [3]]]), 0)
    assert len(batch) == 2 * 3 + 4 * 3 and len(tr.calls) == 2
    # second-turn prompts: worst (…100) and best (…102) first-turn conversation of every prompt + the reflect message
    assert tr.calls[1] == [[1, 2, 100, 9, 9], [1, 2, 102, 9, 9], [3, 100, 9, 9], [3, 102, 9, 9]]
    second = [s for s in batch if s["turn"] == 2]
    assert sorted({s["group_id"] for s in second}) == [2, 3, 4, 5] and second[0]["reflect_kind"] == "worst"
    assert second[0]["prompt_length"] == 5      # the first turn is context in the second turn


def test_eval_server_and_client_over_http():
    from gcore_b200.client.rpc import serve
    from gcore_b200.tools.eval_server import EvalClient, EvalService

    def reward(samples):
        return torch.tensor([1.0 if int(s["tokens"][-1]) % 2 == 0 else 0.0 for s in samples])

    srv, url = serve(EvalService(reward), allowed=["score", "evaluate", "health"])
    try:
        c = EvalClient([url])
        samples = [{"tokens": torch.tensor([5, 6, t]), "prompt_length": 2} for t in (2, 3, 4, 5, 7, 9)]
        assert c.score(samples) == [1.0, 0.0, 1.0, 0.0, 0.0, 0.0]
        m = c.evaluate(samples, n=3, ks=(1, 3))      # prompt 0: 2 of 3 correct, prompt 1: none
        assert abs(m["eval/pass@1"] - (2 / 3) / 2) < 1e-6 and abs(m["eval/pass@3"] - 0.5) < 1e-6
        assert c.health()[0]["samples"] == 12
    finally:
        srv.shutdown()


def test_qwen2_moe_shared_expert_gate_and_hf_round_trip(tmp_path):
    """qwen2_moe: the shared expert's output is scaled by sigmoid(x . g); HF import / export use the family's names
    (``shared_expert.*``, ``shared_expert_gate``) and round-trip the weights."""
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "workers"))
    from gcore_b200.checkpoint.hf import load_hf, read_hf_dir, save_hf
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import from_hf_config
    hf = {"model_type": "qwen2_moe", "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 2,
          "num_key_value_heads": 2, "intermediate_size": 128, "vocab_size": 128, "num_experts": 4,
          "num_experts_per_tok": 2, "moe_intermediate_size": 32, "shared_expert_intermediate_size": 48,
          "norm_topk_prob": False, "torch_dtype": "float32"}
    cfg = from_hf_config(hf)
    cfg.dtype = "float32"
    assert cfg.arch == "qwen2_moe" and cfg.moe_shared_expert_gate and cfg.qkv_bias and cfg.moe_shared_expert_ffn == 48

    def engine(seed):
        e = TrainingEngine(PolicyConfig(recompute="none", without_ref=True), OptimizerConfig(lr=1e-3),
                           TrainingConfig(train_mbs=2, train_gbs=2), model_cfg=cfg)
        e.setup_model_and_get_optimizer(seed=seed)
        return e

    a = engine(1)
    layer = a.model.decoder.layers[0].mlp
    with torch.no_grad():
        layer.shared_expert_gate.weight.normal_(0, 0.5)
    x = torch.randn(6, 64)
    with torch.no_grad():
        y, _ = layer(x)
        w = layer.shared_expert_gate.weight.clone()
        shared = layer.shared_experts(x) * torch.sigmoid(x @ w.t())
        layer.shared_experts.linear_fc2.weight.zero_()
        y_routed, _ = layer(x)
    assert torch.allclose(y - y_routed, shared, atol=2e-2)     # bf16-rounded expert outputs
    save_hf(a, str(tmp_path / "hf"))
    names = set(read_hf_dir(str(tmp_path / "hf")))
    assert "model.layers.0.mlp.shared_expert_gate.weight" in names
    assert "model.layers.1.mlp.shared_expert.up_proj.weight" in names and "model.layers.0.mlp.experts.3.down_proj.weight" in names
    b = engine(2)
    load_hf(b, str(tmp_path / "hf"))
    for (n, p), (_, q) in zip(a.model.named_parameters(), b.model.named_parameters()):
        assert torch.equal(p, q), n


def test_native_planners_properties():
    """The C++ planners of the runtime library on random inputs: every index placed once, bins within capacity and no
    more of them than first-fit-decreasing in Python, k-way partitions balanced (and of equal size when asked)."""
    import random
    from gcore_b200.core.packing import ffd_pack, kk_partition
    rng = random.Random(7)
    for trial in range(60):
        n = rng.randrange(1, 120)
        cap = rng.choice([512, 2048, 8192])
        lens = [rng.randrange(1, cap + 1) for _ in range(n)]
        bins = ffd_pack(lens, cap)
        assert sorted(i for b in bins for i in b) == list(range(n))
        assert all(sum(lens[i] for i in b) <= cap for b in bins)
        # python first-fit-decreasing as the yardstick
        loads = []
        for i in sorted(range(n), key=lambda i: -lens[i]):
            for j in range(len(loads)):
                if loads[j] + lens[i] <= cap:
                    loads[j] += lens[i]
                    break
            else:
                loads.append(lens[i])
        assert len(bins) <= len(loads)
        assert len(bins) >= -(-sum(lens) // cap)          # and never fewer than the volume bound
        k = rng.randrange(1, min(n, 8) + 1)
        parts = kk_partition(lens, k)
        assert sorted(i for p in parts for i in p) == list(range(n)) and len(parts) == k
        sums = [sum(lens[i] for i in p) for p in parts]
        assert max(sums) - min(sums) <= 2 * max(lens)
        if n % k == 0:
            eq = kk_partition(lens, k, equal_size=True)
            assert all(len(p) == n // k for p in eq) and sorted(i for p in eq for i in p) == list(range(n))


def test_loss_free_load_balancing_moves_the_router_bias_towards_even_load():
    """A sigmoid router with a selection bias, released by ``freeze_router_correction_bias=false``: every step the bias
    of over-loaded experts drops and that of under-loaded ones rises by the update speed, the counts are reset, and
    over the steps the load violation shrinks; the frozen default leaves the bias alone."""
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import ModelConfig
    from gcore_b200.models.moe import Router, update_router_bias
    mc = ModelConfig(arch="deepseek_v3", num_layers=2, hidden_size=64, num_attention_heads=2, num_kv_heads=2,
                     ffn_hidden_size=128, vocab_size=128, num_experts=8, moe_top_k=2, moe_ffn_hidden_size=32,
                     moe_router_type="sigmoid_group", moe_router_bias=True, moe_n_group=1, moe_topk_group=1,
                     dtype="float32")

    def engine(**tk):
        e = TrainingEngine(PolicyConfig(recompute="none", without_ref=True),
                           OptimizerConfig(lr=0.0, lr_decay_style="constant", weight_decay=0.0),
                           TrainingConfig(train_mbs=4, train_gbs=4, **tk), model_cfg=mc)
        e.setup_model_and_get_optimizer(seed=3)
        return e

    g = torch.Generator().manual_seed(0)
    batch = [{"tokens": torch.randint(3, 128, (64,), generator=g), "loss_mask": torch.ones(64)} for _ in range(4)]
    e = engine()
    e.finetune_step(batch)
    routers = [m for m in e.model.modules() if isinstance(m, Router)]
    assert routers and all(float(r.expert_bias.abs().sum()) == 0.0 for r in routers)

    e = engine(freeze_router_correction_bias=False, router_correction_bias_update_speed=0.01)
    routers = [m for m in e.model.modules() if isinstance(m, Router)]
    # make the first expert of the first MoE layer the favourite, so that the start is clearly unbalanced
    with torch.no_grad():
        routers[0].weight[0] += 0.5 * routers[0].weight[0].sign()
    first = e.finetune_step(batch)
    r = routers[0]
    assert float(r.tokens_per_expert.sum()) == 0.0                       # reset after the update
    assert all(min(abs(v), abs(v - 0.01)) < 1e-6 for v in r.expert_bias.abs().tolist())
    assert "moe/max_violation" in first
    vio = [first["moe/max_violation"]] + [e.finetune_step(batch)["moe/max_violation"] for _ in range(30)]
    assert min(vio[-5:]) < vio[0], vio
    # counts: one per routed (token, k) pair of the step, each layer
    e.model.train()
    hidden = torch.randn(10, 64)
    routers[0](hidden)
    assert float(routers[0].tokens_per_expert.sum()) == 20.0
    with torch.no_grad():
        routers[0](hidden)                                               # passes without grad are not counted
    assert float(routers[0].tokens_per_expert.sum()) == 20.0
    before = routers[0].expert_bias.clone()
    c = routers[0].tokens_per_expert.clone()
    update_router_bias(e.model, 0.1, use_abs=False)
    want = before + 0.1 * torch.log((c.mean() + 1) / (c + 1))
    assert torch.allclose(routers[0].expert_bias, want, atol=1e-6)


def test_async_controller_hands_a_batched_sampler_all_groups_of_a_round_at_once():
    """A sampler with ``generate_groups`` (the colocated engine) gets every prompt group fired in a round in one
    call, so the engine decodes groups x samples sequences per step instead of one group at a time."""
    from gcore_b200.rollout_generator.async_rollout import RolloutController
    calls = []

    class Batched:
        def generate_groups(self, prompts, n, params=None):
            calls.append(len(prompts))
            return [{"tokens": list(p) + [j]} for p in prompts for j in range(n)]

    def prompts():
        k = 0
        while True:
            yield [[k, k + 1], [k + 2, k + 3]]
            k += 4

    def score(samples):
        for s in samples:
            s["rewards"] = float(s["tokens"][-1])
        return samples

    c = RolloutController(prompts(), [Batched()], score, repeat_n=3, groups_per_batch=4, max_staleness=0)
    batch = c.collect(timeout_s=20)
    assert calls[0] == 4 and len(batch) == 12 and c.stats["batched_calls"] >= 1
    assert [s["group_id"] for s in batch] == [0] * 3 + [1] * 3 + [2] * 3 + [3] * 3
    assert [s["tokens"][-1] for s in batch[:3]] == [0, 1, 2]
    c.shutdown()


def test_grouped_fp8_expert_projection_cpu_definition():
    """``policy.fp8`` reaches the grouped expert projections: forward through quantise -> grouped product (here the
    PyTorch definition of the kernel), backward in the compute dtype; close to the unquantised projection."""
    import torch
    from gcore_b200.models.moe import grouped_linear
    torch.manual_seed(0)
    G, N, K = 3, 128, 256
    offs = torch.tensor([0, 128, 256, 384], dtype=torch.int32)
    x = torch.randn(384, K).requires_grad_(True)
    w = (torch.randn(G, N, K) * 0.05).requires_grad_(True)
    y = grouped_linear(x, w, offs, "fp8", {})
    x2, w2 = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    y2 = grouped_linear(x2, w2, offs)
    assert (y - y2).abs().max() / y2.abs().max() < 0.08
    y.sum().backward()
    y2.sum().backward()
    assert (x.grad - x2.grad).abs().max() / x2.grad.abs().max() < 0.08
    assert torch.allclose(w.grad, w2.grad, atol=1e-4)


def test_fp8_data_and_weight_gradients_follow_the_bf16_ones(monkeypatch):
    """The fp8 linear's backward on the block-fp8 product: the data gradient from the transposed e4m3 weight cache
    (codes moved, not re-quantised), and, when switched on, the weight gradient with both operands quantised along
    the token axis; dense and grouped (per-expert) forms, against the unquantised gradients."""
    import torch
    from gcore_b200.models.moe import grouped_linear
    from gcore_b200.ops import quant
    from gcore_b200.ops.lowp_linear import fp8_linear
    torch.manual_seed(1)
    # the transposed cache holds exactly the transposed values
    w = torch.randn(2 * 256, 128) * 0.05
    q, s = quant.quant_weight_128x128(w.bfloat16())
    qt, st = quant.transpose_weight_128x128(q, s, groups=2)
    full = quant.dequant_128x128(q, s).view(2, 256, 128)
    assert torch.equal(quant.dequant_128x128(qt, st).view(2, 128, 256), full.transpose(1, 2))

    def grads(env_d, env_w):
        monkeypatch.setenv("GCORE_FP8_DGRAD", env_d)
        monkeypatch.setenv("GCORE_FP8_WGRAD", env_w)
        x = (torch.randn(200, 256, generator=torch.Generator().manual_seed(2))).requires_grad_(True)
        wt = (torch.randn(384, 256, generator=torch.Generator().manual_seed(3)) * 0.05).requires_grad_(True)
        y = fp8_linear(x, wt, None, None, {})
        y.backward(torch.randn(200, 384, generator=torch.Generator().manual_seed(4)))
        return x.grad, wt.grad
    dx0, dw0 = grads("0", "0")
    dx1, dw1 = grads("1", "1")
    assert not torch.equal(dx0, dx1) and (dx0 - dx1).abs().max() / dx0.abs().max() < 0.08
    assert not torch.equal(dw0, dw1) and (dw0 - dw1).abs().max() / dw0.abs().max() < 0.08

    offs = torch.tensor([0, 128, 128, 384], dtype=torch.int32)    # the middle expert has no rows
    outs = []
    for flag in ("0", "1"):
        monkeypatch.setenv("GCORE_FP8_DGRAD", flag)
        x = torch.randn(384, 256, generator=torch.Generator().manual_seed(5)).requires_grad_(True)
        wg = (torch.randn(3, 128, 256, generator=torch.Generator().manual_seed(6)) * 0.05).requires_grad_(True)
        grouped_linear(x, wg, offs, "fp8", {}).backward(
            torch.randn(384, 128, generator=torch.Generator().manual_seed(7)))
        outs.append(x.grad)
    assert not torch.equal(outs[0], outs[1]) and (outs[0] - outs[1]).abs().max() / outs[0].abs().max() < 0.08
