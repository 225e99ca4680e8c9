"""Logging subsystem (aggregated log written by several processes, DEBUG shards, descriptor-level engine log
redirection) and reloadable process groups (gloo)."""
import os
import re
import subprocess
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_WORKER = r'''
import os, sys
sys.path.insert(0, sys.argv[1])
from gcore_b200.utils import logging_utils as L
rank = int(sys.argv[2])
os.environ["GCORE_TASK_DIR"] = sys.argv[3]
L.setup_logging(run_name="t", role="train", rank=rank, debug_shards=True)
lg = L.get_logger("w")
for i in range(200):
    lg.info("line %d of rank %d " % (i, rank) + "x" * 150)
lg.debug("only in the shard")
with L.redirect_engine_output(step=7):
    os.write(1, b"printed by native code\n")      # bypasses sys.stdout, as a C library would
    print("printed by python", flush=True)
print("after redirect rank", rank, flush=True)
'''


def test_ranks_share_one_log_without_interleaving_and_engine_output_is_redirected(tmp_path):
    d = str(tmp_path / "task")
    w = tmp_path / "w.py"
    w.write_text(_WORKER)
    procs = [subprocess.Popen([sys.executable, str(w), ROOT, str(r), d], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                              text=True) for r in range(3)]
    outs = [p.communicate(timeout=120) for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    lines = open(os.path.join(d, "training.log")).read().splitlines()
    pat = re.compile(r"^\S+ \S+ - INFO - role=train - rank=(\d) - pid=\d+ - node=\S+ - line (\d+) of rank (\d) x{150}$")
    seen = {}
    for ln in lines:
        m = pat.match(ln)
        assert m, ln[:120]                       # every line is one whole record
        assert m.group(1) == m.group(3)
        seen.setdefault(m.group(1), []).append(int(m.group(2)))
    assert sorted(seen) == ["0", "1", "2"] and all(v == list(range(200)) for v in seen.values())
    shards = os.listdir(os.path.join(d, "debug"))
    assert len(shards) == 3 and any("only in the shard" in open(os.path.join(d, "debug", s)).read() for s in shards)
    eng = open(os.path.join(d, "infer_engine_log", "sampler_rank1.log")).read()
    assert "ppo_step 7 begin" in eng and "printed by native code" in eng and "printed by python" in eng \
        and eng.rstrip().splitlines()[-1].startswith("===== ppo_step 7 end")
    assert "after redirect rank 1" in outs[1][0] and "printed by native code" not in outs[1][0]


def _pg_worker(rank, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=4)
    from gcore_b200.utils import reloadable_process_group as R
    a = R.new_reloadable_group([0, 1], name="left")
    b = R.new_reloadable_group([2, 3], name="right")
    c = R.new_reloadable_group([0, 1, 2, 3], name="all")
    mine = a if rank < 2 else b
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=mine.group)
    first = float(t)
    assert R.offload_all(only_backend=None) == 3 and not c.loaded
    try:
        _ = c.group
        raised = False
    except RuntimeError:
        raised = True
    assert R.reload_all() == 3 and c.loads == 2
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=mine.group)
    u = torch.tensor([1.0])
    dist.all_reduce(u, group=c.group)
    q.put((rank, first, float(t), float(u), raised, mine.rank(), mine.size()))
    dist.barrier()
    dist.destroy_process_group()


def test_process_groups_survive_an_offload_reload_cycle():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_pg_worker, args=(r, 29611, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(4))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, first, again, total, raised, grank, gsize in res:
        want = 1.0 if rank < 2 else 5.0
        assert first == want and again == want and total == 4.0 and raised and grank == rank % 2 and gsize == 2
