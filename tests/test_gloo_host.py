"""Host-side multi-process logic on CPU (gloo, world size 2): every process compiles the same plan and takes the
ops of its own ranks; together they must cover the plan exactly once and agree on sizes found by a reduction."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    import torch
    import torch.distributed as dist
    sys.path.insert(0, %r)
    from rbruck_alltoallv_b200 import Plan
    from rbruck_alltoallv_b200.utils import distributions as D

    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    P = 8
    L = P // world
    mine = set(range(rank * L, (rank + 1) * L))
    for algo, kw in (("rbruck", dict(r=2)), ("tuna2", dict(r=3, b=2)), ("ttpl_bt_s1", dict(n=4, r=2)), ("spreadout", {})):
        plan = Plan(algo, P, **kw).check()
        ops = plan.ops()
        local = [tuple(int(v) for v in o) for o in ops if int(o["src"]) in mine]
        gathered = [None] * world
        dist.all_gather_object(gathered, local)
        merged = sorted(sum(gathered, []))
        assert merged == sorted(tuple(int(v) for v in o) for o in ops), algo
        # each process's share keeps the plan's order (keys never decrease)
        keys = [t[6] for t in local]
        assert keys == sorted(keys), algo
    # the agreed cell size of the eager protocol: a MAX reduction over every process's own rows
    counts = D.zipf(P, 4096, seed=3)
    local_max = int(counts[sorted(mine)].max()) * 4
    t = torch.tensor([local_max], dtype=torch.int64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert int(t.item()) == int(counts.max()) * 4
    # algo="auto": per-process totals that differ by far more than a size class must still give one choice
    from types import SimpleNamespace
    from rbruck_alltoallv_b200.ops import alltoallv as A
    from rbruck_alltoallv_b200.parallel import tuner
    tuner._TABLE = {}
    tuner.record(8, 2, 300, {"algo": "linear", "protocol": "eager"}, 10.0)
    tuner.record(8, 2, 40000, {"algo": "rbruck", "r": 2, "protocol": "rendezvous"}, 10.0)
    tuner.record(8, 2, 700000, {"algo": "pairwise", "protocol": "rendezvous"}, 10.0)
    side = dist.new_group(backend="gloo")
    comm = SimpleNamespace(P=8, L=4, nproc=2, arena_bytes=64 << 20, _side=side, _dist=dist,
                           max_block_bytes=lambda sc, ts: 4096)
    sc = np.full((4, 8), 64 if rank == 0 else 20000, dtype=np.int32)      # 256 B blocks here, 80 KB blocks there
    recv = [torch.empty(4, dtype=torch.float32)]
    got = A._auto_choice(comm, recv, sc, {}, agree_on_max=True)
    both = [None] * world
    dist.all_gather_object(both, (got["algo"], got.get("r"), "eager_max_bytes" in got))
    assert both[0] == both[1], both
    assert got["algo"] == "rbruck", got                                    # the class of the global mean (40 KB)
    # a one-shot call has no agreement step: without a hint that is the same everywhere it must not consult its own rows
    one = A._auto_choice(comm, recv, sc, {}, agree_on_max=False)
    assert one["algo"] == "spreadout" and "eager_max_bytes" not in one
    hinted = A._auto_choice(comm, recv, sc, {"mean_block_bytes": 700000.0}, agree_on_max=False)
    assert hinted["algo"] == "pairwise"
    dist.barrier()
    dist.destroy_process_group()
    print("worker", rank, "ok")
""")


def test_two_gloo_processes_partition_the_plan(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29591", str(script)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("ok") == 2
