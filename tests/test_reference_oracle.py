"""The reference's own code as the oracle (no GPU).

Its sources are compiled unchanged against the threads-as-ranks MPI stand-in (``baseline/``) and run on 8 CPU
ranks with int32 elements and block sizes drawn uniformly from [0, 256] (fixed seed).  For every algorithm the
harness knows, the bytes the reference leaves in each rank's receive buffer are compared, byte for byte, with
what this library's schedule of the same algorithm produces through its CPU executor, and with the direct-copy
expectation.  Skipped where neither the reference tree nor a copy of it is available.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from rbruck_alltoallv_b200 import Plan, host_alltoallv
from rbruck_alltoallv_b200.utils import distributions as dist
from rbruck_alltoallv_b200.utils import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))

P, TS, SEED = 8, 4, 20240104

#            algorithm            runner arguments n r r2 b b2     our plan's arguments
CASES = [("rbruck", (0, 2, 0, 0, 0), dict(r=2)), ("rbruck", (0, 4, 0, 0, 0), dict(r=4)),
         ("rbruck", (0, 3, 0, 0, 0), dict(r=3)), ("rbruck", (0, 8, 0, 0, 0), dict(r=8)),
         ("rbruck_om", (0, 2, 0, 0, 0), dict(r=2)), ("rbruck_om", (0, 4, 0, 0, 0), dict(r=4)),
         ("tuna", (0, 2, 0, 1, 0), dict(r=2, b=1)), ("tuna", (0, 3, 0, 2, 0), dict(r=3, b=2)),
         ("tuna2", (0, 2, 0, 1, 0), dict(r=2, b=1)), ("tuna2", (0, 4, 0, 1, 0), dict(r=4, b=1)),
         ("ttpl_bt", (4, 2, 0, 1, 0), dict(n=4, r=2, b=1)), ("ttpl_bt", (2, 2, 0, 0, 0), dict(n=2, r=2)),
         ("ttpl_bt_s1", (4, 2, 0, 2, 0), dict(n=4, r=2, b=2)), ("ttpl_bt_s1", (2, 2, 0, 0, 0), dict(n=2, r=2)),
         ("scattered", (0, 2, 0, 3, 0), dict(b=3)), ("linear", (0, 2, 0, 0, 0), {}), ("pairwise", (0, 2, 0, 0, 0), {}),
         ("xor", (0, 2, 0, 0, 0), {}), ("twolayer_linear", (4, 2, 0, 0, 0), dict(n=4)),
         ("twolayer_linear_s2", (4, 2, 0, 2, 3), dict(n=4, b=2, b2=3))]


@pytest.fixture(scope="module")
def runner():
    import install_reference
    try:
        path = install_reference.ensure_built()
    except Exception as e:   # no compiler, broken copy
        pytest.skip(f"reference build failed: {e}")
    if path is None:
        pytest.skip("no reference tree (set RBV_REFERENCE_DIR) and no copy under baseline/_ref")
    return str(path)


@pytest.fixture(scope="module")
def problem(tmp_path_factory):
    counts = dist.uniform(P, 256, seed=SEED)
    prob = oracle.make_problem(counts, TS, SEED, packed=True)
    send = oracle.fill_send(prob, SEED)
    d = tmp_path_factory.mktemp("refio")
    np.savetxt(d / "counts.txt", counts, fmt="%d")
    for r in range(P):
        send[r][: int(prob.send_bytes[r])].tofile(d / f"send_{r}.bin")
    return prob, send, d


@pytest.mark.parametrize("algo,rargs,kw", CASES, ids=[f"{a}-{'-'.join(map(str, r))}" for a, r, _ in CASES])
def test_receive_bytes_equal_the_references(runner, problem, algo, rargs, kw):
    prob, send, d = problem
    env = dict(os.environ, REF_SEND_DIR=str(d), REF_RECV_DIR=str(d))
    cmd = [runner, algo, str(P), str(TS), str(d / "counts.txt"), "1", "0", *map(str, rargs)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=120, env=env)
    assert res.returncode == 0, res.stderr[-500:]
    info = json.loads(res.stdout.strip().splitlines()[-1])
    assert info["rc"] == 0
    ref = [np.fromfile(d / f"recv_{r}.bin", dtype=np.uint8) for r in range(P)]
    # this library's schedule of the same algorithm, executed on the CPU
    recv = oracle.empty_recv(prob)
    assert host_alltoallv(Plan(algo, P, **kw).check(), send, recv, prob.counts, prob.sdispls, prob.rdispls, TS) == 0
    want = oracle.expected_recv(prob, send, tail=0)
    for r in range(P):
        n = int(prob.recv_bytes[r])
        assert len(ref[r]) == n
        assert np.array_equal(recv[r][:n], ref[r]), f"{algo}: rank {r} differs from the reference's receive buffer"
        assert np.array_equal(ref[r], want[r][:n]), f"{algo}: the reference itself differs from a direct copy on rank {r}"


def test_the_references_unfinished_two_layer_bruck_is_not_an_oracle(runner, problem):
    """TTPL_rbruck_alltoallv never unpacks its inter-group phase (src/twophase_twolayer_rbruck.cpp:178-227), so
    its receive buffers are wrong; this library completes the algorithm.  Recorded so that nobody uses it as one."""
    prob, send, d = problem
    env = dict(os.environ, REF_SEND_DIR=str(d), REF_RECV_DIR=str(d))
    res = subprocess.run([runner, "ttpl", str(P), str(TS), str(d / "counts.txt"), "1", "0", "4", "2"], capture_output=True,
                         text=True, timeout=120, env=env)
    assert res.returncode == 0
    want = oracle.expected_recv(prob, send, tail=0)
    ref = [np.fromfile(d / f"recv_{r}.bin", dtype=np.uint8) for r in range(P)]
    assert any(not np.array_equal(ref[r], want[r][: len(ref[r])]) for r in range(P))
    recv = oracle.empty_recv(prob)
    assert host_alltoallv(Plan("ttpl", P, n=4, r=2).check(), send, recv, prob.counts, prob.sdispls, prob.rdispls, TS) == 0
    assert oracle.first_mismatch(recv, oracle.expected_recv(prob, send)) is None
