"""The driver programs run and their self checks pass (single GPU, all ranks on one device)."""
import subprocess
import sys
import os

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*argv):
    env = dict(os.environ, PYTHONPATH=ROOT)
    return subprocess.run([sys.executable, "-m", "rbruck_alltoallv_b200.drivers", *argv], cwd=ROOT, env=env,
                          capture_output=True, text=True, timeout=600)


@pytest.mark.parametrize("argv", [
    ("rbruckv", "3", "2", "4", "--nranks", "8", "--nmax", "64"),
    ("combAlltoallv", "2", "4", "2", "--nranks", "8", "--nmax", "32"),
    ("LTRNA", "2", "4", "2", "--nranks", "8", "--nmax", "32"),
    ("TLLiner_S2", "2", "4", "--nranks", "8", "--nmax", "32"),
    ("twolayer", "2", "4", "2", "--nranks", "8", "--nmax", "8"),
    ("otherDis", "2", "4", "--nranks", "8"),
    ("FFT", "2", "4", "--nranks", "8"),
    ("MLinputs", "2", "4", "--nranks", "4", "--heap-mb", "3072"),   # the reference's inputs/4proc trace when it is at hand
    ("merge", "2", "4", "16", "4096", "--nranks", "8"),
    ("simple_merge", "2", "4", "--nranks", "8", "--nmax", "64"),
    ("split", "2", "16", "1048576", "--nranks", "8"),
    ("gather", "2", "4", "--nranks", "8", "--nmax", "16"),
    ("balance", "2", "4", "--nranks", "8", "--nmax", "16"),
])
def test_driver_runs_clean(argv):
    res = _run(*argv)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "has errors" not in res.stdout and "failed" not in res.stdout and "refused" not in res.stdout
    assert "[" in res.stdout or "TUNA" in res.stdout


def test_recorded_trace_of_the_reference_runs_on_eight_ranks(tmp_path):
    """inputs/8proc/global_comm_pattern_8proc.txt of the reference (29 MB mean blocks, up to 324 MB per rank): the
    only bandwidth-heavy workload the reference ships.  Skipped where the file is not at hand."""
    sys.path.insert(0, ROOT)
    from rbruck_alltoallv_b200.drivers import _reference_input
    path = _reference_input(8)
    if path is None:
        pytest.skip("the reference's inputs/8proc matrix is not available on this machine")
    out = tmp_path / "ml.jsonl"
    res = _run("MLinputs", "2", "8", "--nranks", "8", "--heap-mb", "6144", "--input", str(path), "--jsonl", str(out))
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "failed" not in res.stdout and "Spread-out" in res.stdout and "TUNA" in res.stdout
    import json
    rows = [json.loads(l) for l in out.read_text().splitlines()]
    assert rows and all(r["status"] == "ok" and r["algbw_GBps"] > 0 for r in rows)
    assert rows[0]["total_bytes"] > 1_500_000_000


def test_recorded_trace_of_128_ranks_runs_as_logical_ranks(tmp_path):
    """inputs/128proc of the reference (6.7 GB in 15 000 blocks) on one GPU: 128 logical ranks, static kernel."""
    sys.path.insert(0, ROOT)
    from rbruck_alltoallv_b200.drivers import _reference_input
    path = _reference_input(128)
    if path is None:
        pytest.skip("the reference's inputs/128proc matrix is not available on this machine")
    res = _run("MLinputs", "2", "128", "--nranks", "128", "--heap-mb", "16000", "--arena-mb", "1", "--input", str(path))
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "failed" not in res.stdout and "Spread-out" in res.stdout


def test_timer_breakdown_lines_are_printed():
    res = _run("TLLiner_S2", "2", "4", "--nranks", "8", "--nmax", "32")
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "[TLLiner_S2-timers]" in res.stdout and "intra_time=" in res.stdout
    assert "[TLLiner_S2-iteration_time]" in res.stdout
