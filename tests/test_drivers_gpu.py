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
    ("MLinputs", "2", "2", "--nranks", "4"),
])
def test_driver_runs_clean(argv):
    res = _run(*argv)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "has errors" not in res.stdout and "failed" not in res.stdout and "refused" not in res.stdout
    assert "[" in res.stdout or "TUNA" in res.stdout
