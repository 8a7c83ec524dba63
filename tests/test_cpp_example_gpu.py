"""The C++ example builds against the in-tree library and its self check passes."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_example(tmp_path):
    from rbruck_alltoallv_b200 import _build
    lib = _build.build_cuda()
    exe = tmp_path / "rbruckv_example"
    nvcc = _build._nvcc()
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
           f"-I{_build.INCLUDE}", os.path.join(ROOT, "examples", "rbruckv_example.cu"), "-o", str(exe),
           str(lib), f"-Xlinker=-rpath={lib.parent}"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    run = subprocess.run([str(exe), "2", "8", "2", "4"], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
    assert "has errors" not in run.stdout and run.stdout.count("[Rbruckv]") == 22
