"""Host-side native code under sanitizers (no GPU): AddressSanitizer + UBSan over the plan compiler and the CPU
executor for every algorithm, ThreadSanitizer over the threads-as-ranks MPI stand-in.  The reference is built
with default flags only (CMakeLists.txt:5) and has no such checks."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "rbruck_alltoallv_b200" / "csrc"

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")


def _build_and_run(tmp_path, name, sources, flags, includes, env=None):
    exe = tmp_path / name
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *flags, *[f"-I{i}" for i in includes],
           *[str(s) for s in sources], "-o", str(exe), "-pthread"]
    b = subprocess.run(cmd, capture_output=True, text=True)
    if b.returncode != 0 and "sanitize" in (b.stderr or "") and "cannot find" in b.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert b.returncode == 0, b.stderr[-2000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    return r.stdout


def test_plan_compiler_and_executor_under_asan_ubsan(tmp_path):
    out = _build_and_run(tmp_path, "plan_asan",
                         [ROOT / "tests" / "native" / "plan_sanitize_main.cpp", CSRC / "plan" / "plan.cpp"],
                         ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], [CSRC / "include"])
    assert " 0 bad" in out


def test_mpi_stand_in_under_tsan(tmp_path):
    out = _build_and_run(tmp_path, "shim_tsan",
                         [ROOT / "tests" / "native" / "shim_tsan_main.cpp", ROOT / "baseline" / "mpi_shim" / "mpi_shim.cpp"],
                         ["-fsanitize=thread"], [ROOT / "baseline" / "mpi_shim"])
    assert "bad 0" in out
