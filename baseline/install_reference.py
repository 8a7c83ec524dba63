"""Installs the reference into ``baseline/_ref`` (git-ignored) and builds it, unchanged, against the MPI
stand-in of ``baseline/mpi_shim``.

Steps: (1) the offline ``pip install`` the task prescribes is attempted and its outcome is written to
``baseline/_ref/PIP_INSTALL.log`` (the reference is a CMake/MPI C++ project without Python packaging, so
it is expected to fail); (2) the reference's ``src/``, ``rbrucks.h``, ``examples/``, ``benchmarks/`` and the
small ``inputs/`` are copied verbatim to ``baseline/_ref/reference``; (3) ``src/*.cpp`` + the stand-in +
``ref_runner.cpp`` are compiled into ``baseline/_ref/ref_runner``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"
SRC_COPY = REF / "reference"


def pip_attempt(reference: Path) -> str:
    cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--find-links",
           "/opt/wheelhouse", "--target", str(REF), str(reference)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = "$ " + " ".join(cmd) + f"\nexit code {res.returncode}\n" + res.stdout[-2000:] + res.stderr[-2000:]
    (REF / "PIP_INSTALL.log").write_text(log)
    return log


def copy_sources(reference: Path) -> None:
    if SRC_COPY.exists():
        shutil.rmtree(SRC_COPY)
    SRC_COPY.mkdir(parents=True)
    shutil.copy2(reference / "rbrucks.h", SRC_COPY / "rbrucks.h")
    for d in ("src", "examples", "benchmarks"):
        shutil.copytree(reference / d, SRC_COPY / d)
    for p in ("4proc", "8proc", "16proc", "32proc", "64proc", "128proc", "256proc", "512proc", "1024proc"):
        if (reference / "inputs" / p).exists():
            shutil.copytree(reference / "inputs" / p, SRC_COPY / "inputs" / p)


def build() -> Path:
    """Compiles the copied reference sources; also usable on a machine that only has the copy."""
    out = REF / "ref_runner"
    srcs = sorted((SRC_COPY / "src").glob("*.cpp"))
    cmd = ["g++", "-O2", "-std=c++11", "-pthread", "-w", f"-I{HERE / 'mpi_shim'}", f"-I{SRC_COPY / 'src'}",
           *map(str, srcs), "-std=c++17", str(HERE / "mpi_shim" / "mpi_shim.cpp"), str(HERE / "ref_runner.cpp"),
           "-o", str(out)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode:
        raise RuntimeError("reference build failed:\n" + res.stdout + res.stderr)
    return out


def find_reference() -> Path | None:
    """The reference's source tree: ``$RBV_REFERENCE_DIR``, or a folder named ``reference`` beside this repository."""
    cands = []
    if os.environ.get("RBV_REFERENCE_DIR"):
        cands.append(Path(os.environ["RBV_REFERENCE_DIR"]))
    cands.append(HERE.parent.parent / "reference")
    for cand in cands:
        if (cand / "src" / "rbruckv.h").exists():
            return cand
    return None


def ensure_built() -> Path | None:
    """Path of the runner, building it from the copied sources when needed (and when the harness is newer than
    the binary); None if there is neither a copy nor a reference tree to copy from."""
    out = REF / "ref_runner"
    fresh = out.exists() and out.stat().st_mtime >= (HERE / "ref_runner.cpp").stat().st_mtime
    if fresh:
        return out
    if not (SRC_COPY / "src").exists():
        cand = find_reference()
        if cand is None:
            return out if out.exists() else None
        REF.mkdir(exist_ok=True)
        copy_sources(cand)
    return build()


def main():
    reference = Path(sys.argv[1]) if len(sys.argv) > 1 else find_reference()
    if reference is None:
        raise SystemExit("usage: install_reference.py <path of the reference tree>  (or set RBV_REFERENCE_DIR)")
    REF.mkdir(exist_ok=True)
    print(pip_attempt(reference))
    copy_sources(reference)
    print("built", build())


if __name__ == "__main__":
    main()
