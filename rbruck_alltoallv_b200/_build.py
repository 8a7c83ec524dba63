"""In-tree native builds.

Two shared libraries are produced beside this file:

* ``librbv_host.so``  -- plan compiler + CPU executor (g++, no CUDA dependency),
* ``librbv_cuda.so``  -- communicator, kernels and the C API (nvcc, sm_100a only).

A library is rebuilt only when the hash of its sources and flags changes; the hash is kept in a
``.stamp`` file next to the library so that a tree copied to another machine is not rebuilt.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = CSRC / "include"

HOST_SOURCES = ["plan/plan.cpp", "plan/capi_host.cpp", "api/tuner_native.cpp"]
CUDA_SOURCES = [
    "plan/plan.cpp",
    "plan/capi_host.cpp",
    "comm/comm.cu",
    "kernels/a2av_kernel.cu",
    "kernels/a2av_eager.cu",
    "kernels/a2av_static.cu",
    "kernels/moe_kernels.cu",
    "kernels/grouped_gemm_sm100.cu",
    "kernels/grouped_gemm_pair_sm100.cu",
    "kernels/grouped_gemm_fp8_sm100.cu",
    "kernels/grouped_gemm_fp8_pair_sm100.cu",
    "kernels/grouped_gemm_mxfp8_sm100.cu",
    "kernels/fft_transpose.cu",
    "kernels/noalloc.cu",
    "api/c_api.cu",
    "api/tuner_native.cpp",
    "api/drivers.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-shared",
    "-Xcompiler", "-Wall",
    "--expt-relaxed-constexpr",
]
GXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-Wall"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def _hash(files, flags) -> str:
    h = hashlib.sha256()
    for f in sorted(files):
        h.update(str(f.relative_to(PKG)).encode())
        h.update(f.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _headers():
    return sorted(list(INCLUDE.rglob("*.h")) + list(CSRC.rglob("*.cuh")))


def _needs_build(lib: Path, digest: str) -> bool:
    stamp = lib.with_suffix(".stamp")
    return not (lib.exists() and stamp.exists() and stamp.read_text().strip() == digest)


def _run(cmd, verbose):
    if verbose:
        print("[rbv build]", " ".join(str(c) for c in cmd), file=sys.stderr, flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("native build failed:\n" + " ".join(map(str, cmd)) + "\n" + res.stdout + res.stderr)
    if verbose and (res.stdout or res.stderr):
        print(res.stdout + res.stderr, file=sys.stderr)
    return res.stdout + res.stderr


def build_host(force: bool = False, verbose: bool = False) -> Path:
    lib = PKG / "librbv_host.so"
    srcs = [CSRC / s for s in HOST_SOURCES]
    digest = _hash(srcs + _headers(), GXX_FLAGS)
    if force or _needs_build(lib, digest):
        tmp = lib.with_suffix(f".tmp{os.getpid()}.so")
        _run(["g++", *GXX_FLAGS, f"-I{INCLUDE}", *map(str, srcs), "-o", str(tmp)], verbose)
        os.replace(tmp, lib)
        lib.with_suffix(".stamp").write_text(digest)
    return lib


def cuda_sources():
    return [CSRC / s for s in CUDA_SOURCES if (CSRC / s).exists()]


def _compile_one(args):
    src, obj, flags, verbose = args
    return _run([_nvcc(), *flags, "-c", f"-I{INCLUDE}", f"-I{CSRC}", str(src), "-o", str(obj)], verbose)


def build_cuda(force: bool = False, verbose: bool = False, ptxas_verbose: bool = False) -> Path:
    """Compiles every source to an object of its own (in parallel; an object is kept while its source, the headers
    and the flags are unchanged) and links them into ``librbv_cuda.so``."""
    from concurrent.futures import ThreadPoolExecutor

    lib = PKG / "librbv_cuda.so"
    srcs = cuda_sources()
    flags = [f for f in NVCC_FLAGS if f != "-shared"]
    if ptxas_verbose:
        flags += ["-Xptxas", "-v"]
    digest = _hash(srcs + _headers(), flags)
    if force or _needs_build(lib, digest):
        objdir = PKG / "_obj"
        objdir.mkdir(exist_ok=True)
        heads = _headers()
        jobs, objs = [], []
        for src in srcs:
            obj = objdir / (src.stem + ".o")
            d = _hash([src] + heads, flags)
            stamp = obj.with_suffix(".stamp")
            objs.append(obj)
            if force or not (obj.exists() and stamp.exists() and stamp.read_text().strip() == d):
                jobs.append((src, obj, flags, verbose, stamp, d))
        with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
            outs = list(pool.map(_compile_one, [j[:4] for j in jobs]))
        for j in jobs:
            j[4].write_text(j[5])
        tmp = lib.with_suffix(f".tmp{os.getpid()}.so")
        _run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *map(str, objs), "-o", str(tmp)],
             verbose)
        os.replace(tmp, lib)
        lib.with_suffix(".stamp").write_text(digest)
        if ptxas_verbose:
            print("".join(outs))
    return lib


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_host(force, verbose)
    build_cuda(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
