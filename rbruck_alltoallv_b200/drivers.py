"""Benchmark drivers: one sub-command per driver program of the reference (its ``examples/`` and
``benchmarks/`` folders), printing the same tagged lines (``[Rbruckv] P, n, b, base, seconds`` ...) plus,
optionally, one JSON line per measurement.

    python -m rbruck_alltoallv_b200.drivers rbruckv 20 2 4 8 --nranks 8
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m rbruck_alltoallv_b200.drivers LTRNA 20 4 2

Single process: all ``--nranks`` logical ranks run on one GPU.  Under torchrun: one rank per GPU.

Reference drivers covered (file in the reference -> sub-command): rbruckv_example -> ``rbruckv``;
twolayer_example -> ``twolayer``; twophaseLayer_example -> ``combAlltoallv``; twophaseLayer_example2 -> ``LTRNA``;
twophaseLayer_example3 -> ``TTPL``; twophaseLayer_example4 -> ``TLLiner_S2``; twophaseLayer_example5 -> ``TLLiner_S3``;
MLinputs_example -> ``MLinputs``; FFT_distribution -> ``FFT``; other_distributions -> ``otherDis``;
balanced_benchmark -> ``balance``; gather_benchmark -> ``gather``; benchmarks/intra_node_comm -> ``intra_node_comm``;
benchmarks/split_benchmark -> ``split``; benchmarks/merge_benchmark and simple_merge_benchmark -> ``merge``
(leader-based exchange expressed as a two-layer alltoallv).  mpich_twolayer_alltoall and ms_benchmark are toy /
empty programs in the reference and map to ``twolayer`` with n = 1.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

import numpy as np
import torch

from .parallel.comm import Communicator
from .utils import distributions as D
from .utils.timing import L2Flusher, RankAligner, time_steps


def _comm(args) -> Communicator:
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    nranks = args.nranks or max(world, 1)
    return Communicator(nranks=nranks, heap_bytes=args.heap_mb << 20, arena_bytes=args.arena_mb << 20)


def _native_sweep(comm, tag, algo, args, n_group=0, radix=2, b=0, b2=0, nmin=2, nmax=2048, mode=0):
    lib = comm._lib
    lib.rbv_driver_sweep.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p] + [C.c_int] * 9 + [C.c_ulonglong, C.c_char_p]
    lib.rbv_ctx_set_stream(comm._ctx, C.c_void_p(torch.cuda.current_stream(comm.device).cuda_stream))
    return lib.rbv_driver_sweep(comm._ctx, tag.encode(), algo.encode(), args.loop, args.warmup, n_group, radix, b, b2,
                                nmin, min(nmax, args.nmax), mode, args.seed, b"")


def _timed(comm, tag, counts, ts, args, extra="", **kw):
    """Times one alltoallv configuration on a count matrix (elements of ts bytes); prints a tagged line."""
    L, P, mine = comm.L, comm.P, comm.local_ranks
    dev = f"cuda:{comm.device}"
    sc = counts[mine].astype(np.int32)
    rc = counts.T[mine].astype(np.int32)
    send = [torch.zeros(max(int(sc[i].sum()), 1) * ts, dtype=torch.uint8, device=dev) for i in range(L)]
    recv = [comm.symm_empty(max(int(rc[i].sum()), 1) * ts, torch.uint8) for i in range(L)]
    call = comm.prepare(send, recv, sc, None, rc, None, type_size=ts, **kw)
    t = time_steps(call.launch, args.loop, args.warmup, flush=_timed.flush, align=_timed.align)
    st = comm.status()
    sec = float(np.mean(t)) * 1e-3
    if comm.proc == 0:
        if st["code"]:
            print(f"[{tag}] {P}, {extra} failed: {st['name']}")
        else:
            print(f"[{tag}] {P}, {extra}{sec:.9f}")
        if args.jsonl:
            with open(args.jsonl, "a") as fh:
                fh.write(json.dumps({"tag": tag, "P": P, "gpus": comm.nproc, "params": kw, "extra": extra,
                                     "total_bytes": int(counts.sum()) * ts, "us": sec * 1e6,
                                     "status": st["name"]}) + "\n")
    if st["code"]:
        comm.reset()
    return sec


def _sizes(lo, hi):
    n = lo
    while n <= hi:
        yield n
        n *= 2


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="rbruck_alltoallv_b200.drivers")
    ap.add_argument("driver")
    ap.add_argument("params", nargs="*", help="positional parameters of the reference driver (loop count first)")
    ap.add_argument("--nranks", type=int, default=0)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--nmax", type=int, default=2048)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--heap-mb", type=int, default=2048)
    ap.add_argument("--arena-mb", type=int, default=64)
    ap.add_argument("--jsonl", default="")
    ap.add_argument("--input", default="", help="count matrix file for MLinputs")
    args = ap.parse_args(argv)
    p = args.params
    args.loop = int(p[0]) if p and p[0].lstrip("-").isdigit() else 10
    comm = _comm(args)
    P = comm.P
    _timed.flush = L2Flusher(f"cuda:{comm.device}")
    _timed.align = RankAligner(comm)
    # the reference's CMake target and file names are accepted too
    aliases = {"merge_benckmark": "merge", "merge_benchmark": "merge", "simple_merge_benchmark": "merge",
               "simply_merge": "merge", "split_benchmark": "split", "balanced_benchmark": "balance",
               "gather_benchmark": "gather", "mpich_twolayer_alltoall": "twolayer", "ms_benchmark": "twolayer",
               "rbruckv_example": "rbruckv", "twolayer_example": "twolayer", "twophaseLayer_example": "combAlltoallv",
               "twophaseLayer_example2": "LTRNA", "twophaseLayer_example3": "TTPL", "twophaseLayer_example4": "TLLiner_S2",
               "twophaseLayer_example5": "TLLiner_S3", "MLinputs_example": "MLinputs", "FFT_distribution": "FFT",
               "other_distributions": "otherDis"}
    drv = aliases.get(args.driver, args.driver)
    if args.driver in ("mpich_twolayer_alltoall", "ms_benchmark"):
        p = [p[0] if p else "10", "1"] + list(p[1:])       # toy programs of the reference: one rank per group
        args.nmax = min(args.nmax, 2)
    ints = [int(v) for v in p[1:] if v.lstrip("-").isdigit()]
    fails = 0
    if drv == "rbruckv":                       # <loop> <bases...>
        for base in (ints or [2]):
            fails += max(0, _native_sweep(comm, "Rbruckv", "tuna2", args, radix=base, b=1))
    elif drv == "twolayer":                    # <loop> <ncores> <bases...>
        n = ints[0] if ints else max(1, P // 2)
        for base in (ints[1:] or [2]):
            for cnt in _sizes(2, args.nmax):
                c = D.constant(P, cnt)
                _timed(comm, "SOR_alltoall", c, 8, args, f"{cnt}, {base}, ", algo="uniform_spreadout_twolayer", n=n, r=base)
                _timed(comm, "BR_alltoall", c, 8, args, f"{cnt}, {base}, ", algo="uniform_isplit_rbruck", n=n, r=base, r2=base)
    elif drv == "combAlltoallv":               # <loop> <ncores> <bases...>
        b = 1
        while b <= P:
            fails += max(0, _native_sweep(comm, "MPICH_scattered", "scattered", args, b=b, mode=1))
            b *= 2
        fails += max(0, _native_sweep(comm, "OMPI_linear", "linear", args, mode=1))
        fails += max(0, _native_sweep(comm, "OMPI_pairwise", "pairwise", args, mode=1))
        if P & (P - 1) == 0:
            fails += max(0, _native_sweep(comm, "ExcOr", "xor", args, mode=1))
    elif drv in ("LTRNA", "TTPL"):             # <loop> <ncores> <bases...>
        n = ints[0] if ints else max(1, P // 2)
        for base in (ints[1:] or [2]):
            if drv == "TTPL":
                fails += max(0, _native_sweep(comm, "TTPL_S2", "ttpl_bt_s2", args, n_group=n, radix=base, nmin=4, nmax=4, mode=1))
                continue
            b = 1
            while b <= max(1, P // n):
                fails += max(0, _native_sweep(comm, "TTPL", "ttpl_bt", args, n_group=n, radix=base, b=b, nmax=1024, mode=1))
                b *= 2
            b = 1
            while b <= P:
                fails += max(0, _native_sweep(comm, "TTPL_S1", "ttpl_bt_s1", args, n_group=n, radix=base, b=b, nmax=1024, mode=1))
                b *= 2
    elif drv in ("TLLiner_S2", "TLLiner_S3"):  # <loop> <ncores>
        algo = "twolayer_linear_s2" if drv == "TLLiner_S2" else "twolayer_linear_s3"
        fails += max(0, _native_sweep(comm, "MPICH_scattered", "scattered", args, b=P, mode=1))
        for nc in [g for g in (2, 4, 8, 16, 32, 64) if g < P and P % g == 0]:
            fails += max(0, _native_sweep(comm, drv, algo, args, n_group=nc, b=nc, b2=P, mode=1))
    elif drv == "MLinputs":                    # --input <matrix file> <loop> <bases...>
        counts = D.read_matrix(args.input) if args.input else D.synthetic_ml_trace(P, args.seed, mean_bytes=4e6)
        if counts.shape[0] != P:
            raise SystemExit(f"matrix is {counts.shape[0]} x {counts.shape[0]} but the communicator has {P} ranks")
        _timed(comm, "Spread-out", counts, 1, args, "", algo="spreadout")
        for base in (ints or [2]):
            _timed(comm, "TUNA,", counts, 1, args, f"{base}, ", algo="rbruck", r=base)
    elif drv == "FFT":   # <loop> <ncores> <bblock1> <radix1> <bblock2> <radix2> <xzero> <yzero> <number> <last>
        n = ints[0] if ints else max(1, P // 2)
        b1, r1, b2, r2 = (ints[1:5] + [0, 2, 0, 2])[:4] if len(ints) >= 5 else (0, 2, 0, 2)
        fl = [float(v) for v in p[6:8]] if len(p) >= 8 else [0.0, 0.0]
        number = int(p[8]) if len(p) > 8 else 1024
        last = int(p[9]) if len(p) > 9 else 0
        c = D.fft_pattern(P, number, fl[0], fl[1], last)
        _timed(comm, "Spread-out", c, 8, args, "", algo="spreadout")
        _timed(comm, "TTPL_S1", c, 8, args, f"{b1}, {r1}, ", algo="ttpl_bt_s1", n=n, r=r1, b=b1)
        _timed(comm, "TTPL", c, 8, args, f"{b2}, {r2}, ", algo="ttpl_bt", n=n, r=r2, b=b2)
    elif drv == "otherDis":  # <loop> <ncores> <bblock1> <radix1> <bblock2> <radix2> <dist> <mean> <dev> <x> <max> <radix0>
        n = ints[0] if ints else max(1, P // 2)
        dist_id = int(p[6]) if len(p) > 6 else 0
        mean = float(p[7]) if len(p) > 7 else 512
        devi = float(p[8]) if len(p) > 8 else 128
        x = float(p[9]) if len(p) > 9 else 0.9
        mx = int(p[10]) if len(p) > 10 else 4096
        r0 = int(p[11]) if len(p) > 11 else 2
        c = D.normal(P, mean, devi / max(mean, 1e-9), args.seed, max_value=mx) if dist_id == 0 else D.power_law(P, mx, x, args.seed)
        _timed(comm, "Spread-out", c, 8, args, "", algo="spreadout")
        _timed(comm, "TUNA", c, 8, args, f"{r0}, ", algo="rbruck", r=r0)
        _timed(comm, "TTPL_S1", c, 8, args, "", algo="ttpl_bt_s1", n=n, r=2)
        _timed(comm, "TTPL", c, 8, args, "", algo="ttpl_bt", n=n, r=2)
    elif drv in ("balance", "gather", "merge"):   # <loop> <ncores>
        n = ints[0] if ints else max(1, P // 2)
        for cnt in _sizes(2, min(args.nmax, 4096)):
            if drv == "balance":
                _timed(comm, "balance", D.sparse_groups(P, cnt, n), 8, args, f"{cnt}, ", algo="spreadout")
                _timed(comm, "balance_T", D.sparse_groups(P, cnt, n, True), 8, args, f"{cnt}, ", algo="spreadout")
            else:
                _timed(comm, "Spread-out", D.constant(P, cnt), 8, args, f"{cnt}, ", algo="spreadout")
                if P % n == 0 and n < P:
                    _timed(comm, "Merge" if drv == "merge" else "gather", D.constant(P, cnt), 8, args, f"{cnt}, ",
                           algo="ttpl_bt", n=n, r=2)
    elif drv == "intra_node_comm":
        cnt = 1
        while cnt <= 10 ** 6:
            _timed(comm, "intra_node_comm", D.constant(P, cnt), 1, args, f"{cnt}, ", algo="spreadout")
            cnt *= 10
    elif drv == "split":                       # one huge block rank 0 -> rank P-1
        lsize = int(p[1]) if len(p) > 1 else 1 << 24
        c = np.zeros((P, P), dtype=np.int64)
        c[0, P - 1] = lsize
        _timed(comm, "Spread-out", c, 1, args, f"{lsize}, ", algo="spreadout")
        _timed(comm, "Split", c, 1, args, f"{lsize}, ", algo="spreadout", chunk_bytes=max(4096, lsize // max(P, 1) // 16 * 16))
    else:
        raise SystemExit(f"unknown driver {drv}")
    comm.close()
    return 1 if fails else 0


if __name__ == "__main__":
    sys.exit(main())
