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
benchmarks/split_benchmark -> ``split``; benchmarks/merge_benchmark -> ``merge``; benchmarks/simple_merge_benchmark ->
``simple_merge``.  mpich_twolayer_alltoall and ms_benchmark are toy / empty programs in the reference and map to
``twolayer`` with n = 1.

Where the reference times the vendor's ``MPI_Alltoallv`` next to its own algorithms and prints ``[MPIAlltoallv]``
(examples/twophaseLayer_example.cpp:99-113, twophaseLayer_example2.cpp:197-211, MLinputs_example.cpp:74-82), these
drivers time NCCL's grouped send/recv on the same counts and print ``[NCCLAlltoallv]`` (one rank per GPU only: NCCL
has one rank per process).  With ``--jsonl`` every measurement is also written as a record with per-rank algbw,
busbw and the fraction of the NVLink roofline (``utils/metrics.py``).
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
from .parallel.plan import Plan
from .utils import distributions as D
from .utils.metrics import alltoallv_row
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
    nccl = kw.pop("nccl", False)
    if nccl:
        if comm.nproc < 2 or L != 1:
            return None
        import torch.distributed as dist
        dt = {1: torch.uint8, 2: torch.bfloat16, 4: torch.float32, 8: torch.float64}[ts]
        s1, r1 = send[0].view(dt), recv[0].view(dt)
        ns, nr = int(sc[0].sum()), int(rc[0].sum())
        ins, outs = [int(x) for x in sc[0]], [int(x) for x in rc[0]]
        fn = lambda: dist.all_to_all_single(r1[:nr], s1[:ns], output_split_sizes=outs, input_split_sizes=ins)
        t = time_steps(fn, args.loop, args.warmup, flush=_timed.flush, align=_timed.align)
        st, kind, ops = {"code": 0, "name": "ok"}, "nccl", None
    else:
        call = comm.prepare(send, recv, sc, None, rc, None, type_size=ts, **kw)
        t = time_steps(call.launch, args.loop, args.warmup, flush=_timed.flush, align=_timed.align)
        st, kind = comm.status(), call.kind
        pk = {k: v for k, v in kw.items() if k in ("n", "r", "r2", "b", "b2")}
        ops = Plan(kw.get("algo", "spreadout"), P, **pk).ops()
    sec = float(np.mean(t)) * 1e-3
    if comm.proc == 0:
        if st["code"]:
            print(f"[{tag}] {P}, {extra} failed: {st['name']}")
        else:
            print(f"[{tag}] {P}, {extra}{sec:.9f}")
        if args.jsonl:
            rec = {"tag": tag, "P": P, "gpus": comm.nproc, "params": kw, "extra": extra, "kernel": kind,
                   "total_bytes": int(counts.sum()) * ts, "status": st["name"]}
            rec.update(alltoallv_row(counts, ts, sec * 1e6, ops, L))
            with open(args.jsonl, "a") as fh:
                fh.write(json.dumps(rec) + "\n")
    if st["code"]:
        comm.reset()
    return sec


def _vendor(comm, counts, ts, args, extra=""):
    """The vendor baseline line: NCCL grouped send/recv where the reference prints [MPIAlltoallv]."""
    return _timed(comm, "NCCLAlltoallv", counts, ts, args, extra, nccl=True)


def _breakdown(comm, tag):
    """Prints the phase timers of the most recent traced call the way the reference's LTRNA / TLLiner_S2 drivers do
    (examples/twophaseLayer_example2.cpp:119-128, twophaseLayer_example4.cpp): one line of seconds per name."""
    lib = comm._lib
    lib.rbv_ctx_set_stream(comm._ctx, C.c_void_p(torch.cuda.current_stream(comm.device).cuda_stream))
    lib.rbv_update_timers(comm._ctx)
    names = ["init_time", "findMax_time", "rotateIndex_time", "alcCopy_time", "getBlock_time", "prepData_time",
             "excgMeta_time", "excgData_time", "replace_time", "orgData_time", "prepSP_time", "SP_time", "intra_time"]
    vals = [C.c_double.in_dll(lib, n).value for n in names]
    nb = lib.rbv_iteration_count(comm._ctx)
    it = C.POINTER(C.c_double).in_dll(lib, "iteration_time")
    iters = [it[i] for i in range(nb)] if nb and it else []
    if it:
        C.CDLL(None).free(it)
    if comm.proc == 0:
        print(f"[{tag}-timers] " + ", ".join(f"{n}={v:.9f}" for n, v in zip(names, vals)))
        if iters:
            print(f"[{tag}-iteration_time] " + ", ".join(f"{v:.9f}" for v in iters))


def _traced(comm, tag, counts, ts, args, extra="", **kw):
    """One configuration timed like the others, then once more with the phase stamps on, for the breakdown."""
    sec = _timed(comm, tag, counts, ts, args, extra, **kw)
    L, mine = comm.L, comm.local_ranks
    sc, rc = counts[mine].astype(np.int32), counts.T[mine].astype(np.int32)
    dev = f"cuda:{comm.device}"
    send = [torch.zeros(max(int(sc[i].sum()), 1) * ts, dtype=torch.uint8, device=dev) for i in range(L)]
    recv = [comm.symm_empty(max(int(rc[i].sum()), 1) * ts, torch.uint8) for i in range(L)]
    comm.enable_trace(True)
    call = comm.prepare(send, recv, sc, None, rc, None, type_size=ts, **kw)
    call.launch()
    call.launch()
    _breakdown(comm, tag)
    comm.enable_trace(False)
    return sec


def _reference_input(P):
    """The reference's recorded count matrix for P ranks (inputs/<P>proc/global_comm_pattern_<P>proc.txt), looked for
    in $RBV_REFERENCE_DIR, beside this repository, and in the copy the baseline install keeps; None if absent."""
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cands = [Path(os.environ["RBV_REFERENCE_DIR"])] if os.environ.get("RBV_REFERENCE_DIR") else []
    cands += [root.parent / "reference", root / "baseline" / "_ref" / "reference"]
    for c in cands:
        f = c / "inputs" / f"{P}proc" / f"global_comm_pattern_{P}proc.txt"
        if f.exists():
            return f
    return None


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
    aliases = {"merge_benckmark": "merge", "merge_benchmark": "merge", "simple_merge_benchmark": "simple_merge",
               "simply_merge": "simple_merge", "split_benchmark": "split", "balanced_benchmark": "balance",
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
        for cnt in _sizes(2, args.nmax):
            _vendor(comm, D.uniform_fraction(P, cnt, args.seed + cnt), 8, args, f"{cnt}, ")
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
            for cnt in _sizes(2, min(args.nmax, 1024)):
                c = D.uniform_fraction(P, cnt, args.seed + cnt)
                _vendor(comm, c, 8, args, f"{cnt}, ")
                if cnt == min(args.nmax, 1024):      # the 12-timer breakdown of the reference's driver, once per base
                    _traced(comm, "TTPL", c, 8, args, f"{cnt}, 0, {base}, ", algo="ttpl_bt", n=n, r=base, b=0)
                    _traced(comm, "TTPL_S1", c, 8, args, f"{cnt}, 0, {base}, ", algo="ttpl_bt_s1", n=n, r=base, b=0)
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
        for cnt in _sizes(2, args.nmax):
            _vendor(comm, D.uniform_fraction(P, cnt, args.seed + cnt), 8, args, f"{cnt}, ")
        fails += max(0, _native_sweep(comm, "MPICH_scattered", "scattered", args, b=P, mode=1))
        for nc in [g for g in (2, 4, 8, 16, 32, 64) if g < P and P % g == 0]:
            fails += max(0, _native_sweep(comm, drv, algo, args, n_group=nc, b=nc, b2=P, mode=1))
            # intra_time and iteration_time[] per inter-group batch, as the reference's driver prints them
            c = D.uniform_fraction(P, min(args.nmax, 2048), args.seed)
            _traced(comm, drv, c, 8, args, f"{min(args.nmax, 2048)}, {nc}, ", algo=algo, n=nc, b=nc, b2=max(1, P // 4))
    elif drv == "MLinputs":                    # --input <matrix file> <loop> <bases...>
        path = args.input or _reference_input(P)
        counts = D.read_matrix(path) if path else D.synthetic_ml_trace(P, args.seed, mean_bytes=4e6)
        if comm.proc == 0:
            print(f"[MLinputs] count matrix: {path or 'synthetic trace (no recorded matrix for this rank count found)'}")
        if counts.shape[0] != P:
            raise SystemExit(f"matrix is {counts.shape[0]} x {counts.shape[0]} but the communicator has {P} ranks")
        _vendor(comm, counts, 1, args)
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
        _vendor(comm, c, 8, args)
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
        _vendor(comm, c, 8, args)
        _timed(comm, "Spread-out", c, 8, args, "", algo="spreadout")
        _timed(comm, "TUNA", c, 8, args, f"{r0}, ", algo="rbruck", r=r0)
        _timed(comm, "TTPL_S1", c, 8, args, "", algo="ttpl_bt_s1", n=n, r=2)
        _timed(comm, "TTPL", c, 8, args, "", algo="ttpl_bt", n=n, r=2)
    elif drv == "balance":                     # <loop> <ncores>: send only to every ncores-th rank, and the transpose
        n = ints[0] if ints else max(1, P // 2)
        for cnt in _sizes(2, min(args.nmax, 4096)):
            for tag, c in (("balance", D.sparse_groups(P, cnt, n)), ("balance_T", D.sparse_groups(P, cnt, n, True))):
                _vendor(comm, c, 8, args, f"{cnt}, ")
                _timed(comm, tag, c, 8, args, f"{cnt}, ", algo="spreadout")
    elif drv == "gather":                      # <loop> <ncores>: uniform exchange vs leaders-only exchange of n * ncores
        n = ints[0] if ints else max(1, P // 2)
        for cnt in _sizes(2, min(args.nmax, 4096)):
            uni, lead = D.constant(P, cnt), D.leaders_only(P, cnt * n, n)
            _vendor(comm, uni, 8, args, f"{cnt}, ")
            _timed(comm, "Alltoallv-1", uni, 8, args, f"{cnt}, ", algo="spreadout")
            _vendor(comm, lead, 8, args, f"{cnt}, ")
            _timed(comm, "Alltoallv-2", lead, 8, args, f"{cnt}, ", algo="spreadout")
    elif drv == "merge":                       # <loop> <ncores> <csize> <lsize>: small blocks, large ones from local rank 0
        n = ints[0] if ints else max(1, P // 2)
        csize = ints[1] if len(ints) > 1 else 16
        lsize = ints[2] if len(ints) > 2 else 16384
        c = D.merge_pattern(P, csize, lsize, n)
        _vendor(comm, c, 8, args, f"{csize}, {lsize}, ")
        _timed(comm, "Spread-out", c, 8, args, f"{csize}, {lsize}, ", algo="spreadout")
        if P % n == 0:
            _traced(comm, "Merge", c, 8, args, f"{csize}, {lsize}, ", algo="merge", n=n)
    elif drv == "simple_merge":                # <loop> <ncores>: uniform blocks through the group leaders
        n = ints[0] if ints else max(1, P // 2)
        for cnt in _sizes(2, min(args.nmax, 4096)):
            c = D.constant(P, cnt)
            _vendor(comm, c, 8, args, f"{cnt}, ")
            _timed(comm, "Spread-out", c, 8, args, f"{cnt}, ", algo="spreadout")
            if P % n == 0:
                # gather_time / ata_time / scatter_time of the reference = phases 1 / 2 / 3 of the schedule
                (_traced if cnt == min(args.nmax, 4096) else _timed)(comm, "simply_merge", c, 8, args, f"{cnt}, ",
                                                                     algo="simple_merge", n=n)
    elif drv == "intra_node_comm":
        cnt = 1
        while cnt <= 10 ** 6:
            _timed(comm, "intra_node_comm", D.constant(P, cnt), 1, args, f"{cnt}, ", algo="spreadout")
            cnt *= 10
    elif drv == "split":                       # <loop> <csize> <lsize>: one huge block rank 0 -> rank P-1 among small ones
        csize = int(p[1]) if len(p) > 1 else 16
        lsize = int(p[2]) if len(p) > 2 else 1 << 21
        c = np.full((P, P), csize, dtype=np.int64)
        c[0, P - 1] = lsize
        _vendor(comm, c, 8, args, f"{csize}, {lsize}, ")
        _timed(comm, "Spread-out", c, 8, args, f"{csize}, {lsize}, ", algo="spreadout")
        _timed(comm, "Split", c, 8, args, f"{csize}, {lsize}, ", algo="split")
    else:
        raise SystemExit(f"unknown driver {drv}")
    comm.close()
    return 1 if fails else 0


if __name__ == "__main__":
    sys.exit(main())
