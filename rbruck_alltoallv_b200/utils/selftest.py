"""Multi-process self test: every algorithm against the direct-copy expectation, one process per GPU.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 -m rbruck_alltoallv_b200.utils.selftest [--nranks P]

Each process checks its own ranks; the exit code is non-zero when any block differs.  With ``--bench`` it
also prints device-timed latencies next to NCCL's grouped send/recv for a few block sizes.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

from ..parallel.comm import Communicator
from . import distributions as D
from . import oracle
from .timing import L2Flusher, RankAligner, time_steps

CASES = [("linear", {}), ("spreadout", {}), ("scattered", dict(b=2)), ("pairwise", {}), ("xor", {}),
         ("merge", dict(n=2)), ("simple_merge", dict(n=2)), ("split", {}),
         ("rbruck", dict(r=2)), ("rbruck", dict(r=3)), ("rbruck_om", dict(r=2)), ("tuna", dict(r=2, b=1)),
         ("tuna2", dict(r=2, b=0)), ("ttpl", dict(n=2, r=2)), ("ttpl_bt", dict(n=2, r=2)),
         ("ttpl_bt_s1", dict(n=2, r=2, b=2)), ("ttpl_bt_s2", dict(n=2, r=2)),
         ("uniform_spreadout_twolayer", dict(n=2, r=2)), ("uniform_isplit_rbruck", dict(n=2, r=2, r2=2)),
         ("twolayer_linear", dict(n=2)), ("twolayer_linear_s2", dict(n=2, b=1, b2=2)),
         ("twolayer_linear_s3", dict(n=2, b=1, b2=1))]


def check_all(comm: Communicator, ts: int = 4, seed: int = 3) -> int:
    P, mine = comm.P, comm.local_ranks
    failures = ran = 0
    for ci, (algo, kw) in enumerate(CASES):
        if algo == "xor" and P & (P - 1):
            continue
        if kw.get("n") and (P % kw["n"] or (kw["n"] >= P and algo not in ("merge", "simple_merge"))):
            continue
        counts = D.uniform(P, 3000, seed=seed + ci)
        counts[counts < 200] = 0
        prob = oracle.make_problem(counts, ts, seed + ci, packed=(ci % 2 == 0))
        send_h = oracle.fill_send(prob, seed + ci)
        want = oracle.expected_recv(prob, send_h)
        send = [torch.from_numpy(send_h[r]).cuda() for r in mine]
        recv = [comm.symm_empty(len(want[r]), torch.uint8) for r in mine]
        for t in recv:
            t.fill_(oracle.CANARY)
        torch.cuda.synchronize()
        comm.host_barrier()
        emax = comm.max_block_bytes(prob.counts[mine], ts)
        inplace_algo = algo == "ttpl_bt_s2"
        wanted = [want[r] for r in mine]
        args = (send, recv, prob.counts[mine], prob.sdispls[mine], prob.recvcounts[mine], prob.rdispls[mine])
        # Every way a call can run, each checked on its own: one-shot rendezvous (metadata exchanged by the kernel),
        # one-shot eager, a persistent call (static kernel: everything resolved on the host) launched twice, and
        # eager again; back-to-back calls exercise both parities.
        for rep, mode in enumerate(("rendezvous", "eager", "static", "eager")):
            if mode == "eager" and (inplace_algo or algo == "split"):   # neither takes the eager protocol
                continue
            ran += 1
            for t in recv:
                t.fill_(oracle.CANARY)
            if mode == "static":
                call = comm.prepare(*args, algo=algo, type_size=ts, **kw)
                call.launch()
                call.launch()
            else:
                comm.alltoallv(*args, algo=algo, type_size=ts, eager_max_bytes=(emax if mode == "eager" else 0), **kw)
            st = comm.status()
            bad = oracle.first_mismatch([t.cpu().numpy() for t in recv], wanted)
            if st["code"] or bad is not None:
                failures += 1
                print(f"[proc {comm.proc}] FAIL {algo} {kw} ({mode}): status={st['name']}@{st['site']} {st['detail']} "
                      f"mismatch={bad}", flush=True)
            # a failure on any process resets all of them together (reset is collective)
            flag = torch.tensor([1 if (st["code"] or bad is not None) else 0], dtype=torch.int64)
            if comm._side is not None:
                comm._dist.all_reduce(flag, op=comm._dist.ReduceOp.MAX, group=comm._side)
            if int(flag.item()):
                comm.reset()
            if mode == "static":
                del call
        comm.host_barrier()
        del send, recv
    check_all.cases = ran
    return failures


def bench(comm: Communicator, sizes=(16, 1024, 65536, 1 << 20, 4 << 20), aligned: bool = False) -> list:
    P, L, mine = comm.P, comm.L, comm.local_ranks
    dev = f"cuda:{comm.device}"
    flush, align = L2Flusher(dev), RankAligner(comm)
    rows = []
    for nbytes in sizes:
        elems = max(1, nbytes // 2)
        counts = D.normal(P, elems, 0.25, seed=nbytes)
        if aligned:   # every block starts on a 16-byte boundary (8 bf16 elements)
            counts = (counts // 8) * 8
        sc = counts[mine].astype(np.int32)
        rc = counts.T[mine].astype(np.int32)
        send = [torch.zeros(max(int(sc[i].sum()), 1), dtype=torch.bfloat16, device=dev) for i in range(L)]
        recv = [comm.symm_empty(max(int(rc[i].sum()), 1), torch.bfloat16) for i in range(L)]
        row = {"mean_block_bytes": nbytes, "total_bytes": int(counts.sum()) * 2, "us": {}}
        emax = comm.max_block_bytes(sc, 2)
        cases = [("spreadout", dict(algo="spreadout")), ("rbruck_r2", dict(algo="rbruck", r=2)),
                 ("tuna2_r2", dict(algo="tuna2", r=2)), ("pairwise", dict(algo="pairwise"))]
        if nbytes >= (64 << 10):   # the two copy engines of the rendezvous protocol, side by side
            cases += [("spreadout_vector", dict(algo="spreadout", bulk=0)), ("spreadout_bulk", dict(algo="spreadout", bulk=1))]
            if comm.nproc == 1:
                cases += [("rbruck_r2_vector", dict(algo="rbruck", r=2, bulk=0)),
                          ("rbruck_r2_bulk", dict(algo="rbruck", r=2, bulk=1))]
        if emax <= (256 << 10):
            cases += [("spreadout_eager", dict(algo="spreadout", eager_max_bytes=emax)),
                      ("rbruck_r2_eager", dict(algo="rbruck", r=2, eager_max_bytes=emax))]
        for name, kw in cases:
            try:
                call = comm.prepare(send, recv, sc, None, rc, None, **kw)
            except Exception as e:  # noqa: BLE001
                row["us"][name] = f"n/a ({e})"
                continue
            t = time_steps(call.launch, steps=20, warmup=3, flush=flush, align=align)
            st = comm.status()
            if st["code"]:
                row["us"][name] = st["name"]
                comm.reset()
            else:
                row["us"][name] = round(float(np.median(t)) * 1e3, 2)
        if comm.nproc > 1 and L == 1:
            r1 = torch.empty(max(int(rc[0].sum()), 1), dtype=torch.bfloat16, device=dev)
            ns, nr = int(sc[0].sum()), int(rc[0].sum())
            ins, outs = [int(x) for x in sc[0]], [int(x) for x in rc[0]]
            fn = lambda: dist.all_to_all_single(r1[:nr], send[0][:ns], output_split_sizes=outs, input_split_sizes=ins)
            t = time_steps(fn, steps=20, warmup=3, flush=flush, align=align)
            row["us"]["nccl_grouped_sendrecv"] = round(float(np.median(t)) * 1e3, 2)
        rows.append(row)
        del send, recv
    return rows


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--nranks", type=int, default=0)
    ap.add_argument("--bench", action="store_true")
    ap.add_argument("--out", default="")
    ap.add_argument("--sizes", default="", help="comma-separated mean block sizes in bytes for --bench")
    ap.add_argument("--heap-mb", type=int, default=1024)
    ap.add_argument("--aligned", action="store_true", help="--bench with block sizes that are multiples of 16 bytes")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    comm = Communicator(nranks=args.nranks or max(world, 1), heap_bytes=args.heap_mb << 20, arena_bytes=64 << 20)
    failures = check_all(comm)
    if world > 1:
        f = torch.tensor([failures], device="cuda")
        dist.all_reduce(f)
        failures = int(f.item())
    sizes = tuple(int(x) for x in args.sizes.split(",")) if args.sizes else None
    rows = None
    if args.bench and failures == 0:
        rows = bench(comm, sizes, args.aligned) if sizes else bench(comm, aligned=args.aligned)
    if comm.proc == 0:
        line = {"selftest": "ok" if failures == 0 else "FAILED", "failures": failures, "P": comm.P, "gpus": comm.nproc,
                "nvls_metadata": bool(comm.nvls)}
        if rows is not None:
            line["bench"] = rows
        print(json.dumps(line), flush=True)
        if args.out:
            with open(args.out, "a") as fh:
                fh.write(json.dumps(line) + "\n")
    comm.close()
    if world > 1:
        dist.destroy_process_group()
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())
