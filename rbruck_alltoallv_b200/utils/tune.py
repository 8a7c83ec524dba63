"""Fill the tuner table by measurement on the machine at hand.

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m rbruck_alltoallv_b200.utils.tune [--nranks 8] [--skew both]

Writes the winners to the tuner cache (``$RBV_TUNER_CACHE`` or ``parallel/tuner_table.json``) and, with ``--out``,
all timings as JSON lines.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from ..parallel import tuner
from ..parallel.comm import Communicator


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--nranks", type=int, default=0)
    ap.add_argument("--skew", default="both", choices=["normal", "zipf", "both"])
    ap.add_argument("--steps", type=int, default=tuner.MIN_STEPS)
    ap.add_argument("--quick", action="store_true", help="one batch value per schedule instead of the 1, 2, 4, ... sweep")
    ap.add_argument("--sizes", default="16,256,4096,65536,1048576,4194304")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    comm = Communicator(nranks=a.nranks or max(world, 1), heap_bytes=2 << 30, arena_bytes=128 << 20)
    rows = []
    for skew in (["normal", "zipf"] if a.skew == "both" else [a.skew]):
        rows += tuner.sweep(comm, tuple(int(x) for x in a.sizes.split(",")), skew=skew, steps=a.steps, full=not a.quick,
                            verbose=False)
    if comm.proc == 0:
        tuner.save_table()
        if a.out:
            with open(a.out, "a") as fh:
                for r in rows:
                    fh.write(json.dumps(dict(r, P=comm.P, gpus=comm.nproc)) + "\n")
    comm.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
