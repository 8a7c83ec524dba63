"""Check and time the fused pencil transposes (optionally next to the NCCL baseline).

    python -m rbruck_alltoallv_b200.utils.fft_bench --size 256 --check
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m rbruck_alltoallv_b200.utils.fft_bench --size 1024 --pr 2 --pc 4
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

from ..ops.fft import PencilTranspose
from ..parallel.comm import Communicator
from .timing import L2Flusher, time_steps


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", dest="n", type=int, default=256, help="grid points per dimension")
    ap.add_argument("--pr", type=int, default=0)
    ap.add_argument("--pc", type=int, default=0)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check", action="store_true", help="element-exact check and a full 3-D FFT against torch.fft.fftn")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    pr = a.pr or (2 if world % 2 == 0 and world > 1 else 1)
    pc = a.pc or world // pr
    n = a.n
    per_rank = (n ** 3 * 8) // world
    comm = Communicator(nranks=world, heap_bytes=int(2.3 * per_rank) + (64 << 20), arena_bytes=1 << 20)
    tp = PencilTranspose(comm, n, pr, pc, seed=11)
    dev = f"cuda:{comm.device}"
    res = {"n": n, "gpus": world, "grid": [pr, pc], "dtype": "complex64"}
    ok = True
    if a.check:
        g = torch.Generator(device=dev)
        g.manual_seed(5)   # the same full array on every rank
        full = torch.view_as_complex(torch.randn(n, n, n, 2, device=dev, generator=g))
        xp = tp.local_x_pencil_of(full)
        y = tp.x_to_y(xp)
        torch.cuda.synchronize()
        ok &= bool(torch.equal(y, tp.expected_y(full)))
        z = tp.y_to_z(y.clone())
        torch.cuda.synchronize()
        ok &= bool(torch.equal(z, tp.expected_z(full)))
        # distributed FFT: x (local), transpose, y, transpose, z
        fx = torch.fft.fft(xp, dim=2)
        fy = torch.fft.fft(tp.x_to_y(fx.contiguous()), dim=2)
        fz = torch.fft.fft(tp.y_to_z(fy.contiguous()), dim=2)
        want = tp.expected_z(torch.fft.fftn(full))
        err = (fz - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
        res["fft_rel_err"] = err
        ok &= err < 1e-4
        tp.check()
        res["check"] = "ok" if ok else "FAILED"
        del full
    src_x = torch.view_as_complex(torch.randn(*tp.shape_x, 2, device=dev))
    src_y = torch.view_as_complex(torch.randn(*tp.shape_y, 2, device=dev))
    flush = L2Flusher(dev)
    t_xy = time_steps(lambda: tp.x_to_y(src_x), a.steps, a.warmup, flush=flush)
    t_yz = time_steps(lambda: tp.y_to_z(src_y), a.steps, a.warmup, flush=flush)
    tp.check()
    total, remote = tp.bytes_sent_xy()
    ms_xy, ms_yz = float(np.median(t_xy)), float(np.median(t_yz))
    res.update({"ms_x_to_y": ms_xy, "ms_y_to_z": ms_yz, "bytes_per_gpu": total, "bytes_leaving_gpu_xy": remote,
                "GBps_per_gpu_xy": total / ms_xy / 1e6, "nvlink_fraction_xy_of_770": remote / ms_xy / 1e6 / 770.0})
    if world > 1:
        col_groups = [dist.new_group([r * pc + c for r in range(pr)]) for c in range(pc)]
        grp = col_groups[tp.me_c]
        t_n = time_steps(lambda: tp.nccl_x_to_y(src_x, grp), a.steps, a.warmup, flush=flush)
        res["ms_x_to_y_nccl_pack_unpack"] = float(np.median(t_n))
    if comm.proc == 0:
        print(json.dumps(res), flush=True)
        if a.out:
            with open(a.out, "a") as fh:
                fh.write(json.dumps(res) + "\n")
    comm.close()
    if world > 1:
        dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
