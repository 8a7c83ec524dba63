"""Failure handling across processes, without faulting a GPU.  Run under torchrun with 2 or more processes.

Scenario (every failure is made on the host, between calls, with no kernel of the leaving process in flight):

1. a normal alltoallv (checked against the oracle);
2. the last process silently skips the next call: the others' kernels wait for its metadata until the device-side
   deadline, report ``timeout`` at the metadata phase and return normally (the CUDA context stays usable);
3. everybody resets the communicator (collective) and repeats the call successfully;
4. the last process announces in the job's store that it leaves; the others see it on the host before launching
   and refuse to launch (no device time spent);
5. it returns, and a final call succeeds.

The reference has no failure handling beyond MPI error codes (src/MPICH_scattered.cpp:51,63,69).
"""
from __future__ import annotations

import json
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

from ..parallel.comm import CommError, Communicator
from . import distributions as D
from . import oracle


def main() -> int:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world < 2:
        raise SystemExit("run under torchrun with at least 2 processes")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    comm = Communicator(nranks=world, heap_bytes=64 << 20, arena_bytes=1 << 20, timeout_ms=300.0)
    me, last = comm.proc, world - 1
    counts = D.uniform(world, 2000, seed=5)
    prob = oracle.make_problem(counts, 4, 5, packed=True)
    send_h = oracle.fill_send(prob, 5)
    want = oracle.expected_recv(prob, send_h)
    send = torch.from_numpy(send_h[me]).cuda()
    recv = comm.symm_empty(len(want[me]), torch.uint8)
    args = (prob.counts[me], prob.sdispls[me], prob.recvcounts[me], prob.rdispls[me])
    log = {}

    def exchange():
        recv.fill_(oracle.CANARY)
        comm.alltoallv(send, recv, *args, algo="spreadout", type_size=4)
        st = comm.status()
        return st, bool(np.array_equal(recv.cpu().numpy(), want[me]))

    st, ok = exchange()
    log["1_normal"] = {"status": st["name"], "data_ok": ok}

    # 2. the last process never joins
    comm.host_barrier()
    if me != last:
        t0 = time.time()
        st, ok = exchange()
        log["2_peer_absent"] = {"status": st["name"], "site": st["site"], "seconds": round(time.time() - t0, 2)}
    comm.host_barrier()

    # 3. recovery
    comm.reset()
    st, ok = exchange()
    log["3_after_reset"] = {"status": st["name"], "data_ok": ok}

    # 4. an announced departure is seen on the host
    comm.host_barrier()
    if me == last:
        comm.announce_leave()
    comm.host_barrier()
    if me != last:
        try:
            comm.require_peers()
            log["4_announced_leave"] = "not noticed"
        except CommError as e:
            log["4_announced_leave"] = "refused to launch: " + str(e)
    comm.host_barrier()

    # 5. it returns
    if me == last:
        comm.announce_return()
    comm.host_barrier()
    comm.require_peers()
    st, ok = exchange()
    log["5_after_return"] = {"status": st["name"], "data_ok": ok}

    good = (log["1_normal"] == {"status": "ok", "data_ok": True} and log["3_after_reset"] == {"status": "ok", "data_ok": True}
            and log["5_after_return"] == {"status": "ok", "data_ok": True})
    if me != last:
        good = good and log["2_peer_absent"]["status"] == "timeout" and log["4_announced_leave"].startswith("refused")
    flag = torch.tensor([0 if good else 1], device="cuda")
    dist.all_reduce(flag)
    if me == 0:
        print(json.dumps({"fault_case": "ok" if int(flag.item()) == 0 else "FAILED", "processes": world, "log": log}), flush=True)
    comm.close()
    dist.destroy_process_group()
    return 0 if int(flag.item()) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
