"""Functional alltoallv API and the NCCL baseline.

``alltoallv`` is the call a user makes; ``algo="auto"`` asks the tuner (``parallel/tuner.py``) for the
algorithm, radix and batch that measured fastest for the message-size class.  ``nccl_alltoallv`` is the
grouped ``ncclSend``/``ncclRecv`` exchange (through ``torch.distributed.all_to_all_single``), kept as the
baseline only: it stands where ``MPI_Alltoallv`` stands in the reference's drivers
(e.g. examples/twophaseLayer_example.cpp:99-113).
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..parallel import comm as _comm
from ..parallel import tuner as _tuner


def alltoallv(send, recv, sendcounts, sdispls=None, recvcounts=None, rdispls=None, *, comm=None,
              algo: str = "auto", **kw) -> None:
    c = comm or _comm.get_default_comm()
    if algo == "auto":
        ts = kw.get("type_size") or (recv.element_size() if isinstance(recv, torch.Tensor) else recv[0].element_size())
        if isinstance(sendcounts, torch.Tensor) and sendcounts.is_cuda:
            hint = kw.get("bytes_hint", -1)
            mean_block = hint / (c.L * c.P) if hint and hint > 0 else 64 << 10
        else:
            mean_block = float(np.mean(np.asarray(sendcounts))) * ts
        choice = _tuner.choose(c.P, c.nproc, mean_block)
        algo = choice.pop("algo")
        protocol = choice.pop("protocol", "rendezvous")
        host_counts = not (isinstance(sendcounts, torch.Tensor) and sendcounts.is_cuda)
        if protocol == "eager" and host_counts and "eager_max_bytes" not in kw:
            emax = c.max_block_bytes(sendcounts, ts)       # collective: agrees on the cell size
            if 0 < emax <= (256 << 10) and (c.P + 64) * (2 * emax + 16) <= c.arena_bytes:
                kw["eager_max_bytes"] = emax
        for k, v in choice.items():
            kw.setdefault(k, v)
    c.alltoallv(send, recv, sendcounts, sdispls, recvcounts, rdispls, algo=algo, **kw)


def alltoall(send, recv, count: int, *, comm=None, algo: str = "auto", **kw) -> None:
    """Uniform all-to-all: ``count`` elements per pair, standard layout (block s of recv comes from rank s)."""
    c = comm or _comm.get_default_comm()
    sc = np.full((c.L, c.P), int(count), dtype=np.int32)
    sd = np.tile(np.arange(c.P, dtype=np.int64) * int(count), (c.L, 1))
    alltoallv(send, recv, sc, sd, sc, sd, comm=c, algo=algo, **kw)


def nccl_alltoallv(send: torch.Tensor, recv: torch.Tensor, sendcounts: Sequence[int], recvcounts: Sequence[int],
                   group=None) -> None:
    """Baseline: NCCL grouped send/recv.  One rank per process, packed layouts, counts in elements."""
    import torch.distributed as dist
    dist.all_to_all_single(recv, send, output_split_sizes=[int(x) for x in recvcounts],
                           input_split_sizes=[int(x) for x in sendcounts], group=group)
