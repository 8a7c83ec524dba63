"""Functional alltoallv API and the NCCL baseline.

``alltoallv`` is the call a user makes; ``algo="auto"`` asks the tuner (``parallel/tuner.py``) for the
algorithm, radix and batch that measured fastest for the message-size class.  ``nccl_alltoallv`` is the
grouped ``ncclSend``/``ncclRecv`` exchange (through ``torch.distributed.all_to_all_single``), kept as the
baseline only: it stands where ``MPI_Alltoallv`` stands in the reference's drivers
(e.g. examples/twophaseLayer_example.cpp:99-113).
"""
from __future__ import annotations

import os
from typing import Optional, Sequence

import numpy as np
import torch

from ..parallel import comm as _comm
from ..parallel import tuner as _tuner


_ENV_INT = {"RBV_RADIX": "r", "RBV_RADIX2": "r2", "RBV_BATCH": "b", "RBV_BATCH2": "b2", "RBV_GROUP": "n"}


def env_overrides() -> dict:
    """Choices forced from the environment: ``RBV_ALGO`` (any algorithm name), ``RBV_RADIX`` / ``RBV_RADIX2``,
    ``RBV_BATCH`` / ``RBV_BATCH2``, ``RBV_GROUP`` (ranks per group of the two-layer algorithms) and ``RBV_PROTOCOL``
    (``eager`` or ``rendezvous``).  They take precedence over the tuner table in ``algo="auto"`` calls.  The
    reference's drivers take the same knobs as positional arguments (examples/rbruckv_example.cpp:23-44)."""
    out = {}
    if os.environ.get("RBV_ALGO"):
        out["algo"] = os.environ["RBV_ALGO"]
    for var, key in _ENV_INT.items():
        if os.environ.get(var):
            out[key] = int(os.environ[var])
    proto = os.environ.get("RBV_PROTOCOL", "")
    if proto:
        if proto not in ("eager", "rendezvous"):
            raise ValueError("RBV_PROTOCOL must be 'eager' or 'rendezvous'")
        out["protocol"] = proto
    return out


def _auto_choice(c, recv, sendcounts, kw, agree_on_max: bool):
    """Resolves ``algo="auto"`` into keyword arguments for the communicator, using the tuner table."""
    ts = kw.get("type_size") or (recv.element_size() if isinstance(recv, torch.Tensor) else recv[0].element_size())
    host_counts = not (isinstance(sendcounts, torch.Tensor) and sendcounts.is_cuda)
    if host_counts:
        mean_block = float(np.mean(np.asarray(sendcounts))) * ts
    else:
        hint = kw.get("bytes_hint", -1)
        mean_block = hint / (c.L * c.P) if hint and hint > 0 else 64 << 10
    choice = _tuner.choose(c.P, c.nproc, mean_block)
    forced = env_overrides()
    if "algo" in forced and forced["algo"] != choice.get("algo"):
        choice = {"algo": forced["algo"], "protocol": choice.get("protocol", "rendezvous")}   # drop the other algorithm's knobs
    choice.update(forced)
    out = dict(kw)
    out["algo"] = choice.pop("algo")
    protocol = choice.pop("protocol", "rendezvous")
    # The eager protocol needs one cell size on all ranks: either the caller promises an upper bound
    # (``max_block_bytes=``) or, where a collective host reduction is affordable, the ranks agree on the maximum.
    emax = out.pop("max_block_bytes", 0)
    if protocol == "eager" and "eager_max_bytes" not in out:
        if not emax and agree_on_max and host_counts:
            emax = c.max_block_bytes(sendcounts, ts)
        if 0 < emax <= (256 << 10) and (c.P + 64) * (2 * emax + 16) <= c.arena_bytes:
            out["eager_max_bytes"] = int(emax)
    for k, v in choice.items():
        out.setdefault(k, v)
    return out


def alltoallv(send, recv, sendcounts, sdispls=None, recvcounts=None, rdispls=None, *, comm=None,
              algo: str = "auto", **kw) -> None:
    """One-shot call.  With ``algo="auto"`` the tuner picks algorithm, radix and batch; the low-latency eager
    protocol is used only when the caller bounds the block size with ``max_block_bytes=`` (a one-shot call does
    not pay for a host-side reduction; :func:`prepare` does)."""
    c = comm or _comm.get_default_comm()
    if algo == "auto":
        kw = _auto_choice(c, recv, sendcounts, kw, agree_on_max=False)
        algo = kw.pop("algo")
    else:
        kw.pop("max_block_bytes", None)
    c.alltoallv(send, recv, sendcounts, sdispls, recvcounts, rdispls, algo=algo, **kw)


def prepare(send, recv, sendcounts, sdispls=None, recvcounts=None, rdispls=None, *, comm=None, algo: str = "auto",
            **kw):
    """Persistent call (``.launch()`` repeats it).  ``algo="auto"`` resolves algorithm AND protocol once, including
    the collective agreement on the eager cell size.  Collective over the processes when counts are on the host."""
    c = comm or _comm.get_default_comm()
    if algo == "auto":
        kw = _auto_choice(c, recv, sendcounts, kw, agree_on_max=True)
        algo = kw.pop("algo")
    else:
        kw.pop("max_block_bytes", None)
    kw.pop("stream", None)
    return c.prepare(send, recv, sendcounts, sdispls, recvcounts, rdispls, algo=algo, **kw)


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
