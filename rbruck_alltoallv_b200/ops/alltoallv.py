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


SAFE_CHOICE = {"algo": "spreadout", "protocol": "rendezvous"}


def agreed_block_stats(c, sendcounts, ts: int):
    """(mean block bytes, coefficient of variation) of the WHOLE exchange: the sums over this process's rows are
    added up over the host side group, so every process gets the same two numbers (a process that looked at its
    own rows only would, with skewed counts, land in another size class than its peers and pick another
    algorithm or protocol, which ends in a time-out)."""
    a = np.asarray(sendcounts, dtype=np.float64).ravel() * ts
    acc = torch.tensor([float(a.sum()), float((a * a).sum()), float(a.size)], dtype=torch.float64)
    side = getattr(c, "_side", None)
    if side is not None:
        c._dist.all_reduce(acc, group=side)
    s1, s2, n = (float(v) for v in acc)
    if n <= 0 or s1 <= 0:
        return 0.0, 0.0
    mean = s1 / n
    return mean, float(np.sqrt(max(s2 / n - mean * mean, 0.0)) / mean)


def _auto_choice(c, recv, sendcounts, kw, agree_on_max: bool):
    """Resolves ``algo="auto"`` into keyword arguments for the communicator, using the tuner table.  The outcome is
    the same on every process: persistent calls (``agree_on_max``) agree on the size and skew class by a host-side
    reduction; one-shot calls of a multi-process communicator use the caller's ``mean_block_bytes=`` hint (which
    must be the same everywhere) or, without it, the spread-out order with the rendezvous protocol, which mixes
    safely with itself whatever the counts are."""
    ts = kw.get("type_size") or (recv.element_size() if isinstance(recv, torch.Tensor) else recv[0].element_size())
    host_counts = not (isinstance(sendcounts, torch.Tensor) and sendcounts.is_cuda)
    kw = dict(kw)
    hint = kw.pop("mean_block_bytes", None)
    cv = float(kw.pop("block_cv", 0.0) or 0.0)
    multi = getattr(c, "nproc", 1) > 1
    if hint is not None:
        mean_block = float(hint)
    elif host_counts and (agree_on_max or not multi):
        mean_block, cv = agreed_block_stats(c, sendcounts, ts) if agree_on_max else _tuner.block_stats(sendcounts, ts)
    elif not host_counts and kw.get("bytes_hint", -1) and kw.get("bytes_hint", -1) > 0 and not multi:
        mean_block = kw["bytes_hint"] / (c.L * c.P)
    else:
        mean_block = None
    choice = _tuner.choose(c.P, c.nproc, mean_block, cv) if mean_block is not None else dict(SAFE_CHOICE)
    forced = env_overrides()
    if "algo" in forced and forced["algo"] != choice.get("algo"):
        choice = {"algo": forced["algo"], "protocol": choice.get("protocol", "rendezvous")}   # drop the other algorithm's knobs
    choice.update(forced)
    out = kw
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
    not pay for a host-side reduction; :func:`prepare` does).  Across several processes the choice needs a number
    that is the same on all of them: pass ``mean_block_bytes=`` (and optionally ``block_cv=``), or the call uses
    the spread-out order with the rendezvous protocol."""
    c = comm or _comm.get_default_comm()
    if algo == "auto":
        kw = _auto_choice(c, recv, sendcounts, kw, agree_on_max=False)
        algo = kw.pop("algo")
    else:
        for k in ("max_block_bytes", "mean_block_bytes", "block_cv"):
            kw.pop(k, None)
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
        for k in ("max_block_bytes", "mean_block_bytes", "block_cv"):
            kw.pop(k, None)
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
