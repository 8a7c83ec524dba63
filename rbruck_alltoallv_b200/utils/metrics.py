"""Figures of merit for one alltoallv measurement.

The reference prints seconds only (examples/rbruckv_example.cpp:123-131).  Here every row carries, besides the
time (device-timed, max over ranks): *algbw* = the largest number of bytes any rank sends (its self block included,
as nccl-tests counts an all-to-all) divided by the time; *busbw* = algbw (P - 1) / P; and the fraction of the
NVLink roofline = the bytes the ALGORITHM pushes out of (or into) the busiest GPU, forwarded hops of the Bruck
schedules included, divided by the link rate and by the time.
"""
from __future__ import annotations

from typing import Optional

import numpy as np

NVLINK_GBS = 900.0          # per direction per GPU (nominal NVLink 5 figure the roofline is stated against)
NVLINK_MEASURED_GBS = 770.0   # peer copy measured on this pool


def link_bytes(plan_ops: np.ndarray, counts: np.ndarray, type_size: int, L: int) -> int:
    """Bytes that cross between GPUs on the busiest GPU (the larger of what it sends and what it receives) when
    ranks are placed L per GPU, for the schedule given by ``Plan.ops()``."""
    if len(plan_ops) == 0:
        return 0
    src_p = plan_ops["src"].astype(np.int64) // L
    dst_p = plan_ops["dst"].astype(np.int64) // L
    cnt = np.asarray(counts, dtype=np.int64)[plan_ops["origin"].astype(np.int64), plan_ops["dest"].astype(np.int64)]
    nparts = (plan_ops["flags"].astype(np.int64) >> 9) & 127
    part = (plan_ops["flags"].astype(np.int64) >> 2) & 127
    div = np.where(nparts > 0, cnt // np.maximum(nparts, 1), cnt)
    size = np.where(nparts > 0, np.where(part == nparts - 1, cnt - part * div, div), cnt) * type_size
    cross = src_p != dst_p
    nproc = int(max(src_p.max(), dst_p.max())) + 1
    out_b = np.bincount(src_p[cross], weights=size[cross], minlength=nproc)
    in_b = np.bincount(dst_p[cross], weights=size[cross], minlength=nproc)
    return int(max(out_b.max(), in_b.max()))


def alltoallv_row(counts: np.ndarray, type_size: int, us: Optional[float], plan_ops: Optional[np.ndarray] = None,
                  L: int = 1) -> dict:
    """One measurement as a record: microseconds, per-rank algbw / busbw in GB/s, and (when the schedule is given)
    the bytes that cross NVLink on the busiest GPU with the fraction of the 900 GB/s roofline they stand for."""
    c = np.asarray(counts, dtype=np.int64)
    P = c.shape[0]
    row = {"us": None if us is None else round(float(us), 2)}
    if us is None or us <= 0:
        return row
    own = int(c.sum(axis=1).max()) * type_size
    algbw = own / (us * 1e-6) / 1e9
    row["algbw_GBps"] = round(algbw, 3)
    row["busbw_GBps"] = round(algbw * (P - 1) / P, 3)
    if plan_ops is not None:
        lb = link_bytes(plan_ops, c, type_size, L)
        row["link_bytes_busiest_gpu"] = lb
        row["frac_of_900GBps"] = round(lb / (NVLINK_GBS * 1e9) / (us * 1e-6), 4)
    return row
