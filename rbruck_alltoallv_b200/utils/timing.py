"""Device-side timing of collectives.

Rules followed everywhere: warm-up first; every timed call is preceded (outside the timed span) by an L2
flush (a write of a buffer larger than the 126 MB L2) and by a zero-byte alltoallv that lines the ranks up
on the device, so that launch skew between processes is not billed to the collective; the span itself is
a pair of CUDA events on the launching stream; multi-process results are the per-step maximum over ranks.
The reference times with MPI_Wtime around the call and an MPI_Allreduce(MAX)
(examples/rbruckv_example.cpp:101-131); this is the device-side counterpart.
"""
from __future__ import annotations

import subprocess
import threading
import time
from typing import Callable, Optional

import numpy as np
import torch

L2_FLUSH_BYTES = 256 << 20


class L2Flusher:
    def __init__(self, device, nbytes: int = L2_FLUSH_BYTES):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def __call__(self):
        self.buf.fill_(1)


class RankAligner:
    """A zero-byte alltoallv across the processes: returns on every rank within a couple of microseconds of the
    last rank entering it.  Nothing to do (and nothing launched) when one process hosts all ranks."""

    def __init__(self, comm):
        self.comm = comm
        self.call = None
        self._own = None
        if comm.nproc == 1:
            return
        if comm.P > 64:   # the aligning kernel exchanges metadata in the kernel, which takes at most 64 ranks
            from ..parallel.comm import Communicator
            comm = self._own = Communicator(nranks=comm.nproc, heap_bytes=1 << 20, arena_bytes=1 << 16)
        L, P = comm.L, comm.P
        self.z = np.zeros((L, P), dtype=np.int32)
        self.zd = np.zeros((L, P), dtype=np.int64)
        self.recv = [comm.symm_empty(16, torch.uint8) for _ in range(L)]
        self.send = [torch.empty(16, dtype=torch.uint8, device=f"cuda:{comm.device}") for _ in range(L)]
        # the kernel that exchanges metadata waits for every rank's row: that wait is the alignment (the static
        # kernel would find nothing to do for an exchange of empty blocks and return at once)
        self.call = comm.prepare(self.send, self.recv, self.z, self.zd, self.z, self.zd, algo="spreadout",
                                 type_size=1, grid=1, static=False)

    def __call__(self):
        if self.call is not None:
            self.call.launch()


def time_steps(fn: Callable[[], None], steps: int, warmup: int, flush: Optional[Callable[[], None]] = None,
               align: Optional[Callable[[], None]] = None, dist_group=None) -> np.ndarray:
    """Per-step device times in milliseconds (max over ranks when torch.distributed is initialised)."""
    import torch.distributed as dist

    for _ in range(warmup):
        if flush:
            flush()
        if align:
            align()
        fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    if multi:
        dist.barrier(group=dist_group)
    torch.cuda.synchronize()
    for i in range(steps):
        if flush:
            flush()
        if align:
            align()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    if multi:
        dist.barrier(group=dist_group)
    t = torch.tensor([s.elapsed_time(e) for s, e in zip(starts, ends)], dtype=torch.float64)
    if multi:
        tt = t.cuda()
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t = tt.cpu()
    return t.numpy()


class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi while a measurement runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0, period_ms: int = 100):
        self.idx = device_index
        self.period_ms = period_ms
        self.proc = None
        self.lines = []
        self._t = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.idx),
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._t = threading.Thread(target=self._read, daemon=True)
            self._t.start()
            time.sleep(0.25)
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}
