"""Pencil transposes of a distributed 3-D grid (the communication of a distributed 3-D FFT).

The N^3 grid is decomposed over a Pr x Pc process grid with near-balanced, seeded, jittered splits:

* x-pencils  ``[z_l][y_l][x]``   y split over Pr, z split over Pc   (FFT along x is local),
* y-pencils  ``[z_l][x_l][y]``   x split over Pr, z split over Pc,
* z-pencils  ``[x_l][y_l][z]``   x split over Pr, y split over Pc.

``x_to_y`` and ``y_to_z`` are each ONE kernel (``csrc/kernels/fft_transpose.cu``): the strided gather, the
alltoallv inside the row / column group and the transposed scatter are fused, peers are written directly over
NVLink.  ``nccl_x_to_y`` is the baseline (pack with torch ops, NCCL all-to-all, unpack).  The reference only
generates the count patterns of such an exchange (examples/FFT_distribution.cpp:66-87).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Tuple

import numpy as np
import torch

from .. import _native
from .._cuda_decl import Box


def jittered_split(n: int, parts: int, frac: float, seed: int) -> np.ndarray:
    """``parts`` positive sizes that sum to n, each within about +-frac of n / parts."""
    rng = np.random.default_rng(seed)
    w = 1.0 + rng.uniform(-frac, frac, size=parts)
    s = np.floor(w / w.sum() * n).astype(np.int64)
    s[: n - int(s.sum())] += 1
    assert s.sum() == n and (s > 0).all()
    return s


class PencilTranspose:
    def __init__(self, comm, n: int, pr: int, pc: int, dtype=torch.complex64, jitter: float = 0.05, seed: int = 0):
        if comm.L != 1 or pr * pc != comm.P:
            raise ValueError("need one rank per process and pr * pc == number of ranks")
        self.comm, self.lib, self.n, self.pr, self.pc, self.dtype = comm, _native.cuda_lib(), n, pr, pc, dtype
        self.me_r, self.me_c = comm.proc // pc, comm.proc % pc
        self.esize = torch.empty(0, dtype=dtype).element_size()
        self.ysplit = jittered_split(n, pr, jitter, seed + 1)     # x-pencils: y over Pr
        self.zsplit = jittered_split(n, pc, jitter, seed + 2)     # x- and y-pencils: z over Pc
        self.xsplit = jittered_split(n, pr, jitter, seed + 3)     # y- and z-pencils: x over Pr
        self.y2split = jittered_split(n, pc, jitter, seed + 4)    # z-pencils: y over Pc
        off = lambda s: np.concatenate([[0], np.cumsum(s)[:-1]])
        self.y0, self.z0, self.x0, self.y20 = off(self.ysplit), off(self.zsplit), off(self.xsplit), off(self.y2split)
        r, c = self.me_r, self.me_c
        self.shape_x = (int(self.zsplit[c]), int(self.ysplit[r]), n)
        self.shape_y = (int(self.zsplit[c]), int(self.xsplit[r]), n)
        self.shape_z = (int(self.xsplit[r]), int(self.y2split[c]), n)
        # destination arrays live in the symmetric heap (peers write into them)
        # Peers address these arrays by their offset inside the heap, so the offset must be the same on every
        # rank: allocate the largest shape any rank has (the splits are known everywhere) and use a prefix of it.
        cap_y = int(self.zsplit.max()) * int(self.xsplit.max()) * n
        cap_z = int(self.xsplit.max()) * int(self.y2split.max()) * n
        self._store_y = comm.symm_empty(cap_y, dtype)
        self._store_z = comm.symm_empty(cap_z, dtype)
        self.buf_y = self._store_y[: int(np.prod(self.shape_y))].view(self.shape_y)
        self.buf_z = self._store_z[: int(np.prod(self.shape_z))].view(self.shape_z)
        self.error = torch.zeros(2, dtype=torch.int32, device=f"cuda:{comm.device}")
        heap0 = self.lib.rbv_ctx_heap(comm._ctx, comm.proc)
        self.off_y = self.buf_y.data_ptr() - heap0
        self.off_z = self.buf_z.data_ptr() - heap0
        comm.require_same_offsets(self.off_y, self.off_z)
        self._boxes_xy = self._make_boxes_xy()
        self._boxes_yz = self._make_boxes_yz()

    def _rank(self, r, c):
        return r * self.pc + c

    def _make_boxes_xy(self):
        n, r, c = self.n, self.me_r, self.me_c
        nz, ny = self.shape_x[0], self.shape_x[1]
        boxes = (Box * self.comm.P)()
        for r2 in range(self.pr):                       # same column group (same z range)
            b = boxes[self._rank(r2, c)]
            nx2 = int(self.xsplit[r2])
            b.n0, b.n1, b.n2 = nz, ny, nx2
            b.src_off, b.s0, b.s1 = int(self.x0[r2]), ny * n, n
            b.dst_off, b.t0, b.t1, b.t2 = int(self.y0[r]), nx2 * n, 1, n
        return boxes

    def _make_boxes_yz(self):
        n, r, c = self.n, self.me_r, self.me_c
        nz, nx = self.shape_y[0], self.shape_y[1]
        boxes = (Box * self.comm.P)()
        for c2 in range(self.pc):                       # same row group (same x range)
            b = boxes[self._rank(r, c2)]
            ny2 = int(self.y2split[c2])
            b.n0, b.n1, b.n2 = nz, nx, ny2
            b.src_off, b.s0, b.s1 = int(self.y20[c2]), nx * n, n
            b.dst_off, b.t0, b.t1, b.t2 = int(self.z0[c]), 1, ny2 * n, n
        return boxes

    def _run(self, src, off, boxes, err):
        st = C.c_void_p(torch.cuda.current_stream(src.device).cuda_stream)
        rc = self.lib.rbv_transpose_exchange(self.comm._ctx, C.c_void_p(src.data_ptr()), off, self.esize, boxes,
                                             C.c_void_p(err.data_ptr()), 0, st)
        if rc:
            raise RuntimeError(f"transpose launch failed (CUDA error {rc})")

    def x_to_y(self, src: torch.Tensor) -> torch.Tensor:
        assert tuple(src.shape) == self.shape_x and src.is_contiguous() and src.dtype == self.dtype
        self._run(src, self.off_y, self._boxes_xy, self.error[0:1])
        return self.buf_y

    def y_to_z(self, src: torch.Tensor) -> torch.Tensor:
        assert tuple(src.shape) == self.shape_y and src.is_contiguous() and src.dtype == self.dtype
        self._run(src, self.off_z, self._boxes_yz, self.error[1:2])
        return self.buf_z

    def check(self):
        e = self.error.cpu().tolist()
        if any(e):
            raise RuntimeError(f"transpose kernels reported a time-out: {e}")

    # ---- helpers for tests and benchmarks -----------------------------------------------------------------
    def local_x_pencil_of(self, full: torch.Tensor) -> torch.Tensor:
        """Cuts this rank's x-pencil out of a full [z][y][x] array."""
        r, c = self.me_r, self.me_c
        return full[self.z0[c]:self.z0[c] + self.zsplit[c], self.y0[r]:self.y0[r] + self.ysplit[r], :].contiguous()

    def expected_y(self, full: torch.Tensor) -> torch.Tensor:
        r, c = self.me_r, self.me_c
        return full[self.z0[c]:self.z0[c] + self.zsplit[c], :, self.x0[r]:self.x0[r] + self.xsplit[r]] \
            .permute(0, 2, 1).contiguous()

    def expected_z(self, full: torch.Tensor) -> torch.Tensor:
        r, c = self.me_r, self.me_c
        return full[:, self.y20[c]:self.y20[c] + self.y2split[c], self.x0[r]:self.x0[r] + self.xsplit[r]] \
            .permute(2, 1, 0).contiguous()

    def bytes_sent_xy(self) -> Tuple[int, int]:
        """(all bytes of this rank's x-pencil, bytes that leave the GPU) for the x -> y transpose."""
        nz, ny, n = self.shape_x
        total = nz * ny * n * self.esize
        local = nz * ny * int(self.xsplit[self.me_r]) * self.esize
        return total, total - local

    def nccl_x_to_y(self, src: torch.Tensor, group) -> torch.Tensor:
        """Baseline: pack per destination, NCCL all-to-all inside the column group, unpack with a transposition."""
        import torch.distributed as dist
        nz = self.shape_x[0]
        send = [src[:, :, self.x0[r2]:self.x0[r2] + self.xsplit[r2]].contiguous() for r2 in range(self.pr)]
        nx = int(self.xsplit[self.me_r])
        recv = [torch.empty(nz, int(self.ysplit[r2]), nx, dtype=self.dtype, device=src.device) for r2 in range(self.pr)]
        dist.all_to_all(recv, send, group=group)
        return torch.cat(recv, dim=1).permute(0, 2, 1).contiguous()

    def bytes_sent_yz(self) -> Tuple[int, int]:
        """(all bytes of this rank's y-pencil, bytes that leave the GPU) for the y -> z transpose."""
        nz, nx, n = self.shape_y
        total = nz * nx * n * self.esize
        local = nz * nx * int(self.y2split[self.me_c]) * self.esize
        return total, total - local

    def nccl_y_to_z(self, src: torch.Tensor, group) -> torch.Tensor:
        """Baseline for the second transpose: pack per destination, NCCL all-to-all inside the row group, unpack
        with a transposition."""
        import torch.distributed as dist
        nx = self.shape_y[1]
        send = [src[:, :, self.y20[c2]:self.y20[c2] + self.y2split[c2]].contiguous() for c2 in range(self.pc)]
        ny2 = int(self.y2split[self.me_c])
        recv = [torch.empty(int(self.zsplit[c2]), nx, ny2, dtype=self.dtype, device=src.device) for c2 in range(self.pc)]
        dist.all_to_all(recv, send, group=group)
        return torch.cat(recv, dim=0).permute(1, 2, 0).contiguous()
