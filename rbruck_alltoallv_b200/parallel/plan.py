"""Python view of the native plan compiler (``csrc/plan/plan.cpp``).

``Plan`` objects are cheap handles on native plans.  ``host_alltoallv`` runs a plan with the CPU
executor on numpy buffers; it is the host fallback and the reference point for the GPU kernels.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Sequence

import numpy as np

from .. import _native

ALGOS = (
    "linear", "spreadout", "scattered", "pairwise", "xor",
    "twolayer_linear", "twolayer_linear_s2", "twolayer_linear_s3", "twolayer_linear_s4",
    "rbruck", "rbruck_om", "tuna", "tuna2",
    "ttpl", "ttpl_bt", "ttpl_bt_s1", "ttpl_bt_s2",
    "uniform_spreadout_twolayer", "uniform_isplit_rbruck",
    "merge", "simple_merge", "split",
)
ALGO_ID = {name: i for i, name in enumerate(ALGOS)}
HIERARCHICAL = {"ttpl", "ttpl_bt", "ttpl_bt_s1", "ttpl_bt_s2", "uniform_spreadout_twolayer",
                "uniform_isplit_rbruck", "twolayer_linear", "twolayer_linear_s2", "twolayer_linear_s3",
                "twolayer_linear_s4"}
LEADER_ROUTED = {"merge", "simple_merge"}

OP_DTYPE = np.dtype([("src", "<u2"), ("dst", "<u2"), ("origin", "<u2"), ("dest", "<u2"),
                     ("src_cell", "<i4"), ("dst_cell", "<i4"), ("key", "<u4"), ("flags", "<u4")])


@dataclass(frozen=True)
class PlanStats:
    w: int
    K: int
    w2: int
    K2: int
    max_blocks_per_round: int
    phases: int
    hops: int


class PlanError(ValueError):
    """Invalid algorithm arguments; ``code`` is the reference's return code (-1) or -2 for its aborts."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"{msg} (code {code})")
        self.code = code


class Plan:
    def __init__(self, algo: str | int, P: int, n: int = 0, r: int = 2, r2: int = 0, b: int = 0, b2: int = 0,
                 lib=None):
        self._lib = lib or _native.host_lib()
        algo_id = ALGO_ID[algo] if isinstance(algo, str) else int(algo)
        self._h = C.c_void_p(self._lib.rbv_plan_create(algo_id, P, n, r, r2, b, b2))
        self.err = self._lib.rbv_plan_err(self._h)
        self.errmsg = self._lib.rbv_plan_errmsg(self._h).decode()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rbv_plan_destroy(h)

    def check(self) -> "Plan":
        if self.err:
            raise PlanError(self.err, self.errmsg)
        return self

    @property
    def handle(self):
        return self._h

    @property
    def ncells(self) -> int:
        return self._lib.rbv_plan_ncells(self._h)

    @property
    def uniform(self) -> bool:
        return bool(self._lib.rbv_plan_uniform(self._h))

    @property
    def inplace_ok(self) -> bool:
        return bool(self._lib.rbv_plan_inplace_ok(self._h))

    @property
    def spec(self) -> dict:
        out = (C.c_int * 7)()
        self._lib.rbv_plan_spec(self._h, out)
        return dict(algo=ALGOS[out[0]], P=out[1], n=out[2], r=out[3], r2=out[4], b=out[5], b2=out[6])

    @property
    def stats(self) -> PlanStats:
        out = (C.c_longlong * 7)()
        self._lib.rbv_plan_stats(self._h, out)
        return PlanStats(*[int(v) for v in out])

    def ops(self) -> np.ndarray:
        n = self._lib.rbv_plan_nops(self._h)
        if n == 0:
            return np.zeros(0, dtype=OP_DTYPE)
        ptr = self._lib.rbv_plan_ops(self._h)
        buf = (C.c_char * (n * OP_DTYPE.itemsize)).from_address(ptr)
        return np.frombuffer(buf, dtype=OP_DTYPE).copy()


def host_alltoallv(plan: Plan, sendbufs: Sequence[np.ndarray], recvbufs: Sequence[np.ndarray],
                   sendcounts: np.ndarray, sdispls: np.ndarray, rdispls: np.ndarray, type_size: int) -> int:
    """Run ``plan`` on host buffers.

    ``sendcounts[s, d]`` and ``sdispls[s, d]`` are rank s's arguments, ``rdispls[d, s]`` rank d's;
    all in elements of ``type_size`` bytes.  Buffers are 1-D ``uint8`` arrays, one per rank.
    """
    plan.check()
    P = len(sendbufs)
    sc = np.ascontiguousarray(sendcounts, dtype=np.int32)
    sd = np.ascontiguousarray(sdispls, dtype=np.int64)
    rd = np.ascontiguousarray(rdispls, dtype=np.int64)
    assert sc.shape == (P, P) and sd.shape == (P, P) and rd.shape == (P, P)
    sp = (C.c_void_p * P)(*[b.ctypes.data for b in sendbufs])
    rp = (C.c_void_p * P)(*[b.ctypes.data for b in recvbufs])
    return plan._lib.rbv_host_alltoallv(plan.handle, int(type_size), sp, rp,
                                        sc.ctypes.data_as(_native.c_int_p), sd.ctypes.data_as(_native.c_ll_p),
                                        rd.ctypes.data_as(_native.c_ll_p))
