"""rbruck_alltoallv_b200: a Blackwell-native non-uniform all-to-all (alltoallv) library.

Host-only parts (plan compiler, CPU executor, distributions, oracle) import without a GPU; the CUDA
library is loaded on first use of a GPU entry point.
"""
from .parallel.plan import ALGOS, Plan, PlanError, host_alltoallv  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    # GPU-facing API is imported lazily so that ``import rbruck_alltoallv_b200`` works on CPU boxes.
    if name in ("Communicator", "init", "get_default_comm"):
        from .parallel import comm as _c
        return getattr(_c, name)
    if name in ("alltoallv", "alltoall", "nccl_alltoallv", "prepare"):
        from .ops import alltoallv as _a
        return getattr(_a, name)
    if name == "symm_empty":
        # receive buffers of the default communicator (peers write into them): rbv.symm_empty(n, dtype)
        from .parallel import comm as _c
        return lambda *a, **k: _c.get_default_comm().symm_empty(*a, **k)
    if name == "bench":
        # latency table of the default communicator: rbv.bench(sizes=(16, 65536, ...)) -> list of rows
        from .parallel import comm as _c
        from .utils import selftest as _s
        return lambda *a, **k: _s.bench(_c.get_default_comm(), *a, **k)
    if name in ("MoEExpertParallel", "grouped_gemm", "grouped_gemm_fp8"):
        from .ops import moe as _m
        return getattr(_m, name)
    if name == "PencilTranspose":
        from .ops.fft import PencilTranspose
        return PencilTranspose
    if name == "UlyssesExchange":
        from .ops.ulysses import UlyssesExchange
        return UlyssesExchange
    raise AttributeError(name)
