"""ctypes loaders for the two native libraries (see ``_build.py``)."""
from __future__ import annotations

import ctypes as C
import os
import threading

from . import _build

_lock = threading.Lock()
_host = None
_cuda = None

c_int_p = C.POINTER(C.c_int)
c_ll_p = C.POINTER(C.c_longlong)


class Choice(C.Structure):
    """``rbv_choice`` of the C API: a configuration as the tuner table stores it."""
    _fields_ = [("algo", C.c_int), ("n", C.c_int), ("r", C.c_int), ("r2", C.c_int), ("b", C.c_int), ("b2", C.c_int),
                ("eager", C.c_int)]


def _declare_host(lib):
    lib.rbv_plan_create.restype = C.c_void_p
    lib.rbv_plan_create.argtypes = [C.c_int] * 7
    lib.rbv_plan_destroy.argtypes = [C.c_void_p]
    lib.rbv_plan_err.argtypes = [C.c_void_p]
    lib.rbv_plan_errmsg.restype = C.c_char_p
    lib.rbv_plan_errmsg.argtypes = [C.c_void_p]
    lib.rbv_plan_ncells.argtypes = [C.c_void_p]
    lib.rbv_plan_nops.restype = C.c_longlong
    lib.rbv_plan_nops.argtypes = [C.c_void_p]
    lib.rbv_plan_ops.restype = C.c_void_p
    lib.rbv_plan_ops.argtypes = [C.c_void_p]
    lib.rbv_plan_uniform.argtypes = [C.c_void_p]
    lib.rbv_plan_inplace_ok.argtypes = [C.c_void_p]
    lib.rbv_plan_stats.argtypes = [C.c_void_p, c_ll_p]
    lib.rbv_plan_spec.argtypes = [C.c_void_p, c_int_p]
    lib.rbv_algo_name.restype = C.c_char_p
    lib.rbv_algo_name.argtypes = [C.c_int]
    lib.rbv_algo_from_name.argtypes = [C.c_char_p]
    lib.rbv_host_alltoallv.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                       c_int_p, c_ll_p, c_ll_p]
    lib.rbv_ipow.argtypes = [C.c_int, C.c_uint]
    lib.rbv_ndigits.argtypes = [C.c_int, C.c_int]
    lib.rbv_to_base.argtypes = [C.c_int, C.c_int, C.c_int, c_int_p]
    lib.rbv_tuner_set_table.argtypes = [C.c_char_p]
    lib.rbv_tuner_entries.argtypes = []
    lib.rbv_tuner_choose.argtypes = [C.c_int, C.c_int, C.c_double, C.c_double, C.POINTER(Choice)]
    # the C API's automatic entry points read the same table file as parallel/tuner.py
    from .parallel import tuner as _tuner
    lib.rbv_tuner_set_table(str(_tuner._cache_path()).encode())


def host_lib():
    """The host-only library (plan compiler, CPU executor); built on first use."""
    global _host
    with _lock:
        if _host is None:
            path = _build.build_host()
            _host = C.CDLL(str(path))
            _declare_host(_host)
        return _host


def cuda_lib():
    """The CUDA library.  Loading needs libcudart only; running needs a B200.

    The host symbols are also linked into this library, so code that already holds the CUDA
    library can use it for plans as well.
    """
    global _cuda
    with _lock:
        if _cuda is None:
            path = _build.PKG / "librbv_cuda.so"
            if not path.exists() or os.environ.get("RBV_REBUILD"):
                path = _build.build_cuda()
            # RTLD_GLOBAL is not needed: every entry point is reached through this handle.
            _cuda = C.CDLL(str(path))
            _declare_host(_cuda)
            from ._cuda_decl import declare_cuda
            declare_cuda(_cuda)
        return _cuda
