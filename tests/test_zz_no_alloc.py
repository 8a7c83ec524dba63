"""The allocation-free alltoallv entry point, called through its exported C symbol.

Some hosts of this library cannot let it allocate device memory when a collective is issued (a CUDA graph is
being captured, or another framework owns the whole device-memory budget).  For them the library exports
``rbv_alltoallv_noalloc``, whose scratch lives in an array inside the library image.  This test drives that
symbol with ctypes, twice in a row with different data and counts, and requires the receive buffers to be
byte-identical to what the regular context-based entry point produces for the same schedule
(radix-2 ``rbruck_om``).  It also checks that requests beyond the built-in limits are refused.

Collected last on purpose: a failure here must not hide the results of the other tests.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from rbruck_alltoallv_b200.utils import distributions as dist
from rbruck_alltoallv_b200.utils import oracle

pytestmark = pytest.mark.gpu


def _ptr(a):
    return C.c_void_p(a.ctypes.data)


def _run_noalloc(lib, prob, send, recv, ts):
    P = prob.P
    sp = (C.c_void_p * P)(*[t.data_ptr() for t in send])
    rp = (C.c_void_p * P)(*[t.data_ptr() for t in recv])
    sc = np.ascontiguousarray(prob.counts, dtype=np.int32)
    rc = np.ascontiguousarray(prob.recvcounts, dtype=np.int32)
    sd = np.ascontiguousarray(prob.sdispls, dtype=np.int64)
    rd = np.ascontiguousarray(prob.rdispls, dtype=np.int64)
    st = torch.cuda.current_stream().cuda_stream
    rcode = lib.rbv_alltoallv_noalloc(P, ts, sp, rp, _ptr(sc), _ptr(sd), _ptr(rc), _ptr(rd), C.c_void_p(st))
    assert rcode == 0, lib.rbv_noalloc_last_error().decode()
    assert lib.rbv_noalloc_status(C.c_void_p(st)) == 0


@pytest.mark.parametrize("P", [8, 5])
def test_noalloc_matches_regular_entry_point_twice(P):
    from rbruck_alltoallv_b200 import _native
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    lib = _native.cuda_lib()
    comm = Communicator(nranks=P, heap_bytes=64 << 20, arena_bytes=1 << 20)
    try:
        for call, (ts, hi, packed) in enumerate([(4, 3000, True), (2, 9000, False)]):
            counts = dist.uniform(P, hi, seed=50 + call)
            counts[counts < hi // 10] = 0
            prob = oracle.make_problem(counts, ts, 60 + call, packed=packed)
            send_h = oracle.fill_send(prob, 70 + call)
            want = oracle.expected_recv(prob, send_h)
            send = [torch.from_numpy(b).cuda() for b in send_h]
            # regular path: receive buffers in the context's heap
            recv_a = [comm.symm_empty(len(w), torch.uint8) for w in want]
            # allocation-free path: plain device buffers owned by the caller
            recv_b = [torch.empty(len(w), dtype=torch.uint8, device="cuda") for w in want]
            for t in recv_a + recv_b:
                t.fill_(oracle.CANARY)
            comm.alltoallv(send, recv_a, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo="rbruck_om",
                           r=2, type_size=ts)
            comm.check()
            _run_noalloc(lib, prob, send, recv_b, ts)
            torch.cuda.synchronize()
            for d in range(P):
                a, b = recv_a[d].cpu().numpy(), recv_b[d].cpu().numpy()
                assert np.array_equal(a, want[d]), f"regular path wrong at rank {d}"
                assert np.array_equal(b, a), f"call {call}: rank {d} differs from the regular entry point"
    finally:
        comm.close()


def test_noalloc_refuses_requests_beyond_its_limits():
    from rbruck_alltoallv_b200 import _native
    lib = _native.cuda_lib()
    P = 9
    z32 = np.zeros(P * P, dtype=np.int32)
    z64 = np.zeros(P * P, dtype=np.int64)
    bufs = (C.c_void_p * P)(*[None] * P)
    assert lib.rbv_alltoallv_noalloc(P, 4, bufs, bufs, _ptr(z32), _ptr(z64), _ptr(z32), _ptr(z64), None) == -2
    assert b"limit" in lib.rbv_noalloc_last_error()
    P = 2
    big = np.array([0, 20000, 0, 0], dtype=np.int32)   # 80 000 bytes > 64 KB
    z64 = np.zeros(4, dtype=np.int64)
    bufs = (C.c_void_p * P)(*[None] * P)
    assert lib.rbv_alltoallv_noalloc(P, 4, bufs, bufs, _ptr(big), _ptr(z64), _ptr(big), _ptr(z64), None) == -2
    assert lib.rbv_alltoallv_noalloc(0, 4, bufs, bufs, _ptr(big), _ptr(z64), _ptr(big), _ptr(z64), None) == -1


def test_noalloc_status_names_the_failure():
    """A block larger than the receiver's recvcount is refused by the kernel (nothing is written past the slot) and
    the status query returns the recorded code (4 = truncation), not a blanket error; the next call works again."""
    from rbruck_alltoallv_b200 import _native
    lib = _native.cuda_lib()
    P, ts = 4, 4
    counts = dist.constant(P, 64)
    prob = oracle.make_problem(counts, ts, 0, packed=True)
    send_h = oracle.fill_send(prob, 1)
    want = oracle.expected_recv(prob, send_h)
    send = [torch.from_numpy(b).cuda() for b in send_h]
    recv = [torch.full((len(w),), oracle.CANARY, dtype=torch.uint8, device="cuda") for w in want]
    sp = (C.c_void_p * P)(*[t.data_ptr() for t in send])
    rp = (C.c_void_p * P)(*[t.data_ptr() for t in recv])
    sc = np.ascontiguousarray(prob.counts, dtype=np.int32)
    rc = np.ascontiguousarray(prob.recvcounts, dtype=np.int32).copy()
    rc[2, 1] = 10                      # rank 2 expects less from rank 1 than rank 1 sends
    sd = np.ascontiguousarray(prob.sdispls, dtype=np.int64)
    rd = np.ascontiguousarray(prob.rdispls, dtype=np.int64)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.rbv_alltoallv_noalloc(P, ts, sp, rp, _ptr(sc), _ptr(sd), _ptr(rc), _ptr(rd), st) == 0
    assert lib.rbv_noalloc_status(st) == 4
    _run_noalloc(lib, prob, send, recv, ts)      # every call clears the control words: the entry point recovers
    torch.cuda.synchronize()
    assert oracle.first_mismatch([t.cpu().numpy() for t in recv], want) is None
