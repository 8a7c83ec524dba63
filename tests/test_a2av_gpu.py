"""GPU tests of the alltoallv kernel: all logical ranks of a communicator on one device."""
import numpy as np
import pytest
import torch

from rbruck_alltoallv_b200.utils import distributions as dist
from rbruck_alltoallv_b200.utils import oracle

pytestmark = pytest.mark.gpu

_comms = {}


def get_comm(P, big_arena=False):
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    key = (P, big_arena)
    if key not in _comms:
        _comms[key] = Communicator(nranks=P, heap_bytes=256 << 20, arena_bytes=(24 << 20) if big_arena else (4 << 20))
    return _comms[key]


def run_case(P, algo, ts, counts, packed=True, seed=0, with_recvcounts=True, device_counts=False, persistent=False,
             launches=1, big_arena=False, **kw):
    comm = get_comm(P, big_arena)
    prob = oracle.make_problem(counts, ts, seed, packed=packed)
    send_h = oracle.fill_send(prob, seed)
    want = oracle.expected_recv(prob, send_h)
    send = [torch.from_numpy(b).cuda() for b in send_h]
    recv = [comm.symm_empty(len(w), torch.uint8) for w in want]
    for t in recv:
        t.fill_(oracle.CANARY)
    rc = prob.recvcounts if with_recvcounts else None
    sc, sd, rd = prob.counts, prob.sdispls, prob.rdispls
    if device_counts:
        sc = torch.from_numpy(sc.astype(np.int32)).cuda()
        sd = torch.from_numpy(sd).cuda()
        rd = torch.from_numpy(rd).cuda()
        rc = torch.from_numpy(rc.astype(np.int32)).cuda() if rc is not None else None
    call = None
    if persistent:
        call = comm.prepare(send, recv, sc, sd, rc, rd, algo=algo, type_size=ts, **kw)
        for i in range(launches):
            if i:
                for t in recv:
                    t.fill_(oracle.CANARY)
            call.launch()
    else:
        comm.alltoallv(send, recv, sc, sd, rc, rd, algo=algo, type_size=ts, **kw)
    comm.check()
    got = [t.cpu().numpy() for t in recv]
    bad = oracle.first_mismatch(got, want)
    assert bad is None, f"{algo} P={P} {kw}: first mismatch at rank/offset {bad}"
    return call


ALL = [("linear", {}), ("spreadout", {}), ("scattered", dict(b=3)), ("pairwise", {}), ("xor", {}),
       ("rbruck", dict(r=2)), ("rbruck", dict(r=3)), ("rbruck_om", dict(r=2)), ("tuna", dict(r=2, b=1)),
       ("tuna2", dict(r=2, b=2)), ("tuna2", dict(r=4, b=1)), ("tuna2", dict(r=8, b=0)),
       ("ttpl", dict(n=4, r=2)), ("ttpl", dict(n=2, r=2)), ("ttpl_bt", dict(n=4, r=2, b=1)),
       ("ttpl_bt_s1", dict(n=4, r=2, b=3)), ("ttpl_bt_s1", dict(n=2, r=2)), ("ttpl_bt_s2", dict(n=4, r=3, b=2)),
       ("uniform_spreadout_twolayer", dict(n=4, r=2)), ("uniform_isplit_rbruck", dict(n=2, r=2, r2=2)),
       ("twolayer_linear", dict(n=4)), ("twolayer_linear_s2", dict(n=4, b=2, b2=3)),
       ("twolayer_linear_s3", dict(n=2, b=1, b2=1)), ("twolayer_linear_s4", dict(n=4, b=1, b2=2))]


@pytest.mark.parametrize("algo,kw", ALL, ids=[f"{a}-{'-'.join(f'{k}{v}' for k, v in kw.items())}" for a, kw in ALL])
def test_all_algorithms_p8(algo, kw):
    counts = dist.uniform(8, 300, seed=3)
    counts[counts < 30] = 0
    run_case(8, algo, 4, counts, packed=False, seed=5, **kw)


NEW_SCHEMES = [("merge", dict(n=4)), ("merge", dict(n=2)), ("simple_merge", dict(n=4)), ("simple_merge", dict(n=2)),
               ("split", {}), ("split", dict(b=3))]


@pytest.mark.parametrize("algo,kw", ALL + NEW_SCHEMES,
                         ids=[f"{a}-{'-'.join(f'{k}{v}' for k, v in kw.items())}" for a, kw in ALL + NEW_SCHEMES])
def test_static_kernel_all_algorithms_p8(algo, kw):
    """Persistent calls with host-side counts run the static kernel (descriptors resolved on the host)."""
    counts = dist.uniform(8, 300, seed=4)
    counts[counts < 30] = 0
    call = run_case(8, algo, 4, counts, packed=False, seed=6, persistent=True, launches=3, **kw)
    assert call.kind == "static"


@pytest.mark.parametrize("algo,kw", NEW_SCHEMES, ids=[f"{a}-{'-'.join(f'{k}{v}' for k, v in kw.items())}" for a, kw in NEW_SCHEMES])
def test_leader_routed_and_split_schemes_dynamic_kernel(algo, kw):
    counts = dist.uniform(8, 300, seed=14)
    counts[counts < 30] = 0
    run_case(8, algo, 8, counts, packed=False, seed=15, **kw)


def test_static_kernel_forwards_chunk_by_chunk():
    # blocks of about 0.5 MB in 16 KB chunks: relay hops start while earlier chunks of the same block still travel
    counts = dist.normal(8, 120_000, seed=2)
    for algo, kw in (("rbruck", dict(r=2)), ("tuna2", dict(r=2, b=0)), ("ttpl_bt_s1", dict(n=4, r=2)), ("merge", dict(n=4))):
        call = run_case(8, algo, 4, counts, seed=3, persistent=True, launches=2, chunk_bytes=16 << 10, big_arena=True, **kw)
        assert call.kind == "static" and call.items > 8 * 7 * 20
    # the dynamic kernel has the same per-chunk flags
    run_case(8, "rbruck", 4, counts, seed=4, r=2, chunk_bytes=16 << 10, big_arena=True)
    run_case(8, "split", 4, counts, seed=5, persistent=True, chunk_bytes=32 << 10, big_arena=True)


def test_static_kernel_refuses_what_the_host_can_see():
    from rbruck_alltoallv_b200.parallel.comm import CommError
    P, ts = 4, 4
    comm = get_comm(P)
    prob = oracle.make_problem(dist.constant(P, 64), ts, 0)
    send = [torch.zeros(int(b), dtype=torch.uint8, device="cuda") for b in prob.send_bytes]
    recv = [comm.symm_empty(int(b), torch.uint8) for b in prob.recv_bytes]
    rc = prob.recvcounts.copy()
    rc[2, 1] = 10                      # rank 2 expects less from rank 1 than rank 1 sends
    with pytest.raises(CommError, match="larger than the receiver"):
        comm.prepare(send, recv, prob.counts, prob.sdispls, rc, prob.rdispls, algo="spreadout", type_size=ts)
    rd = prob.rdispls.copy()
    rd[3, 0] += 1 << 40                # a displacement that would send a peer's stores outside the heap
    with pytest.raises(CommError, match="heap"):
        comm.prepare(send, recv, prob.counts, prob.sdispls, prob.recvcounts, rd, algo="spreadout", type_size=ts)
    with pytest.raises(CommError, match="heap"):
        comm.alltoallv(send, recv, prob.counts, prob.sdispls, prob.recvcounts, rd, algo="spreadout", type_size=ts)


def test_static_call_of_one_process_takes_pinned_host_buffers():
    """One process hosting every rank: a static call may send from and receive into pinned host memory directly."""
    from rbruck_alltoallv_b200.parallel.comm import CommError
    P, ts = 8, 4
    comm = get_comm(P)
    counts = dist.zipf(P, 4096, seed=9)
    prob = oracle.make_problem(counts, ts, 1, packed=False)
    send_h = oracle.fill_send(prob, 1)
    want = oracle.expected_recv(prob, send_h)
    send = [torch.from_numpy(b.copy()).pin_memory() for b in send_h]
    recv = [torch.full((len(w),), oracle.CANARY, dtype=torch.uint8).pin_memory() for w in want]
    for algo, kw in (("spreadout", {}), ("rbruck", dict(r=2)), ("ttpl_bt_s1", dict(n=4, r=2))):
        for t in recv:
            t.fill_(oracle.CANARY)
        call = comm.prepare(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo=algo,
                            type_size=ts, **kw)
        assert call.kind == "static"
        call.launch()
        comm.check()
        bad = oracle.first_mismatch([t.numpy() for t in recv], want)
        assert bad is None, f"{algo}: first mismatch at rank/offset {bad}"
    # a displacement that leaves the tensor is refused: the extent check of the heap is replaced by one against the tensor
    rd = prob.rdispls.copy()
    rd[3, 0] += 1 << 30
    with pytest.raises(CommError, match="heap"):
        comm.prepare(send, recv, prob.counts, prob.sdispls, prob.recvcounts, rd, algo="spreadout", type_size=ts)


def test_eager_cells_never_show_flags_of_an_earlier_life():
    """Eager units are valid by the call number in their flag words.  The cells must therefore never hold flag
    words that did not come from the current numbering: not from rendezvous staging of user payload (which may
    contain any value), not from calls made before reset() put the call number back, and not from a context whose
    heap memory this context inherited."""
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    P, ts = 8, 4
    for life in range(2):            # the second communicator is likely to get the first one's memory
        comm = Communicator(nranks=P, heap_bytes=64 << 20, arena_bytes=2 << 20)

        def eager_call(hi, seed):
            counts = dist.uniform(P, hi, seed=seed)
            prob = oracle.make_problem(counts, ts, seed, packed=True)
            send_h = oracle.fill_send(prob, seed)
            want = oracle.expected_recv(prob, send_h)
            send = [torch.from_numpy(b).cuda() for b in send_h]
            recv = [comm.symm_empty(len(w), torch.uint8) for w in want]
            for t in recv:
                t.fill_(oracle.CANARY)
            comm.alltoallv(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo="rbruck", r=2,
                           type_size=ts, eager_max_bytes=hi * ts)
            comm.check()
            assert oracle.first_mismatch([t.cpu().numpy() for t in recv], want) is None

        # rendezvous Bruck stages user payload made of small integers that look like call numbers
        words = np.arange(1, 40, dtype=np.int32)
        counts = dist.constant(P, 4096)
        prob = oracle.make_problem(counts, ts, 0)
        send = [torch.from_numpy(np.resize(words, int(b) // 4).view(np.uint8).copy()).cuda() for b in prob.send_bytes]
        recv = [comm.symm_empty(int(b), torch.uint8) for b in prob.recv_bytes]
        for _ in range(2):
            comm.alltoallv(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo="rbruck", r=2,
                           type_size=ts)
        comm.check()
        for i in range(6):
            eager_call(3000, 10 + i)             # large blocks: flags of calls 3..8 far into the cells
        # a rank that never joins: time-out, then reset() restarts the numbering
        comm.set_timeout_ms(50)
        comm.inject_absent_rank(1)
        comm.alltoallv(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo="spreadout", type_size=ts)
        assert comm.status()["name"] == "timeout"
        comm.inject_absent_rank(-1)
        comm.set_timeout_ms(2000)
        comm.reset()
        for i in range(4):
            eager_call(40, 30 + i)               # small blocks overwrite only the front of the cells ...
        for i in range(8):
            eager_call(3000, 40 + i)             # ... and large ones walk the numbering up to the old values
        comm.close()


@pytest.mark.parametrize("P", [1, 2, 3, 5, 6, 7, 12, 16])
def test_rank_counts(P):
    counts = dist.uniform(P, 100, seed=P)
    for algo, kw in [("spreadout", {}), ("rbruck", dict(r=2)), ("tuna2", dict(r=3, b=2)), ("rbruck_om", dict(r=max(P, 2)))]:
        run_case(P, algo, 8, counts, packed=(P % 2 == 0), seed=P, **kw)
        run_case(P, algo, 8, counts, packed=(P % 2 == 1), seed=P + 1, persistent=True, launches=2, **kw)


@pytest.mark.parametrize("ts", [1, 2, 4, 8, 16])
def test_type_sizes_unaligned(ts):
    counts = dist.uniform(8, 777, seed=ts)
    run_case(8, "tuna2", ts, counts, packed=False, seed=ts, r=2, b=1)
    run_case(8, "spreadout", ts, counts, packed=False, seed=ts + 1)


def test_large_blocks_multi_chunk():
    counts = dist.normal(4, 300_000, seed=1)           # ~1.2 MB blocks of 4-byte elements
    run_case(4, "spreadout", 4, counts, seed=1, chunk_bytes=64 << 10)
    run_case(4, "rbruck", 4, counts, seed=2, r=2, chunk_bytes=96 << 10, grid=37)


BULK = [("spreadout", {}), ("rbruck", dict(r=2)), ("tuna2", dict(r=2, b=2)), ("ttpl_bt_s1", dict(n=2, r=2))]


@pytest.mark.parametrize("algo,kw", BULK, ids=[a for a, _ in BULK])
def test_bulk_copy_engine(algo, kw):
    # 16-byte elements keep every block aligned: blocks of up to 80 KB span many 4 KB tiles with ragged last tiles
    run_case(4, algo, 16, dist.uniform(4, 5000, seed=7), seed=7, bulk=1, **kw)
    # 4-byte elements with gaps between blocks: unaligned chunks fall back to the vector path, aligned ones
    # end in tails shorter than 16 bytes; several chunks per block
    run_case(4, algo, 4, dist.uniform(4, 9000, seed=8), packed=False, seed=8, bulk=1, chunk_bytes=8 << 10, **kw)
    if algo == "spreadout":
        # the size-based choice: 2.8 MB blocks give every warp more than 16 KB
        run_case(4, algo, 4, dist.normal(4, 700_000, seed=9), seed=9, bulk=-1, **kw)


def test_zipf_and_empty():
    counts = dist.zipf(8, 16384, seed=11)
    run_case(8, "rbruck", 4, counts, seed=11, r=2)
    run_case(8, "tuna2", 4, np.zeros((8, 8), dtype=np.int64), seed=1, r=2)


def test_device_resident_counts():
    counts = dist.uniform(8, 500, seed=21)
    run_case(8, "tuna2", 2, counts, seed=21, device_counts=True, r=2, b=1)
    run_case(8, "spreadout", 2, counts, seed=22, device_counts=True, with_recvcounts=False)


def test_back_to_back_calls_alternate_parity():
    counts = dist.uniform(8, 200, seed=31)
    for i in range(6):
        run_case(8, "rbruck", 4, counts, seed=31 + i, r=2)


def test_inplace():
    P, ts = 8, 4
    comm = get_comm(P)
    counts = dist.uniform(P, 120, seed=41)
    prob = oracle.make_problem(counts, ts, 41, packed=True)
    send_h = oracle.fill_send(prob, 41)
    want = oracle.expected_recv(prob, send_h, tail=0)
    recv = []
    for d in range(P):
        n = max(len(want[d]), len(send_h[d]))
        t = comm.symm_empty(n, torch.uint8)
        t.fill_(oracle.CANARY)
        t[: len(send_h[d])] = torch.from_numpy(send_h[d]).cuda()
        recv.append(t)
    comm.alltoallv(None, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo="ttpl_bt_s2",
                   n=4, r=2, type_size=ts, inplace=True)
    comm.check()
    for d in range(P):
        got = recv[d].cpu().numpy()[: len(want[d])]
        assert np.array_equal(got, want[d])


def test_truncation_is_reported_not_written():
    P, ts = 4, 4
    comm = get_comm(P)
    counts = dist.constant(P, 64)
    prob = oracle.make_problem(counts, ts, 0)
    send = [torch.zeros(int(b), dtype=torch.uint8, device="cuda") for b in prob.send_bytes]
    recv = [comm.symm_empty(int(b), torch.uint8) for b in prob.recv_bytes]
    rc = prob.recvcounts.copy()
    rc[2, 1] = 10                      # rank 2 expects less from rank 1 than rank 1 sends
    comm.alltoallv(send, recv, prob.counts, prob.sdispls, rc, prob.rdispls, algo="spreadout", type_size=ts)
    st = comm.status()
    assert st["name"] == "truncate" and st["detail"] == (1, 2)
    comm.reset()
    run_case(P, "spreadout", ts, counts)


def test_absent_rank_times_out_and_context_recovers():
    P, ts = 4, 4
    comm = get_comm(P)
    counts = dist.constant(P, 16)
    prob = oracle.make_problem(counts, ts, 0)
    send = [torch.zeros(int(b), dtype=torch.uint8, device="cuda") for b in prob.send_bytes]
    recv = [comm.symm_empty(int(b), torch.uint8) for b in prob.recv_bytes]
    comm.set_timeout_ms(50)
    comm.inject_absent_rank(2)
    comm.alltoallv(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo="tuna2", r=2,
                   type_size=ts)
    st = comm.status()
    assert st["name"] == "timeout" and st["site"] == "metadata"
    comm.inject_absent_rank(-1)
    comm.set_timeout_ms(2000)
    comm.reset()
    run_case(P, "tuna2", ts, counts, r=2)


def test_staging_capacity_error():
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    comm = Communicator(nranks=8, heap_bytes=64 << 20, arena_bytes=64 << 10)
    counts = dist.constant(8, 16384)   # 64 KB blocks, r=2 needs 5 cells
    prob = oracle.make_problem(counts, 4, 0)
    send = [torch.zeros(int(b), dtype=torch.uint8, device="cuda") for b in prob.send_bytes]
    recv = [comm.symm_empty(int(b), torch.uint8) for b in prob.recv_bytes]
    comm.alltoallv(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo="rbruck", r=2,
                   type_size=4)
    assert comm.status()["name"] == "staging_capacity"
    comm.close()


def test_plan_errors_surface():
    from rbruck_alltoallv_b200.parallel.comm import CommError
    comm = get_comm(6)
    t = comm.symm_empty(64, torch.uint8)
    with pytest.raises(CommError):
        comm.alltoallv([t] * 6, [t] * 6, np.zeros((6, 6)), None, np.zeros((6, 6)), None, algo="xor")


EAGER = [("spreadout", {}), ("linear", {}), ("pairwise", {}), ("rbruck", dict(r=2)), ("rbruck", dict(r=3)),
         ("rbruck_om", dict(r=2)), ("tuna2", dict(r=2, b=0)), ("ttpl_bt_s1", dict(n=4, r=2)), ("ttpl", dict(n=2, r=2)),
         ("ttpl_bt", dict(n=4, r=2, b=1)), ("twolayer_linear_s2", dict(n=4, b=2, b2=3))]


@pytest.mark.parametrize("algo,kw", EAGER, ids=[f"{a}-{'-'.join(f'{k}{v}' for k, v in kw.items())}" for a, kw in EAGER])
@pytest.mark.parametrize("ts", [1, 4, 8])
def test_eager_protocol(algo, kw, ts):
    counts = dist.uniform(8, 700, seed=ts)
    counts[counts < 60] = 0
    run_case(8, algo, ts, counts, packed=False, seed=ts + 3, eager_max_bytes=700 * ts, **kw)


def test_eager_plain_receive_buffers_and_repeated_calls():
    P, ts = 8, 4
    comm = get_comm(P)
    for rep in range(5):
        counts = dist.zipf(P, 2048, seed=rep)
        prob = oracle.make_problem(counts, ts, rep, packed=True)
        send_h = oracle.fill_send(prob, rep)
        want = oracle.expected_recv(prob, send_h)
        send = [torch.from_numpy(b).cuda() for b in send_h]
        recv = [torch.full((len(w),), oracle.CANARY, dtype=torch.uint8, device="cuda") for w in want]   # not symmetric
        comm.alltoallv(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo="rbruck", r=2,
                       type_size=ts, eager_max_bytes=comm.max_block_bytes(prob.counts, ts))
        comm.check()
        assert oracle.first_mismatch([t.cpu().numpy() for t in recv], want) is None


def test_eager_rejects_oversize_block_on_the_host():
    from rbruck_alltoallv_b200.parallel.comm import CommError
    comm = get_comm(4)
    counts = dist.constant(4, 1000)
    prob = oracle.make_problem(counts, 4, 0)
    send = [torch.zeros(int(b), dtype=torch.uint8, device="cuda") for b in prob.send_bytes]
    recv = [comm.symm_empty(int(b), torch.uint8) for b in prob.recv_bytes]
    with pytest.raises(CommError):
        comm.alltoallv(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo="spreadout",
                       type_size=4, eager_max_bytes=1024)


def test_protocols_can_alternate_on_one_communicator():
    counts = dist.uniform(8, 300, seed=77)
    for i in range(6):
        run_case(8, "rbruck", 4, counts, seed=80 + i, r=2, eager_max_bytes=(1200 if i % 2 == 0 else 0))
        run_case(8, "spreadout", 4, counts, seed=90 + i, eager_max_bytes=(0 if i % 3 == 0 else 1200))


def test_plain_receive_buffers_go_through_a_bounce_buffer():
    P, ts = 8, 4
    comm = get_comm(P)
    counts = dist.uniform(P, 500, seed=5)
    prob = oracle.make_problem(counts, ts, 5, packed=False)
    send_h = oracle.fill_send(prob, 5)
    want = oracle.expected_recv(prob, send_h)
    send = [torch.from_numpy(b).cuda() for b in send_h]
    recv = [torch.full((len(w),), oracle.CANARY, dtype=torch.uint8, device="cuda") for w in want]   # torch allocations
    for algo, kw in (("spreadout", {}), ("rbruck", dict(r=2))):
        comm.alltoallv(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo=algo, type_size=ts, **kw)
        comm.check()
        assert oracle.first_mismatch([t.cpu().numpy() for t in recv], want) is None


def test_phase_timers_follow_the_reference_names():
    import ctypes as C
    comm = get_comm(8)
    lib = comm._lib
    comm.enable_trace(True)
    counts = dist.uniform(8, 2000, seed=9)
    run_case(8, "ttpl_bt", 8, counts, seed=9, n=4, r=2, b=1)
    lib.rbv_ctx_set_stream(comm._ctx, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert lib.rbv_update_timers(comm._ctx) == 0
    names = ["init_time", "findMax_time", "rotateIndex_time", "alcCopy_time", "getBlock_time", "prepData_time",
             "excgMeta_time", "excgData_time", "replace_time", "orgData_time", "prepSP_time", "SP_time", "intra_time"]
    vals = {n: C.c_double.in_dll(lib, n).value for n in names}
    assert all(v >= 0 for v in vals.values())
    assert vals["excgMeta_time"] > 0 and vals["excgData_time"] > 0 and vals["SP_time"] > 0
    assert vals["intra_time"] == vals["excgData_time"] and vals["alcCopy_time"] > 0
    assert vals["replace_time"] == 0 and vals["orgData_time"] == 0      # pack / unpack / organise no longer exist
    # two-layer linear: intra_time and one iteration_time entry per inter-group batch
    # (src/twolayer_communicator_linear.cpp:125-128,143,183)
    lib.rbv_iteration_count.restype = C.c_int
    for persistent in (False, True):
        run_case(8, "twolayer_linear_s2", 8, counts, seed=10, n=4, b=2, b2=2, persistent=persistent)
        assert lib.rbv_update_timers(comm._ctx) == 0
        nb = lib.rbv_iteration_count(comm._ctx)
        assert nb == 3                          # flat offsets 4..7 reach the other group: batches (f - 1) // 2 = 1, 2, 3
        it = C.POINTER(C.c_double).in_dll(lib, "iteration_time")
        assert C.c_double.in_dll(lib, "intra_time").value > 0 and C.c_double.in_dll(lib, "SP_time").value > 0
        assert all(it[i] > 0 for i in range(nb))
        C.CDLL(None).free(it)
    tr = comm.trace()
    assert {t["phase"] for t in tr} >= {1, 2} and all(t["end_us"] >= t["start_us"] for t in tr)
    # leader-routed exchange: gather, exchange and hand-out are phases 1, 2, 3
    run_case(8, "simple_merge", 8, counts, seed=11, n=4, persistent=True)
    assert lib.rbv_update_timers(comm._ctx) == 0
    assert C.c_double.in_dll(lib, "orgData_time").value > 0
    # eager protocol: unpacking is timed as replace_time
    run_case(8, "rbruck", 4, dist.uniform(8, 300, seed=1), seed=12, r=2, eager_max_bytes=1200)
    assert lib.rbv_update_timers(comm._ctx) == 0
    assert C.c_double.in_dll(lib, "replace_time").value > 0
    comm.enable_trace(False)


def test_functional_api_with_automatic_choice():
    from rbruck_alltoallv_b200.ops import alltoallv as A
    P, ts = 8, 2
    comm = get_comm(P)
    for hi in (40, 40000):                      # a latency-class and a bandwidth-class exchange
        counts = dist.uniform(P, hi, seed=hi)
        prob = oracle.make_problem(counts, ts, hi, packed=True)
        send_h = oracle.fill_send(prob, hi)
        want = oracle.expected_recv(prob, send_h)
        send = [torch.from_numpy(b).cuda() for b in send_h]
        recv = [comm.symm_empty(len(w), torch.uint8) for w in want]
        for t in recv:
            t.fill_(oracle.CANARY)
        A.alltoallv(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, comm=comm, algo="auto",
                    type_size=ts)
        comm.check()
        assert oracle.first_mismatch([t.cpu().numpy() for t in recv], want) is None
        for t in recv:
            t.fill_(oracle.CANARY)
        call = A.prepare(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, comm=comm, algo="auto",
                         type_size=ts)
        call.launch()
        call.launch()
        comm.check()
        assert oracle.first_mismatch([t.cpu().numpy() for t in recv], want) is None
    # uniform helper
    n = 100
    send = [torch.arange(P * n, dtype=torch.int32, device="cuda") + 1000 * r for r in range(P)]
    recv = [comm.symm_empty(P * n, torch.int32) for _ in range(P)]
    A.alltoall(send, recv, n, comm=comm)
    comm.check()
    for d in range(P):
        got = recv[d].cpu()
        for s in range(P):
            assert torch.equal(got[s * n:(s + 1) * n], torch.arange(d * n, (d + 1) * n, dtype=torch.int32) + 1000 * s)


def test_ulysses_sequence_head_exchange_round_trip():
    from rbruck_alltoallv_b200.ops.ulysses import UlyssesExchange
    P, s_l, H, D = 4, 24, 8, 16
    comm = get_comm(P)
    ex = UlyssesExchange(comm, s_l, H, D, dtype=torch.float32)
    g = torch.Generator(device="cuda").manual_seed(3)
    full = torch.randn(P * s_l, H, D, device="cuda", generator=g)                 # [S, H, D]
    x = [full[r * s_l:(r + 1) * s_l].contiguous() for r in range(P)]
    y = ex.seq_to_head(x)
    comm.check()
    for r in range(P):
        assert torch.equal(y[r], full[:, r * (H // P):(r + 1) * (H // P), :])
    back = ex.head_to_seq([t.clone() for t in y])
    comm.check()
    for r in range(P):
        assert torch.equal(back[r], x[r])


def test_more_than_64_ranks_run_as_persistent_calls():
    """Up to 1024 logical ranks (the size of the reference's largest recorded trace) run through the static kernel,
    which keeps no per-rank tables; one-shot calls of such communicators are refused with a clear message."""
    from rbruck_alltoallv_b200.parallel.comm import CommError, Communicator
    for P, algos in ((200, [("spreadout", {}), ("pairwise", {})]), (128, [("rbruck", dict(r=2)), ("ttpl_bt_s1", dict(n=16, r=4))])):
        comm = Communicator(nranks=P, heap_bytes=256 << 20, arena_bytes=1 << 20)
        try:
            counts = dist.uniform(P, 40, seed=P)
            counts[counts < 8] = 0
            prob = oracle.make_problem(counts, 4, P, packed=False)
            send_h = oracle.fill_send(prob, P)
            want = oracle.expected_recv(prob, send_h)
            send = [torch.from_numpy(b).cuda() for b in send_h]
            recv = [comm.symm_empty(len(w), torch.uint8) for w in want]
            for algo, kw in algos:
                for t in recv:
                    t.fill_(oracle.CANARY)
                call = comm.prepare(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo=algo,
                                    type_size=4, **kw)
                assert call.kind == "static"
                call.launch()
                call.launch()
                comm.check()
                assert oracle.first_mismatch([t.cpu().numpy() for t in recv], want) is None, (P, algo)
            with pytest.raises(CommError, match="persistent"):
                comm.alltoallv(send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls, algo="spreadout",
                               type_size=4)
        finally:
            comm.close()


def test_persistent_calls_replay_from_a_cuda_graph():
    """The call number lives in device memory, so a recorded launch can be replayed.  Direct launches get the number
    from the host as a shortcut; the first recorded launch switches that off for the context, because replays advance
    the number without the host seeing them.  Direct launches, replays and direct launches again must all deliver."""
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    P, ts = 8, 4
    comm = Communicator(nranks=P, heap_bytes=64 << 20, arena_bytes=2 << 20)
    try:
        counts = dist.uniform(P, 500, seed=12)
        prob = oracle.make_problem(counts, ts, 12, packed=False)
        send_h = oracle.fill_send(prob, 12)
        want = oracle.expected_recv(prob, send_h)
        send = [torch.from_numpy(b).cuda() for b in send_h]
        recv = [comm.symm_empty(len(w), torch.uint8) for w in want]
        args = (send, recv, prob.counts, prob.sdispls, prob.recvcounts, prob.rdispls)
        calls = [comm.prepare(*args, algo="spreadout", type_size=ts),
                 comm.prepare(*args, algo="spreadout", type_size=ts, eager_max_bytes=500 * ts)]
        assert [c.kind for c in calls] == ["static", "eager"]

        def verify(what):
            comm.check()
            assert oracle.first_mismatch([t.cpu().numpy() for t in recv], want) is None, what
            for t in recv:
                t.fill_(oracle.CANARY)

        for t in recv:
            t.fill_(oracle.CANARY)
        for c in calls:                       # direct launches with the host's call number
            c.launch()
            verify("direct " + c.kind)
        torch.cuda.synchronize()
        graphs = []
        for c in calls:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                c.launch()
            graphs.append(g)
        for rep in range(3):
            for g, c in zip(graphs, calls):
                g.replay()
                verify(f"replay {rep} " + c.kind)
        for c in calls:                       # and direct launches afterwards read the number on the device
            c.launch()
            verify("direct after replays " + c.kind)
    finally:
        comm.close()
