"""GPU tests of the MoE path: grouped tcgen05 GEMM, router, and the full dispatch/FFN/combine layer."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _groups(rows, device):
    start = np.concatenate([[0], np.cumsum(rows)[:-1]]).astype(np.int32)
    return (torch.from_numpy(start).to(device), torch.from_numpy(np.asarray(rows, dtype=np.int32)).to(device))


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("rows,N,K", [([128, 128], 256, 64), ([100, 37, 0, 300], 256, 128), ([513, 64, 1], 512, 256),
                                      ([1000, 24], 1024, 512), ([2000, 129, 1500], 2048, 1024)])
def test_grouped_gemm_matches_fp32(rows, N, K, pair):
    from rbruck_alltoallv_b200.ops.moe import grouped_gemm
    torch.manual_seed(0)
    G, M = len(rows), int(sum(rows))
    A = torch.randn(M + 5, K, device="cuda").to(torch.bfloat16)
    B = (torch.randn(G, N, K, device="cuda") * 0.1).to(torch.bfloat16)
    gs, gr = _groups(rows, "cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((M + 5, N), 7.0, dtype=torch.bfloat16, device="cuda")
    grouped_gemm(A, B, gs, gr, out=out, error=err, pair=pair)
    torch.cuda.synchronize()
    assert err.item() == 0
    r0 = 0
    for g, n in enumerate(rows):
        ref = A[r0:r0 + n].float() @ B[g].float().t()
        got = out[r0:r0 + n].float()
        tol = 0.02 * ref.abs().max().item() + 1e-3 if n else 0
        assert n == 0 or (got - ref).abs().max().item() <= tol, f"group {g}"
        r0 += n
    assert torch.all(out[M:] == 7.0), "rows beyond the last group must stay untouched"


@pytest.mark.parametrize("pair", [False, True])
def test_grouped_gemm_swiglu(pair):
    from rbruck_alltoallv_b200.ops.moe import grouped_gemm, pack_gate_up
    torch.manual_seed(1)
    rows, I, K = [200, 56], 256, 128
    M = sum(rows)
    A = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    gate = (torch.randn(2, I, K, device="cuda") * 0.1).to(torch.bfloat16)
    up = (torch.randn(2, I, K, device="cuda") * 0.1).to(torch.bfloat16)
    gs, gr = _groups(rows, "cuda")
    out = grouped_gemm(A, pack_gate_up(gate, up), gs, gr, swiglu=True, pair=pair)
    torch.cuda.synchronize()
    r0 = 0
    for g, n in enumerate(rows):
        a = A[r0:r0 + n].float()
        ref = torch.nn.functional.silu(a @ gate[g].float().t()) * (a @ up[g].float().t())
        assert (out[r0:r0 + n].float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-3
        r0 += n


def test_router_top2():
    import ctypes as C
    from rbruck_alltoallv_b200 import _native
    lib = _native.cuda_lib()
    T, E = 1000, 64
    torch.manual_seed(2)
    logits = torch.randn(T, E, device="cuda")
    idx = torch.empty(T, 2, dtype=torch.int32, device="cuda")
    w = torch.empty(T, 2, device="cuda")
    hist = torch.empty(E, dtype=torch.int32, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    assert lib.rbv_moe_route(p(logits), T, E, p(idx), p(w), p(hist), None) == 0
    torch.cuda.synchronize()
    pr = torch.softmax(logits, -1)
    tp, ti = torch.topk(pr, 2, dim=-1)
    assert torch.equal(ti.int(), idx)
    assert torch.allclose(w, tp / tp.sum(-1, keepdim=True), atol=1e-5)
    assert torch.equal(hist.long(), torch.bincount(ti.reshape(-1), minlength=E))


def test_moe_layer_single_gpu():
    from rbruck_alltoallv_b200.models.moe_layer import smoke_moe
    smoke_moe()


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("rows,N,K", [([128], 128, 128), ([100, 37, 0, 300], 256, 256), ([513, 64], 512, 1024),
                                      ([1500, 129, 700], 2048, 2048)])
def test_grouped_gemm_fp8_block_scaled(rows, N, K, pair):
    from rbruck_alltoallv_b200.ops import moe
    torch.manual_seed(3)
    G, M = len(rows), int(sum(rows))
    A = (torch.randn(M, K, device="cuda") * torch.rand(M, 1, device="cuda") * 3).to(torch.bfloat16)
    B = (torch.randn(G, N, K, device="cuda") * 0.05).to(torch.bfloat16)
    Aq, As = moe.quantize_rows_fp8(A)
    Bq, Bs = moe.quantize_weight_blocks_fp8(B)
    # the quantiser itself: dequantised values within e4m3 precision of the input
    assert (moe.dequantize_rows_fp8(Aq, As) - A.float()).abs().max().item() <= 0.07 * A.float().abs().max().item()
    gs, gr = _groups(rows, "cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = moe.grouped_gemm_fp8(Aq, As, Bq, Bs, gs, gr, error=err, pair=pair)
    torch.cuda.synchronize()
    assert err.item() == 0
    Ad, Bd = moe.dequantize_rows_fp8(Aq, As), moe.dequantize_weight_blocks_fp8(Bq, Bs)
    r0 = 0
    for g, n in enumerate(rows):
        if n:
            ref = Ad[r0:r0 + n] @ Bd[g].t()          # exact product of the quantised operands, fp32
            got = out[r0:r0 + n].float()
            assert (got - ref).abs().max().item() <= 0.01 * ref.abs().max().item() + 1e-3, f"group {g}"
        r0 += n


@pytest.mark.parametrize("pair", [False, True])
def test_grouped_gemm_fp8_coarse_scales(pair):
    """Scales that are constant along K: the whole tile is accumulated in TMEM and scaled once."""
    from rbruck_alltoallv_b200.ops import moe
    torch.manual_seed(5)
    rows, N, K = [200, 0, 131], 256, 512
    G, M = len(rows), int(sum(rows))
    Aq = torch.randn(M, K, device="cuda").clamp(-3, 3).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    Bq = torch.randn(G, N, K, device="cuda").clamp(-3, 3).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    As = (torch.rand(1, M, device="cuda") + 0.5).expand(K // 128, M).contiguous()
    Bs = (torch.rand(G, N // 128, 1, device="cuda") * 0.1 + 0.01).expand(G, N // 128, K // 128).contiguous()
    gs, gr = _groups(rows, "cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    fine = moe.grouped_gemm_fp8(Aq, As, Bq, Bs, gs, gr, error=err, pair=pair)
    coarse = moe.grouped_gemm_fp8(Aq, As, Bq, Bs, gs, gr, error=err, coarse=True, pair=pair)
    torch.cuda.synchronize()
    assert err.item() == 0
    Ad, Bd = moe.dequantize_rows_fp8(Aq, As), moe.dequantize_weight_blocks_fp8(Bq, Bs)
    r0 = 0
    for g, n in enumerate(rows):
        if n:
            ref = Ad[r0:r0 + n] @ Bd[g].t()
            for got in (fine[r0:r0 + n].float(), coarse[r0:r0 + n].float()):
                assert (got - ref).abs().max().item() <= 0.01 * ref.abs().max().item() + 1e-3, f"group {g}"
        r0 += n


def test_moe_layer_fp8_close_to_bf16():
    from rbruck_alltoallv_b200.ops.moe import MoEExpertParallel, reference_forward
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    comm = Communicator(nranks=1, heap_bytes=256 << 20, arena_bytes=1 << 20)
    try:
        T, H, I, E = 256, 256, 512, 8
        layer = MoEExpertParallel(comm, E, H, I, T, seed=1, fp8=True)
        g = torch.Generator(device="cuda")
        g.manual_seed(7)
        x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
        logits = torch.randn(T, E, device="cuda", generator=g)
        out = layer.forward(x, logits)
        layer.check()
        ref, _, _ = reference_forward(x, logits, layer.w13, layer.w2)
        rel = (out.float() - ref).norm().item() / ref.norm().item()
        assert rel < 0.08, f"fp8 layer deviates {rel:.3f} from the bf16 reference"
    finally:
        comm.close()


def test_gated_gemm_waits_for_its_rows_and_gives_up_after_the_deadline():
    """The loader of the gated GEMM takes a group only when its delivery counter has reached the target.  Counters that
    are already complete change nothing; a counter that nothing ever bumps makes the bounded wait run out: the kernel
    sets its error flag, frees its TMEM and returns (no fault, the context stays usable)."""
    from rbruck_alltoallv_b200.ops.moe import grouped_gemm
    torch.manual_seed(4)
    rows, N, K = [130, 70], 256, 128
    M = sum(rows)
    A = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    B = (torch.randn(2, N, K, device="cuda") * 0.1).to(torch.bfloat16)
    gs, gr = _groups(rows, "cuda")
    want = grouped_gemm(A, B, gs, gr)
    ready = torch.tensor([130, 70], dtype=torch.int64, device="cuda")
    target = torch.tensor([130, 70], dtype=torch.int64, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = grouped_gemm(A, B, gs, gr, error=err, ready=ready, ready_target=target)
    torch.cuda.synchronize()
    assert err.item() == 0 and torch.equal(got, want)
    target[1] = 71                                            # one row that never arrives
    grouped_gemm(A, B, gs, gr, error=err, ready=ready, ready_target=target, timeout_ms=50.0)
    torch.cuda.synchronize()
    assert err.item() != 0
    err.zero_()
    assert torch.equal(grouped_gemm(A, B, gs, gr, error=err), want) and err.item() == 0


@pytest.mark.parametrize("overlap", [False, True])
def test_moe_layer_streamed_dispatch_matches_reference(overlap):
    from rbruck_alltoallv_b200.ops.moe import MoEExpertParallel, reference_forward
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    comm = Communicator(nranks=1, heap_bytes=256 << 20, arena_bytes=1 << 20)
    try:
        T, H, I, E = 384, 256, 512, 8
        layer = MoEExpertParallel(comm, E, H, I, T, seed=2, overlap=overlap)
        assert layer.overlap == overlap
        g = torch.Generator(device="cuda")
        g.manual_seed(9)
        for rep in range(3):                   # the delivery counters run on from call to call
            x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
            logits = torch.randn(T, E, device="cuda", generator=g)
            out = layer.forward(x, logits)
            layer.check()
            ref, _, _ = reference_forward(x, logits, layer.w13, layer.w2)
            assert (out.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-3, (overlap, rep)
    finally:
        comm.close()
