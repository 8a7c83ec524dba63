"""GPU tests of the MoE path: grouped tcgen05 GEMM, router, and the full dispatch/FFN/combine layer."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _groups_aligned(rows, device, align=128):
    """Group starts at multiples of `align` rows; returns (start, rows, rows of the whole buffer)."""
    start, at = [], 0
    for n in rows:
        start.append(at)
        at += (n + align - 1) // align * align
    total = start[-1] + rows[-1] if rows else 0
    return (torch.tensor(start, dtype=torch.int32, device=device),
            torch.tensor(rows, dtype=torch.int32, device=device), max(total, 1), start)


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


def test_mxfp8_quantiser_matches_the_torch_recipe():
    from rbruck_alltoallv_b200.ops import moe
    torch.manual_seed(11)
    x = (torch.randn(300, 256, device="cuda") * torch.rand(300, 1, device="cuda") * 5).to(torch.bfloat16)
    x[7] = 0
    x[9, :32] = 448.0          # amax / 448 an exact power of two
    q, sf = moe.quantize_rows_mxfp8(x)
    torch.cuda.synchronize()
    e = moe._mx_exponents(x.float().view(300, 8, 32).abs().amax(dim=2))            # [rows, K/32]
    want_bytes = (e.to(torch.int64) + 127).view(300, 2, 4)
    want_words = (want_bytes[..., 0] | (want_bytes[..., 1] << 8) | (want_bytes[..., 2] << 16) | (want_bytes[..., 3] << 24))
    assert torch.equal(moe.mx_from_atoms(sf, 300).t().contiguous(), want_words.to(torch.int32))
    d = moe.dequantize_rows_mxfp8(q, sf)
    assert (d - x.float()).abs().max().item() <= 0.07 * x.float().abs().max().item()
    # per-block relative error of e4m3 with a scale that keeps amax in (224, 448]: at most 2^-4 of the block's amax
    blk_err = (d - x.float()).view(300, 8, 32).abs().amax(dim=2)
    blk_max = x.float().view(300, 8, 32).abs().amax(dim=2)
    assert torch.all(blk_err <= blk_max / 16 + 1e-6)


@pytest.mark.parametrize("scales", ["ones", "rows", "kblocks", "columns", "real"])
def test_grouped_gemm_mxfp8_scale_paths(scales):
    """Hardware block scaling, one source of scale variation at a time: no scaling at all, per activation row, per
    32-block of K, per weight row, and the quantisers' own scales."""
    from rbruck_alltoallv_b200.ops import moe
    torch.manual_seed(21)
    rows, N, K = [300, 0, 129, 700], 256, 512
    G = len(rows)
    gs, gr, M, starts = _groups_aligned(rows, "cuda")
    if scales == "real":
        A = (torch.randn(M, K, device="cuda") * torch.rand(M, 1, device="cuda") * 3).to(torch.bfloat16)
        B = (torch.randn(G, N, K, device="cuda") * 0.05).to(torch.bfloat16)
        Aq, sfa = moe.quantize_rows_mxfp8(A)
        Bq, sfb = moe.quantize_weight_mxfp8(B)
    else:
        Aq = torch.randn(M, K, device="cuda").clamp(-3, 3).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
        Bq = torch.randn(G, N, K, device="cuda").clamp(-3, 3).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
        ea = torch.zeros(K // 32, M, dtype=torch.int32, device="cuda")          # exponents, [K/32][rows]
        eb = torch.zeros(G, K // 32, N, dtype=torch.int32, device="cuda")
        if scales == "rows":
            ea += (torch.arange(M, device="cuda", dtype=torch.int32) % 7 - 3)[None, :]
        elif scales == "kblocks":
            ea += (torch.arange(K // 32, device="cuda", dtype=torch.int32) % 5 - 2)[:, None]
            eb += (torch.arange(K // 32, device="cuda", dtype=torch.int32) % 3 - 1)[None, :, None]
        elif scales == "columns":
            eb += (torch.arange(N, device="cuda", dtype=torch.int32) % 9 - 4)[None, None, :]

        def pack(e4):
            b = e4.to(torch.int64) + 127
            return b[..., 0, :] | (b[..., 1, :] << 8) | (b[..., 2, :] << 16) | (b[..., 3, :] << 24)
        sfa = moe.mx_to_atoms(pack(ea.view(K // 128, 4, M)))
        sfb = moe.mx_to_atoms(pack(eb.view(G, K // 128, 4, N)))
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    moe.grouped_gemm_mxfp8(Aq, sfa, Bq, sfb, gs, gr, out=out, error=err)
    torch.cuda.synchronize()
    assert err.item() == 0
    Ad, Bd = moe.dequantize_rows_mxfp8(Aq, sfa), moe.dequantize_weight_mxfp8(Bq, sfb)
    used = torch.zeros(M, dtype=torch.bool, device="cuda")
    for g, n in enumerate(rows):
        r0 = starts[g]
        used[r0:r0 + n] = True
        if n:
            ref = Ad[r0:r0 + n] @ Bd[g].t()
            got = out[r0:r0 + n].float()
            assert (got - ref).abs().max().item() <= 0.01 * ref.abs().max().item() + 1e-3, f"group {g} ({scales})"
    assert torch.all(out[~used] == 7.0), "rows between the groups must stay untouched"


def test_grouped_gemm_mxfp8_refuses_unaligned_groups():
    from rbruck_alltoallv_b200.ops import moe
    rows, N, K = [100, 50], 128, 128
    gs, gr = _groups(rows, "cuda")                      # the second group starts at row 100
    Aq = torch.zeros(150, K, dtype=torch.uint8, device="cuda")
    Bq = torch.zeros(2, N, K, dtype=torch.uint8, device="cuda")
    sfa = moe.mx_to_atoms(torch.full((K // 128, 150), 0x7f7f7f7f, dtype=torch.int32, device="cuda"))
    sfb = moe.mx_to_atoms(torch.full((2, K // 128, N), 0x7f7f7f7f, dtype=torch.int32, device="cuda"))
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    moe.grouped_gemm_mxfp8(Aq, sfa, Bq, sfb, gs, gr, error=err)
    torch.cuda.synchronize()
    assert err.item() == 5


def test_grouped_gemm_mxfp8_many_tiles_and_swiglu():
    from rbruck_alltoallv_b200.ops import moe
    torch.manual_seed(22)
    rows, I, K = [1500, 129, 700], 1024, 2048
    G = len(rows)
    gs, gr, M, starts = _groups_aligned(rows, "cuda")
    A = (torch.randn(M, K, device="cuda") * torch.rand(M, 1, device="cuda") * 2).to(torch.bfloat16)
    gate = (torch.randn(G, I, K, device="cuda") * 0.03).to(torch.bfloat16)
    up = (torch.randn(G, I, K, device="cuda") * 0.03).to(torch.bfloat16)
    Aq, sfa = moe.quantize_rows_mxfp8(A)
    Bq, sfb = moe.quantize_weight_mxfp8(moe.pack_gate_up(gate, up))
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = moe.grouped_gemm_mxfp8(Aq, sfa, Bq, sfb, gs, gr, swiglu=True, error=err)
    torch.cuda.synchronize()
    assert err.item() == 0
    Ad, Bd = moe.dequantize_rows_mxfp8(Aq, sfa), moe.dequantize_weight_mxfp8(Bq, sfb)
    for g, n in enumerate(rows):
        r0 = starts[g]
        a = Ad[r0:r0 + n]
        ref = torch.nn.functional.silu(a @ Bd[g, 0::2].t()) * (a @ Bd[g, 1::2].t())
        assert (out[r0:r0 + n].float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-3, f"group {g}"


def test_grouped_gemm_mxfp8_fused_output_quantiser_matches_the_separate_one():
    """SwiGLU + quantisation in the epilogue: the same bytes and scales as quantising the bf16 result would give,
    up to the rounding of that intermediate to bf16."""
    from rbruck_alltoallv_b200.ops import moe
    torch.manual_seed(23)
    rows, I, K = [700, 129, 300], 512, 1024
    G = len(rows)
    gs, gr, M, starts = _groups_aligned(rows, "cuda")
    A = (torch.randn(M, K, device="cuda") * torch.rand(M, 1, device="cuda") * 2).to(torch.bfloat16)
    gate = (torch.randn(G, I, K, device="cuda") * 0.03).to(torch.bfloat16)
    up = (torch.randn(G, I, K, device="cuda") * 0.03).to(torch.bfloat16)
    Aq, sfa = moe.quantize_rows_mxfp8(A)
    Bq, sfb = moe.quantize_weight_mxfp8(moe.pack_gate_up(gate, up))
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    hq = torch.zeros(M, I, dtype=torch.uint8, device="cuda")
    hs = moe.mx_to_atoms(torch.full((I // 128, M), 0x7f7f7f7f, dtype=torch.int32, device="cuda"))
    moe.grouped_gemm_mxfp8_swiglu_q(Aq, sfa, Bq, sfb, gs, gr, out_q=hq, out_sf=hs, error=err)
    h_bf16 = moe.grouped_gemm_mxfp8(Aq, sfa, Bq, sfb, gs, gr, swiglu=True, error=err)
    torch.cuda.synchronize()
    assert err.item() == 0
    fused = moe.dequantize_rows_mxfp8(hq, hs)
    for g, n in enumerate(rows):
        r0 = starts[g]
        ref = h_bf16[r0:r0 + n].float()
        got = fused[r0:r0 + n]
        # e4m3 keeps 3 mantissa bits: every value within 1/16 of its 32-block's largest magnitude
        blk = ref.view(n, I // 32, 32).abs().amax(dim=2, keepdim=True).expand(n, I // 32, 32).reshape(n, I)
        assert torch.all((got - ref).abs() <= blk / 16 + 1e-6), f"group {g}"
        # and the scales are the smallest powers of two that keep the block inside e4m3 (a bf16 rounding of the
        # largest value may move a block across a power of two: allow one step)
        e_ref = moe._mx_exponents(ref.view(n, I // 32, 32).abs().amax(dim=2))
        words = moe.mx_from_atoms(hs, M)[:, r0:r0 + n]                                  # [I/128, n]
        e_got = torch.stack([((words.to(torch.int64) >> (8 * j)) & 0xFF) - 127 for j in range(4)], dim=-1)
        e_got = e_got.permute(1, 0, 2).reshape(n, I // 32)
        assert (e_got - e_ref).abs().max().item() <= 1


def test_moe_layer_mxfp8_close_to_bf16():
    from rbruck_alltoallv_b200.ops.moe import MoEExpertParallel, reference_forward
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    comm = Communicator(nranks=1, heap_bytes=256 << 20, arena_bytes=1 << 20)
    try:
        T, H, I, E = 512, 512, 1024, 4
        layer = MoEExpertParallel(comm, E, H, I, T, seed=5, fp8="mx")
        g = torch.Generator(device="cuda")
        g.manual_seed(17)
        x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
        logits = torch.randn(T, E, device="cuda", generator=g)
        out = layer.forward(x, logits)
        layer.check()
        ref, _, _ = reference_forward(x, logits, layer.w13, layer.w2)
        rel = (out.float() - ref).norm().item() / ref.norm().item()
        assert rel < 0.08, f"MXFP8 layer deviates {rel:.3f} from the bf16 reference"
    finally:
        comm.close()


@pytest.mark.parametrize("fp8", [False, "mx"], ids=["bf16", "mxfp8"])
def test_moe_push_combine_equals_pull_combine(fp8):
    """The down GEMM that stores its rows straight into the token owners' buffers gives the same layer output as the
    combine that pulls them afterwards."""
    from rbruck_alltoallv_b200.ops.moe import MoEExpertParallel
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    comm = Communicator(nranks=1, heap_bytes=256 << 20, arena_bytes=1 << 20)
    try:
        T, H, I, E = 700, 512, 1024, 4
        g = torch.Generator(device="cuda")
        g.manual_seed(31)
        x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
        logits = torch.randn(T, E, device="cuda", generator=g)
        outs = []
        for push in (True, False):
            layer = MoEExpertParallel(comm, E, H, I, T, seed=9, fp8=fp8, push_combine=push)
            assert layer.push == push
            outs.append(layer.forward(x, logits).clone())
            layer.check()
            del layer
        assert torch.equal(outs[0], outs[1])
    finally:
        comm.close()


def test_moe_mx_quantising_dispatch_equals_the_quantiser_pass(monkeypatch):
    """Rows quantised by the dispatch itself (e4m3 + scale words over the wire) give the same layer output, bit for
    bit, as bf16 rows quantised on arrival."""
    from rbruck_alltoallv_b200.ops.moe import MoEExpertParallel
    from rbruck_alltoallv_b200.parallel.comm import Communicator
    comm = Communicator(nranks=1, heap_bytes=256 << 20, arena_bytes=1 << 20)
    try:
        T, H, I, E = 700, 640, 1024, 4            # H / 128 = 5 scale words per row: an odd count
        g = torch.Generator(device="cuda")
        g.manual_seed(41)
        x = (torch.randn(T, H, device="cuda", generator=g) * 3).to(torch.bfloat16)
        x[5] = 0
        logits = torch.randn(T, E, device="cuda", generator=g)
        outs = []
        for q in ("1", "0"):
            monkeypatch.setenv("RBV_MOE_QDISPATCH", q)
            layer = MoEExpertParallel(comm, E, H, I, T, seed=9, fp8="mx")
            assert layer.qdispatch == (q == "1")
            outs.append(layer.forward(x, logits).clone())
            layer.check()
            del layer
        assert torch.equal(outs[0], outs[1])
    finally:
        comm.close()


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
