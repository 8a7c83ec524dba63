"""Small, self-terminating workloads of one kernel each, sized for profiler captures (inputs larger than the
126 MB L2, at most a few GB on the device, a handful of launches).

    python -m rbruck_alltoallv_b200.utils.profile_case a2av        # spread-out alltoallv, 8 ranks on one GPU, 4 MB blocks
                                                                   # (persistent call: the static kernel)
    python -m rbruck_alltoallv_b200.utils.profile_case a2av_bruck  # radix-2 two-phase Bruck, same sizes (static kernel,
                                                                   # chunk-granular forwarding)
    python -m rbruck_alltoallv_b200.utils.profile_case a2av_dynamic  # the same spread-out exchange through the kernel
                                                                   # that exchanges metadata itself
    python -m rbruck_alltoallv_b200.utils.profile_case a2av_small  # Zipf blocks <= 64 KB (latency regime)
    python -m rbruck_alltoallv_b200.utils.profile_case gemm1       # grouped SwiGLU GEMM, 2 experts x 2048 rows, 4096 -> 2 x 14336
    python -m rbruck_alltoallv_b200.utils.profile_case gemm2       # grouped down GEMM, 14336 -> 4096
    python -m rbruck_alltoallv_b200.utils.profile_case gemm_mx     # MXFP8 up/gate GEMM, SwiGLU + quantiser epilogue
    python -m rbruck_alltoallv_b200.utils.profile_case moe_mx      # MoE layer with MXFP8 experts (quantising dispatch, pushed combine)
    python -m rbruck_alltoallv_b200.utils.profile_case transpose   # fused pencil transpose, 384^3 complex64
    python -m rbruck_alltoallv_b200.utils.profile_case eager       # eager protocol, Zipf blocks <= 64 KB, radix 2
    python -m rbruck_alltoallv_b200.utils.profile_case moe         # MoE layer, 8192 tokens x 4096, 8 experts, FFN 1024
"""
from __future__ import annotations

import sys

import numpy as np
import torch


def _moe(fp8=False):
    from ..ops.moe import MoEExpertParallel
    from ..parallel.comm import Communicator
    T, H, I, E = 8192, 4096, 1024, 8
    comm = Communicator(nranks=1, heap_bytes=1 << 30, arena_bytes=1 << 20)
    layer = MoEExpertParallel(comm, E, H, I, T, capacity_factor=1.0, seed=1, fp8=fp8)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda")
    for _ in range(3):
        layer.forward(x, logits)
    layer.check()
    comm.close()


def _a2av(algo, small=False, **kw):
    from ..parallel.comm import Communicator
    from . import distributions as D
    P = 8
    comm = Communicator(nranks=P, heap_bytes=1 << 30, arena_bytes=40 << 20)
    counts = D.zipf(P, 16384, seed=1) if small else D.normal(P, 1 << 20, 0.25, seed=1)   # fp32 elements
    sc, rc = counts.astype(np.int32), counts.T.astype(np.int32).copy()
    send = [torch.zeros(max(int(sc[i].sum()), 1), dtype=torch.float32, device="cuda") for i in range(P)]
    recv = [comm.symm_empty(max(int(rc[i].sum()), 1), torch.float32) for i in range(P)]
    if kw.pop("eager", False):
        kw["eager_max_bytes"] = comm.max_block_bytes(sc, 4)
    call = comm.prepare(send, recv, sc, None, rc, None, algo=algo, **kw)
    for _ in range(4):
        call.launch()
    comm.check()
    comm.close()


def _gemm(which):
    from ..ops.moe import grouped_gemm
    G, rows, H, I = 2, 2048, 4096, 14336
    gs = torch.tensor([0, rows], dtype=torch.int32, device="cuda")
    gr = torch.tensor([rows, rows], dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    if which == 1:
        A = torch.randn(G * rows, H, device="cuda").to(torch.bfloat16)
        B = (torch.randn(G, 2 * I, H, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(G * rows, I, dtype=torch.bfloat16, device="cuda")
    else:
        A = torch.randn(G * rows, I, device="cuda").to(torch.bfloat16)
        B = (torch.randn(G, H, I, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(G * rows, H, dtype=torch.bfloat16, device="cuda")
    for _ in range(4):
        grouped_gemm(A, B, gs, gr, out=out, swiglu=(which == 1), error=err)
    torch.cuda.synchronize()
    assert err.item() == 0


def _gemm_fp8():
    from ..ops.moe import grouped_gemm_fp8, quantize_rows_fp8, quantize_weight_blocks_fp8
    G, rows, H, I = 2, 2048, 4096, 14336
    gs = torch.tensor([0, rows], dtype=torch.int32, device="cuda")
    gr = torch.tensor([rows, rows], dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    Aq, a_sc = quantize_rows_fp8(torch.randn(G * rows, H, device="cuda").to(torch.bfloat16))
    Bq, b_sc = quantize_weight_blocks_fp8((torch.randn(G, 2 * I, H, device="cuda") * 0.02).to(torch.bfloat16))
    out = torch.empty(G * rows, I, dtype=torch.bfloat16, device="cuda")
    for _ in range(4):
        grouped_gemm_fp8(Aq, a_sc, Bq, b_sc, gs, gr, out=out, swiglu=True, error=err)
    torch.cuda.synchronize()
    assert err.item() == 0


def _gemm_mx():
    from ..ops.moe import grouped_gemm_mxfp8_swiglu_q, quantize_rows_mxfp8, quantize_weight_mxfp8
    G, rows, H, I = 2, 2048, 4096, 14336
    gs = torch.tensor([0, rows], dtype=torch.int32, device="cuda")
    gr = torch.tensor([rows, rows], dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    Aq, sfa = quantize_rows_mxfp8(torch.randn(G * rows, H, device="cuda").to(torch.bfloat16))
    Bq, sfb = quantize_weight_mxfp8((torch.randn(G, 2 * I, H, device="cuda") * 0.02).to(torch.bfloat16))
    hq = torch.empty(G * rows, I, dtype=torch.uint8, device="cuda")
    hs = torch.empty(I // 128, G * rows, dtype=torch.int32, device="cuda")
    for _ in range(4):
        grouped_gemm_mxfp8_swiglu_q(Aq, sfa, Bq, sfb, gs, gr, out_q=hq, out_sf=hs, error=err)
    torch.cuda.synchronize()
    assert err.item() == 0


def _transpose():
    from ..ops.fft import PencilTranspose
    from ..parallel.comm import Communicator
    n = 384
    comm = Communicator(nranks=1, heap_bytes=(n ** 3 * 8) * 2 + (64 << 20), arena_bytes=1 << 20)
    tp = PencilTranspose(comm, n, 1, 1, seed=1)
    src = torch.view_as_complex(torch.randn(n, n, n, 2, device="cuda"))
    for _ in range(4):
        tp.x_to_y(src)
    tp.check()
    comm.close()


def main() -> int:
    case = sys.argv[1] if len(sys.argv) > 1 else "a2av"
    if case == "a2av":
        _a2av("spreadout")
    elif case == "a2av_bruck":
        _a2av("rbruck", r=2)
    elif case == "a2av_dynamic":
        _a2av("spreadout", static=False)
    elif case == "a2av_small":
        _a2av("rbruck", small=True, r=2)
    elif case == "gemm1":
        _gemm(1)
    elif case == "gemm2":
        _gemm(2)
    elif case == "gemm_fp8":
        _gemm_fp8()
    elif case == "gemm_mx":
        _gemm_mx()
    elif case == "transpose":
        _transpose()
    elif case == "eager":
        _a2av("rbruck", small=True, r=2, eager=True)
    elif case == "moe":
        _moe()
    elif case == "moe_mx":
        _moe(fp8="mx")
    else:
        raise SystemExit("unknown case")
    print("case", case, "done")
    return 0


if __name__ == "__main__":
    sys.exit(main())
