"""Device-timed benchmark of the MoE expert-parallel layer (and of its grouped GEMMs alone).

    python -m rbruck_alltoallv_b200.utils.moe_bench [--tokens 8192 --hidden 4096 --inter 14336 --experts-per-rank 8]
    torchrun --nproc-per-node N --master-addr 127.0.0.1 -m rbruck_alltoallv_b200.utils.moe_bench

Prints one JSON line on rank 0: per-stage times (max over ranks), achieved TFLOP/s of the expert FFN and the
fraction of the measured bf16 matmul peak (``MEASURED_PEAKS.json`` beside the repository root when present).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

from ..ops.moe import MoEExpertParallel, grouped_gemm, reference_forward
from ..parallel.comm import Communicator


def _peaks():
    for p in (Path.cwd() / "MEASURED_PEAKS.json", Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"):
        if p.exists():
            d = json.loads(p.read_text())
            return {"bf16_tflops": d.get("bf16_tflops"), "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                    "hbm_gbs": d.get("hbm_gbs"), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def _time(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s, e in ev:
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) for s, e in ev], dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size() > 1:
        tt = t.cuda()
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t = tt.cpu()
    return t.numpy()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--experts-per-rank", type=int, default=8)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--fp8", action="store_true", help="expert GEMMs in block-scaled e4m3 (1x128 / 128x128 scales)")
    ap.add_argument("--mx", action="store_true",
                    help="expert GEMMs in MXFP8 (e4m3, power-of-two scales per 32 elements, scaled by the tensor core)")
    ap.add_argument("--check", action="store_true", help="compare with the fp32 reference (small sizes only)")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    T, H, I, El = a.tokens, a.hidden, a.inter, a.experts_per_rank
    cap_rows = int(np.ceil(2.0 * 2 * T / 128.0)) * 128
    heap = 2 * (cap_rows + 128 * El) * H * 2 + (64 << 20)
    comm = Communicator(nranks=world, heap_bytes=heap, arena_bytes=1 << 20)
    E = El * world
    layer = MoEExpertParallel(comm, E, H, I, T, seed=3, fp8="mx" if a.mx else a.fp8)
    g = torch.Generator(device="cuda")
    g.manual_seed(100 + comm.proc)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda", generator=g)
    out = torch.empty_like(x)
    layer.forward(x, logits, out)
    layer.check()
    rows = int(layer.totals[0].item())
    res = {"gpus": world, "expert_gemm_dtype": "mxfp8" if a.mx else ("fp8_e4m3_block_scaled" if a.fp8 else "bf16"), "tokens_per_gpu": T, "hidden": H, "inter": I, "experts": E, "rows_received_rank0": rows}
    if a.check:
        if world > 1:
            w13 = [torch.empty_like(layer.w13) for _ in range(world)]
            w2 = [torch.empty_like(layer.w2) for _ in range(world)]
            dist.all_gather(w13, layer.w13)
            dist.all_gather(w2, layer.w2)
            w13, w2 = torch.cat(w13), torch.cat(w2)
        else:
            w13, w2 = layer.w13, layer.w2
        ref, _, _ = reference_forward(x, logits, w13, w2)
        err = (out.float() - ref).abs().max().item()
        res["max_abs_err"] = err
        res["ref_scale"] = ref.abs().max().item()
        tol = 0.25 if (a.fp8 or a.mx) else 0.02      # fp8 operands: compared against the unquantised bf16 weights
        res["check"] = "ok" if err <= tol * res["ref_scale"] + 1e-3 else "FAILED"
    t_all = _time(lambda: layer.forward(x, logits, out), a.steps, a.warmup)
    layer.check()
    if a.mx:
        from ..ops.moe import grouped_gemm_mxfp8, quantize_rows_mxfp8
        if layer.qdispatch:      # the dispatch delivered quantised rows
            xq, xs = layer.xq, layer.xs
        else:
            xq, xs = quantize_rows_mxfp8(layer.xrecv)
            t_q = _time(lambda: quantize_rows_mxfp8(layer.xrecv), a.steps, a.warmup)
            res["ms_quantize_x"] = float(np.median(t_q))
        hq, hs = (layer._hq, layer._hs) if getattr(layer, "_hq", None) is not None else quantize_rows_mxfp8(layer.h)
        t_g1 = _time(lambda: grouped_gemm_mxfp8(xq, xs, layer.w13_q, layer.w13_s, layer.group_start, layer.group_rows,
                                                out=layer.h, swiglu=True, error=layer.error[1:2]), a.steps, a.warmup)
        t_g2 = _time(lambda: grouped_gemm_mxfp8(hq, hs, layer.w2_q, layer.w2_s, layer.group_start, layer.group_rows,
                                                out=layer.y, error=layer.error[2:3]), a.steps, a.warmup)
    elif a.fp8:
        from ..ops.moe import grouped_gemm_fp8, quantize_rows_fp8
        xq, xs = quantize_rows_fp8(layer.xrecv)
        hq, hs = quantize_rows_fp8(layer.h)
        t_q = _time(lambda: quantize_rows_fp8(layer.xrecv), a.steps, a.warmup)
        res["ms_quantize_x"] = float(np.median(t_q))
        t_g1 = _time(lambda: grouped_gemm_fp8(xq, xs, layer.w13_q, layer.w13_s, layer.group_start, layer.group_rows,
                                              out=layer.h, swiglu=True, error=layer.error[1:2]), a.steps, a.warmup)
        t_g2 = _time(lambda: grouped_gemm_fp8(hq, hs, layer.w2_q, layer.w2_s, layer.group_start, layer.group_rows,
                                              out=layer.y, error=layer.error[2:3]), a.steps, a.warmup)
        # the same operands with scales taken as constant along K: what the tile shape allows without the
        # per-K-block rescaling (timing only; the layer itself uses the block scales)
        t_c = _time(lambda: grouped_gemm_fp8(xq, xs, layer.w13_q, layer.w13_s, layer.group_start, layer.group_rows,
                                             out=layer.h, swiglu=True, error=layer.error[1:2], coarse=True), a.steps, a.warmup)
        res["ms_gemm1_coarse_scales"] = float(np.median(t_c))
    else:
        t_g1 = _time(lambda: grouped_gemm(layer.xrecv, layer.w13, layer.group_start, layer.group_rows, out=layer.h,
                                          swiglu=True, error=layer.error[1:2]), a.steps, a.warmup)
        t_g2 = _time(lambda: grouped_gemm(layer.h, layer.w2, layer.group_start, layer.group_rows, out=layer.y,
                                          error=layer.error[2:3]), a.steps, a.warmup)
    layer.check()
    rows_t = torch.tensor([rows], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(rows_t, op=dist.ReduceOp.MAX)
    rows_max = int(rows_t.item())
    pk = _peaks()
    f1, f2 = rows_max * 2.0 * H * 2 * I, rows_max * 2.0 * I * H
    ms_all, ms1, ms2 = float(np.median(t_all)), float(np.median(t_g1)), float(np.median(t_g2))
    res.update({"rows_max_over_ranks": rows_max, "ms_layer": ms_all, "ms_gemm1_swiglu": ms1, "ms_gemm2": ms2,
                "tflops_gemm1": f1 / ms1 / 1e9, "tflops_gemm2": f2 / ms2 / 1e9,
                "tflops_layer": (f1 + f2) / ms_all / 1e9, "peaks": pk})
    dispatch_bytes = rows_max * H * 2.0 * (world - 1) / max(world, 1)
    roof_ms = max((f1 + f2) / (pk["bf16_tflops_sustained"] * 1e9), 2 * dispatch_bytes / 770e9 * 1e3)
    res["roofline_ms"] = roof_ms
    res["fraction_of_roofline"] = roof_ms / ms_all
    res["gemm1_fraction_of_burst_peak"] = res["tflops_gemm1"] / pk["bf16_tflops"]
    res["gemm2_fraction_of_burst_peak"] = res["tflops_gemm2"] / pk["bf16_tflops"]
    if comm.proc == 0:
        print(json.dumps(res), flush=True)
        if a.out:
            with open(a.out, "a") as fh:
                fh.write(json.dumps(res) + "\n")
    comm.close()
    if world > 1:
        dist.destroy_process_group()
    return 0 if res.get("check", "ok") == "ok" else 1


if __name__ == "__main__":
    sys.exit(main())
