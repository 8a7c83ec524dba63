"""Expert-parallel MoE forward on the symmetric heap: router -> dispatch -> grouped SwiGLU FFN -> combine.

Kernels: ``csrc/kernels/moe_kernels.cu`` (router, layout, dispatch fused with the token permute, combine
fused with the gate-weighted sum) and ``csrc/kernels/grouped_gemm_sm100.cu`` (tcgen05 / TMEM grouped GEMM
fed by TMA).  The reference library has no MoE code; its only trace of this workload are the recorded
all-to-all count matrices under ``inputs/``.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import numpy as np
import torch

from .. import _native


def _p(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def grouped_gemm(A: torch.Tensor, B: torch.Tensor, group_start: torch.Tensor, group_rows: torch.Tensor,
                 out: Optional[torch.Tensor] = None, swiglu: bool = False, error: Optional[torch.Tensor] = None,
                 max_ctas: int = 0, ready: Optional[torch.Tensor] = None, ready_target: Optional[torch.Tensor] = None,
                 timeout_ms: float = 0.0, pair: Optional[bool] = None) -> torch.Tensor:
    """``out[rows of g] = epi(A[rows of g] @ B[g].T)`` with bf16 operands and fp32 accumulation.

    ``A`` [M, K], ``B`` [G, N, K], ``group_start`` / ``group_rows`` int32 CUDA tensors [G].  With ``swiglu``
    the rows of ``B[g]`` interleave gate and up projections and ``out`` is [M, N // 2].  With ``ready`` /
    ``ready_target`` (int64 CUDA tensors [G]) the rows of group g are loaded only once ``ready[g] >= ready_target[g]``:
    the kernel may be launched while the rows are still being delivered.  ``pair`` picks the kernel of an ungated
    call: True = CTA pairs (``cta_group::2``, 256 x 256 tiles; the default unless ``RBV_GEMM_PAIR=0``), False = one CTA
    per 128 x 256 tile."""
    lib = _native.cuda_lib()
    assert A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16 and A.is_contiguous() and B.is_contiguous()
    G, N, K = B.shape
    M = A.shape[0]
    assert A.shape[1] == K
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty(M, n_out, dtype=torch.bfloat16, device=A.device)
    if error is None:
        error = torch.zeros(1, dtype=torch.int32, device=A.device)
    st = torch.cuda.current_stream(A.device).cuda_stream
    prev = None
    if pair is not None and ready is None:
        prev = lib.rbv_grouped_gemm_pair_enabled()
        lib.rbv_grouped_gemm_set_pair(1 if pair else 0)
    try:
        rc = lib.rbv_grouped_gemm_bf16_gated(_p(A), M, _p(B), _p(out), _p(group_start), _p(group_rows), G, N, K,
                                             out.stride(0), 1 if swiglu else 0, _p(error), int(max_ctas),
                                             C.c_void_p(st), _p(ready), _p(ready_target), float(timeout_ms))
    finally:
        if prev is not None:
            lib.rbv_grouped_gemm_set_pair(prev)
    if rc:
        raise RuntimeError(f"grouped GEMM launch failed (CUDA error {rc})")
    return out


def quantize_rows_fp8(x: torch.Tensor):
    """bf16 [rows, K] -> (e4m3 bytes [rows, K], scales [K // 128, rows]); one scale per row and 128-wide K block."""
    lib = _native.cuda_lib()
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 128 == 0
    rows, K = x.shape
    q = torch.empty(rows, K, dtype=torch.uint8, device=x.device)
    sc = torch.empty(K // 128, rows, dtype=torch.float32, device=x.device)
    st = torch.cuda.current_stream(x.device).cuda_stream
    rc = lib.rbv_quantize_rows_fp8(_p(x), rows, K, x.stride(0), _p(q), _p(sc), C.c_void_p(st))
    if rc:
        raise RuntimeError(f"quantisation launch failed (CUDA error {rc})")
    return q, sc


def quantize_weight_blocks_fp8(w: torch.Tensor):
    """bf16 / fp32 [G, N, K] -> (e4m3 bytes [G, N, K], scales [G, N // 128, K // 128]); one scale per 128 x 128 block."""
    G, N, K = w.shape
    blk = w.float().view(G, N // 128, 128, K // 128, 128)
    amax = blk.abs().amax(dim=(2, 4))
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (blk / scale[:, :, None, :, None]).to(torch.float8_e4m3fn).view(G, N, K)
    return q.view(torch.uint8).contiguous(), scale.contiguous()


def dequantize_rows_fp8(q: torch.Tensor, scale_t: torch.Tensor) -> torch.Tensor:
    rows, K = q.shape
    return (q.view(torch.float8_e4m3fn).float().view(rows, K // 128, 128) * scale_t.t()[:, :, None]).view(rows, K)


def dequantize_weight_blocks_fp8(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    G, N, K = q.shape
    return (q.view(torch.float8_e4m3fn).float().view(G, N // 128, 128, K // 128, 128)
            * scale[:, :, None, :, None]).view(G, N, K)


def grouped_gemm_fp8(Aq: torch.Tensor, a_scale_t: torch.Tensor, Bq: torch.Tensor, b_scale: torch.Tensor,
                     group_start: torch.Tensor, group_rows: torch.Tensor, out: Optional[torch.Tensor] = None,
                     swiglu: bool = False, error: Optional[torch.Tensor] = None, max_ctas: int = 0,
                     coarse: bool = False, pair: Optional[bool] = None) -> torch.Tensor:
    """Block-scaled e4m3 grouped GEMM (see ``csrc/kernels/grouped_gemm_fp8_sm100.cu`` and its CTA-pair version
    ``grouped_gemm_fp8_pair_sm100.cu``, the default; ``pair=False`` or ``RBV_GEMM_PAIR=0`` for the former); bf16 output.

    ``coarse=True`` promises that the scales do not change along K (one per activation row, one per 128 weight
    rows): the kernel then accumulates a whole tile in TMEM and applies ``a_scale_t[0] * b_scale[..., 0]`` once."""
    lib = _native.cuda_lib()
    G, N, K = Bq.shape
    M = Aq.shape[0]
    assert Aq.dtype == torch.uint8 and Bq.dtype == torch.uint8 and Aq.is_contiguous() and Bq.is_contiguous()
    assert a_scale_t.shape == (K // 128, M) and b_scale.shape == (G, N // 128, K // 128)
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty(M, n_out, dtype=torch.bfloat16, device=Aq.device)
    if error is None:
        error = torch.zeros(1, dtype=torch.int32, device=Aq.device)
    st = torch.cuda.current_stream(Aq.device).cuda_stream
    prev = None
    if pair is not None:
        prev = lib.rbv_grouped_gemm_pair_enabled()
        lib.rbv_grouped_gemm_set_pair(1 if pair else 0)
    try:
        rc = lib.rbv_grouped_gemm_fp8(_p(Aq), _p(a_scale_t), M, _p(Bq), _p(b_scale), _p(out), _p(group_start),
                                      _p(group_rows), G, N, K, out.stride(0),
                                      (1 if swiglu else 0) | (2 if coarse else 0), _p(error), int(max_ctas),
                                      C.c_void_p(st))
    finally:
        if prev is not None:
            lib.rbv_grouped_gemm_set_pair(prev)
    if rc:
        raise RuntimeError(f"fp8 grouped GEMM launch failed (CUDA error {rc})")
    return out


# ---- MXFP8: e4m3 with one power-of-two scale per 32 elements along K on both operands, scaled by the tensor core ----
def quantize_rows_mxfp8(x: torch.Tensor):
    """bf16 [rows, K] -> (e4m3 bytes [rows, K], scale words [K // 128, ceil(rows / 128) * 128] int32 in atom order, see
    :func:`mx_to_atoms`): per row and 32 columns one UE8M0 scale 2^(byte - 127) >= amax / 448; the four bytes of a
    128-column block share a word, lowest byte first."""
    lib = _native.cuda_lib()
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 128 == 0
    rows, K = x.shape
    q = torch.empty(rows, K, dtype=torch.uint8, device=x.device)
    sf = torch.empty(K // 128, (rows + 127) // 128 * 128, dtype=torch.int32, device=x.device)
    st = torch.cuda.current_stream(x.device).cuda_stream
    rc = lib.rbv_quantize_rows_mxfp8(_p(x), rows, K, x.stride(0), _p(q), _p(sf), C.c_void_p(st))
    if rc:
        raise RuntimeError(f"MXFP8 quantisation launch failed (CUDA error {rc})")
    return q, sf


def _mx_atom_perm(n: int, device) -> torch.Tensor:
    """Position of row r (r < n, n a multiple of 128) in the atom order of the GEMM's scale words:
    (r // 128) * 128 + (r % 32) * 4 + (r % 128) // 32."""
    r = torch.arange(n, device=device)
    return (r // 128) * 128 + (r % 32) * 4 + (r % 128) // 32


def mx_to_atoms(plain: torch.Tensor) -> torch.Tensor:
    """Scale words with rows along the last dimension (padded to a multiple of 128 with the scale 1.0) -> atom order."""
    n = plain.shape[-1]
    npad = (n + 127) // 128 * 128
    out = torch.full(plain.shape[:-1] + (npad,), 0x7f7f7f7f, dtype=torch.int32, device=plain.device)
    out[..., _mx_atom_perm(npad, plain.device)[:n]] = plain.to(torch.int32)
    return out.contiguous()


def mx_from_atoms(atoms: torch.Tensor, n: int) -> torch.Tensor:
    """Inverse of :func:`mx_to_atoms`: the words of rows 0..n-1 in row order."""
    return atoms[..., _mx_atom_perm(atoms.shape[-1], atoms.device)[:n]].contiguous()


def _mx_exponents(amax: torch.Tensor) -> torch.Tensor:
    """ceil(log2(amax / 448)) as int32, 0 where amax == 0 (plain torch; used for weights and as the test oracle)."""
    t = amax.float() / 448.0
    m, e = torch.frexp(torch.where(t > 0, t, torch.ones_like(t)))       # t = m * 2^e, m in [0.5, 1)
    e = torch.where(m == 0.5, e - 1, e)
    return torch.where(t > 0, e, torch.zeros_like(e)).clamp(-127, 127).to(torch.int32)


def quantize_weight_mxfp8(w: torch.Tensor):
    """bf16 / fp32 [G, N, K] -> (e4m3 bytes [G, N, K], scale words [G, K // 128, N] int32 in atom order along N), one
    scale per weight row and 32 columns."""
    G, N, K = w.shape
    blk = w.float().view(G, N, K // 32, 32)
    e = _mx_exponents(blk.abs().amax(dim=3))                                # [G, N, K/32]
    q = (blk * torch.exp2(-e.float())[..., None]).to(torch.float8_e4m3fn).view(G, N, K)
    b = (e.to(torch.int64) + 127).view(G, N, K // 128, 4)
    words = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16) | (b[..., 3] << 24)      # [G, N, K/128]
    return q.view(torch.uint8).contiguous(), mx_to_atoms(words.permute(0, 2, 1).contiguous())


def _mx_scales(words: torch.Tensor) -> torch.Tensor:
    """int32 words [..., n] -> fp32 scales [..., n, 4] (byte j = 32-block j of the word's 128 columns)."""
    w = words.to(torch.int64) & 0xFFFFFFFF
    b = torch.stack([(w >> (8 * j)) & 0xFF for j in range(4)], dim=-1)
    return torch.exp2(b.float() - 127.0)


def dequantize_rows_mxfp8(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    rows, K = q.shape
    sc = _mx_scales(mx_from_atoms(sf, rows)).permute(1, 0, 2).reshape(rows, K // 32)             # [rows, K/32]
    return (q.view(torch.float8_e4m3fn).float().view(rows, K // 32, 32) * sc[:, :, None]).view(rows, K)


def dequantize_weight_mxfp8(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    G, N, K = q.shape
    sc = _mx_scales(mx_from_atoms(sf, N)).permute(0, 2, 1, 3).reshape(G, N, K // 32)          # [G, N, K/32]
    return (q.view(torch.float8_e4m3fn).float().view(G, N, K // 32, 32) * sc[..., None]).view(G, N, K)


def grouped_gemm_mxfp8(Aq: torch.Tensor, sfa: torch.Tensor, Bq: torch.Tensor, sfb: torch.Tensor,
                       group_start: torch.Tensor, group_rows: torch.Tensor, out: Optional[torch.Tensor] = None,
                       swiglu: bool = False, error: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
    """MXFP8 grouped GEMM on CTA pairs with hardware block scaling (``csrc/kernels/grouped_gemm_mxfp8_sm100.cu``);
    operands and scale words as the ``quantize_*_mxfp8`` functions make them; every group with rows must start at a
    multiple of 128 rows; bf16 output."""
    lib = _native.cuda_lib()
    G, N, K = Bq.shape
    M = Aq.shape[0]
    assert Aq.dtype == torch.uint8 and Bq.dtype == torch.uint8 and Aq.is_contiguous() and Bq.is_contiguous()
    assert sfa.shape == (K // 128, (M + 127) // 128 * 128) and sfb.shape == (G, K // 128, N)
    assert sfa.is_contiguous() and sfb.is_contiguous()
    assert sfa.dtype == torch.int32 and sfb.dtype == torch.int32
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty(M, n_out, dtype=torch.bfloat16, device=Aq.device)
    if error is None:
        error = torch.zeros(1, dtype=torch.int32, device=Aq.device)
    st = torch.cuda.current_stream(Aq.device).cuda_stream
    rc = lib.rbv_grouped_gemm_mxfp8(_p(Aq), _p(sfa), M, _p(Bq), _p(sfb), _p(out), _p(group_start), _p(group_rows),
                                    G, N, K, out.stride(0), 1 if swiglu else 0, _p(error), int(max_ctas),
                                    C.c_void_p(st))
    if rc:
        raise RuntimeError(f"MXFP8 grouped GEMM launch failed (CUDA error {rc})")
    return out


def grouped_gemm_mxfp8_swiglu_q(Aq: torch.Tensor, sfa: torch.Tensor, Bq: torch.Tensor, sfb: torch.Tensor,
                                group_start: torch.Tensor, group_rows: torch.Tensor,
                                out_q: Optional[torch.Tensor] = None, out_sf: Optional[torch.Tensor] = None,
                                error: Optional[torch.Tensor] = None, max_ctas: int = 0):
    """The MXFP8 up/gate GEMM with SwiGLU and the quantiser of the next GEMM fused into its epilogue: returns
    ``(hq, hs)``, e4m3 bytes [M, N // 2] and their scale words [N // 256, ceil(M / 128) * 128] in atom order, i.e. what
    :func:`quantize_rows_mxfp8` would make of the bf16 result, without that result ever going to memory."""
    lib = _native.cuda_lib()
    G, N, K = Bq.shape
    M = Aq.shape[0]
    assert N % 256 == 0 and Aq.dtype == torch.uint8 and Bq.dtype == torch.uint8 and Aq.is_contiguous() and Bq.is_contiguous()
    mp = (M + 127) // 128 * 128
    assert sfa.shape == (K // 128, mp) and sfb.shape == (G, K // 128, N) and sfa.is_contiguous() and sfb.is_contiguous()
    if out_q is None:
        out_q = torch.empty(M, N // 2, dtype=torch.uint8, device=Aq.device)
    if out_sf is None:
        out_sf = torch.empty(N // 256, mp, dtype=torch.int32, device=Aq.device)
    assert out_q.shape == (M, N // 2) and out_q.stride(1) == 1 and out_sf.shape == (N // 256, mp) and out_sf.is_contiguous()
    if error is None:
        error = torch.zeros(1, dtype=torch.int32, device=Aq.device)
    st = torch.cuda.current_stream(Aq.device).cuda_stream
    rc = lib.rbv_grouped_gemm_mxfp8_swiglu_q(_p(Aq), _p(sfa), M, _p(Bq), _p(sfb), _p(out_q), _p(out_sf),
                                             _p(group_start), _p(group_rows), G, N, K, out_q.stride(0), _p(error),
                                             int(max_ctas), C.c_void_p(st))
    if rc:
        raise RuntimeError(f"MXFP8 grouped GEMM launch failed (CUDA error {rc})")
    return out_q, out_sf


def pack_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Interleaves [G, I, H] gate and up weights into the [G, 2I, H] layout the SwiGLU epilogue expects."""
    G, I, H = gate.shape
    return torch.stack([gate, up], dim=2).reshape(G, 2 * I, H).contiguous()


class MoEExpertParallel:
    """One MoE FFN layer sharded by experts over the ranks of a communicator (one rank per GPU)."""

    def __init__(self, comm, num_experts: int, hidden: int, inter: int, tokens: int, capacity_factor: float = 2.0,
                 seed: int = 0, init_std: float = 0.02, fp8: bool = False, overlap: Optional[bool] = None,
                 push_combine: Optional[bool] = None):
        if comm.L != 1:
            raise ValueError("the MoE path needs one rank per process")
        if num_experts % comm.P:
            raise ValueError("experts must divide evenly over the ranks")
        self.comm, self.lib = comm, _native.cuda_lib()
        self.P, self.me = comm.P, comm.proc
        self.E, self.El, self.H, self.I, self.T = num_experts, num_experts // comm.P, hidden, inter, tokens
        dev = f"cuda:{comm.device}"
        self.dev = dev
        g = torch.Generator(device=dev)
        g.manual_seed(seed * 1000 + self.me)
        bf = torch.bfloat16
        self.w13 = (torch.randn(self.El, 2 * inter, hidden, device=dev, generator=g) * init_std).to(bf)
        self.w2 = (torch.randn(self.El, hidden, inter, device=dev, generator=g) * init_std).to(bf)
        self.mx = fp8 == "mx"          # MXFP8: power-of-two scales per 32 elements, applied by the tensor core
        self.fp8 = bool(fp8)
        if self.mx:
            self.w13_q, self.w13_s = quantize_weight_mxfp8(self.w13)
            self.w2_q, self.w2_s = quantize_weight_mxfp8(self.w2)
        elif self.fp8:   # expert weights as e4m3 with one scale per 128 x 128 block
            self.w13_q, self.w13_s = quantize_weight_blocks_fp8(self.w13)
            self.w2_q, self.w2_s = quantize_weight_blocks_fp8(self.w2)
        self.cap = int(np.ceil(capacity_factor * 2 * tokens / 128.0)) * 128 + (128 * self.El if self.mx else 0)
        i32 = torch.int32
        # MXFP8: rows are quantised by the dispatch itself and cross NVLink as e4m3 + scale words (half the bytes, no
        # quantiser pass on the owner); RBV_MOE_QDISPATCH=0 dispatches bf16 rows and quantises them afterwards
        self.qdispatch = self.mx and hidden % 128 == 0 and os.environ.get("RBV_MOE_QDISPATCH", "1") != "0"
        if self.qdispatch:
            self.xrecv = None
            self.xq = comm.symm_empty((self.cap, hidden), torch.uint8)
            self.sfrow = comm.symm_empty((self.cap, hidden // 128), i32)
            self.xs = torch.full((hidden // 128, self.cap), 0x7f7f7f7f, dtype=i32, device=dev)   # atom order
        else:
            self.xrecv = comm.symm_empty((self.cap, hidden), bf)
        self.h = torch.empty(self.cap, inter, dtype=bf, device=dev)
        self.hist = torch.zeros(self.E, dtype=i32, device=dev)
        self.hist_all = comm.symm_zeros((self.P, self.E), i32)
        self.topk_idx = torch.empty(tokens, 2, dtype=i32, device=dev)
        self.topk_w = torch.empty(tokens, 2, dtype=torch.float32, device=dev)
        self.slot = torch.empty(tokens, 2, dtype=i32, device=dev)
        self.dst_base = torch.empty(self.E, dtype=i32, device=dev)
        self.cursor = torch.zeros(self.E, dtype=i32, device=dev)
        self.group_start = torch.zeros(self.El, dtype=i32, device=dev)
        self.group_rows = torch.zeros(self.El, dtype=i32, device=dev)
        self.totals = torch.zeros(2, dtype=i32, device=dev)
        self.error = torch.zeros(4, dtype=i32, device=dev)
        # Streamed dispatch (bf16 path): rows travel expert by expert, every landed row bumps its expert's counter on
        # the owner, and the first grouped GEMM, launched on a second stream next to the dispatch, starts an expert as
        # soon as its rows are complete.  Opt-in (``overlap=True`` or RBV_MOE_OVERLAP=1): measured on B200 with the
        # benchmark configuration it takes 0.09 ms off the 4.50 ms layer on 2 GPUs but adds 0.10 ms to the 4.62 ms
        # layer on 4 GPUs (the dispatch, now sharing every SM with the GEMM and fencing once per row, slows the GEMM
        # by more than the hidden head of the dispatch is worth once three quarters of the rows cross NVLink).
        if overlap is None:
            overlap = os.environ.get("RBV_MOE_OVERLAP", "0") == "1"
        self.overlap = bool(overlap) and not self.fp8
        self.ready = comm.symm_zeros(max(self.El, 2), torch.int64)          # bumped by every GPU, never reset
        self.ready_target = torch.zeros(max(self.El, 2), dtype=torch.int64, device=dev)
        self.loc_off = torch.zeros(self.E, dtype=i32, device=dev)
        self.order = torch.zeros(2 * tokens, dtype=i32, device=dev)
        self._side = torch.cuda.Stream(device=dev)
        self._ev_layout, self._ev_gemm1 = torch.cuda.Event(), torch.cuda.Event()
        # Down GEMM fused with the return all-to-all (bf16 and MXFP8 paths): the dispatch leaves beside every row where
        # its result has to go, the down GEMM's epilogue stores each result row straight into the [T, 2, H] buffer of
        # the token's GPU (over NVLink while the GEMM is still computing other tiles), and the combine only waits for
        # all GEMMs and adds two local rows per token.  ``push_combine=False`` / RBV_MOE_PUSH=0 keeps the combine that
        # pulls the rows after the GEMM.
        if push_combine is None:
            push_combine = os.environ.get("RBV_MOE_PUSH", "1") != "0"
        self.push = bool(push_combine) and (self.mx or not self.fp8) and not self.overlap
        self.ret = comm.symm_zeros(self.cap, i32)
        self.y2 = comm.symm_empty((2 * tokens, hidden), bf) if self.push else None      # results, by (token, k)
        self.y = None if self.push else comm.symm_empty((self.cap, hidden), bf)         # results, expert-sorted
        heap0 = self.lib.rbv_ctx_heap(comm._ctx, comm.proc)
        self.xrecv_off = (self.xq if self.qdispatch else self.xrecv).data_ptr() - heap0
        self.sfrow_off = (self.sfrow.data_ptr() - heap0) if self.qdispatch else 0
        self.y_off = 0 if self.push else self.y.data_ptr() - heap0
        self.ready_off = self.ready.data_ptr() - heap0
        self.ret_off = self.ret.data_ptr() - heap0
        self.y2_off = (self.y2.data_ptr() - heap0) if self.push else 0
        self._heaps = (C.c_void_p * self.P)(*[self.lib.rbv_ctx_heap(comm._ctx, q) for q in range(self.P)])
        comm.require_same_offsets(self.xrecv_off, self.y_off, self.ready_off, self.ret_off, self.y2_off, self.sfrow_off)
        torch.cuda.synchronize(dev)
        comm.host_barrier()          # every rank's counters are zero before anybody's first dispatch
        # the histogram all-gather: every rank sends the same E counters to every rank
        cnt = np.full((1, self.P), self.E, dtype=np.int32)
        self._gather = comm.prepare(self.hist, self.hist_all.view(-1), cnt, np.zeros((1, self.P), dtype=np.int64), cnt,
                                    (np.arange(self.P, dtype=np.int64) * self.E).reshape(1, self.P),
                                    algo="spreadout", type_size=4, grid=1)

    def _check(self, rc, what):
        if rc:
            raise RuntimeError(f"{what} failed (CUDA error {rc})")

    def forward(self, x: torch.Tensor, logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, H = x.shape
        assert T == self.T and H == self.H and x.dtype == torch.bfloat16 and x.is_contiguous()
        assert logits.shape == (T, self.E) and logits.dtype == torch.float32 and logits.is_contiguous()
        lib, ctx = self.lib, self.comm._ctx
        st = C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        if out is None:
            out = torch.empty_like(x)
        self._check(lib.rbv_moe_route(_p(logits), T, self.E, _p(self.topk_idx), _p(self.topk_w), _p(self.hist), st),
                    "router")
        self._gather.launch()
        if self.overlap:
            return self._forward_streamed(x, out, st)
        # the MXFP8 GEMM wants every expert's rows to start at a multiple of 128 rows (its scale atoms)
        self._check(lib.rbv_moe_layout_aligned(_p(self.hist_all), self.P, self.E, self.me, _p(self.dst_base),
                                               _p(self.group_start), _p(self.group_rows), _p(self.cursor),
                                               _p(self.totals), 128 if self.mx else 1, st), "layout")
        if self.qdispatch:
            self._check(lib.rbv_moe_dispatch_mx(ctx, _p(x), T, H, _p(self.topk_idx), _p(self.dst_base),
                                                _p(self.cursor), _p(self.slot), self.xrecv_off, self.sfrow_off,
                                                self.ret_off if self.push else 0, self.cap, self.E,
                                                _p(self.error[0:1]), st), "dispatch")
            self._check(lib.rbv_moe_scale_atoms(_p(self.sfrow), _p(self.xs), self.cap, H // 128, st), "scale layout")
        else:
            self._check(lib.rbv_moe_dispatch_ret(ctx, _p(x), T, H, _p(self.topk_idx), _p(self.dst_base),
                                                 _p(self.cursor), _p(self.slot), self.xrecv_off,
                                                 self.ret_off if self.push else 0, self.cap, self.E,
                                                 _p(self.error[0:1]), st), "dispatch")
        if self.mx:
            # activations are quantised once (by the dispatch, or here); the first GEMM's epilogue (SwiGLU) hands the
            # second GEMM its operand already quantised, so the bf16 intermediate never exists
            xq, xs = (self.xq, self.xs) if self.qdispatch else quantize_rows_mxfp8(self.xrecv)
            if self.I % 128 == 0:
                if getattr(self, "_hq", None) is None:
                    self._hq = torch.empty(self.cap, self.I, dtype=torch.uint8, device=self.dev)
                    self._hs = torch.empty(self.I // 128, self.cap, dtype=torch.int32, device=self.dev)
                hq, hs = grouped_gemm_mxfp8_swiglu_q(xq, xs, self.w13_q, self.w13_s, self.group_start,
                                                     self.group_rows, out_q=self._hq, out_sf=self._hs,
                                                     error=self.error[1:2])
            else:
                grouped_gemm_mxfp8(xq, xs, self.w13_q, self.w13_s, self.group_start, self.group_rows, out=self.h,
                                   swiglu=True, error=self.error[1:2])
                hq, hs = quantize_rows_mxfp8(self.h)
            if self.push:
                self._check(lib.rbv_grouped_gemm_mxfp8_push(
                    _p(hq), _p(hs), self.cap, _p(self.w2_q), _p(self.w2_s), _p(self.group_start), _p(self.group_rows),
                    self.El, H, self.I, _p(self.ret), self._heaps, self.P, self.y2_off, _p(self.error[2:3]), 0, st),
                    "down GEMM")
            else:
                grouped_gemm_mxfp8(hq, hs, self.w2_q, self.w2_s, self.group_start, self.group_rows, out=self.y,
                                   error=self.error[2:3])
        elif self.fp8:
            # activations are quantised row-wise (1 x 128 blocks) right before each GEMM
            xq, xs = quantize_rows_fp8(self.xrecv)
            grouped_gemm_fp8(xq, xs, self.w13_q, self.w13_s, self.group_start, self.group_rows, out=self.h, swiglu=True,
                             error=self.error[1:2])
            hq, hs = quantize_rows_fp8(self.h)
            grouped_gemm_fp8(hq, hs, self.w2_q, self.w2_s, self.group_start, self.group_rows, out=self.y,
                             error=self.error[2:3])
        else:
            grouped_gemm(self.xrecv, self.w13, self.group_start, self.group_rows, out=self.h, swiglu=True,
                         error=self.error[1:2])
            if self.push:
                self._check(lib.rbv_grouped_gemm_bf16_push(
                    _p(self.h), self.cap, _p(self.w2), _p(self.group_start), _p(self.group_rows), self.El, H, self.I,
                    _p(self.ret), self._heaps, self.P, self.y2_off, _p(self.error[2:3]), 0, st), "down GEMM")
            else:
                grouped_gemm(self.h, self.w2, self.group_start, self.group_rows, out=self.y, swiglu=False,
                             error=self.error[2:3])
        if self.push:
            self._check(lib.rbv_moe_combine_pushed(ctx, _p(out), T, H, _p(self.topk_w), _p(self.y2),
                                                   _p(self.error[3:4]), st), "combine")
        else:
            self._check(lib.rbv_moe_combine(ctx, _p(out), T, H, _p(self.topk_idx), _p(self.topk_w), _p(self.slot),
                                            self.y_off, self.E, _p(self.error[3:4]), st), "combine")
        return out

    def _forward_streamed(self, x, out, st):
        lib, ctx, T, H = self.lib, self.comm._ctx, self.T, self.H
        main = torch.cuda.current_stream(self.dev)
        self._check(lib.rbv_moe_layout_streamed(_p(self.hist_all), self.P, self.E, self.me, _p(self.dst_base),
                                                _p(self.group_start), _p(self.group_rows), _p(self.cursor),
                                                _p(self.totals), _p(self.loc_off), _p(self.ready_target),
                                                _p(self.topk_idx), T, _p(self.order), st), "layout")
        self._ev_layout.record(main)
        # The dispatch goes first, so that its CTAs are in place (or done) when the GEMM's arrive: a GEMM that filled
        # the GPU before the dispatch got in would wait for rows that nobody is there to send.
        self._check(lib.rbv_moe_dispatch_streamed(ctx, _p(x), T, H, _p(self.topk_idx), _p(self.dst_base),
                                                  _p(self.loc_off), _p(self.order), _p(self.slot), self.xrecv_off,
                                                  self.ready_off, self.cap, self.E, _p(self.error[0:1]), st), "dispatch")
        # the first GEMM runs next to it, on its own stream, and takes each expert when its counter is complete
        with torch.cuda.stream(self._side):
            self._side.wait_event(self._ev_layout)
            grouped_gemm(self.xrecv, self.w13, self.group_start, self.group_rows, out=self.h, swiglu=True,
                         error=self.error[1:2], ready=self.ready, ready_target=self.ready_target)
            self._ev_gemm1.record(self._side)
        main.wait_event(self._ev_gemm1)
        grouped_gemm(self.h, self.w2, self.group_start, self.group_rows, out=self.y, swiglu=False, error=self.error[2:3])
        self._check(lib.rbv_moe_combine(ctx, _p(out), T, H, _p(self.topk_idx), _p(self.topk_w), _p(self.slot),
                                        self.y_off, self.E, _p(self.error[3:4]), st), "combine")
        return out

    def check(self):
        """Synchronises and raises if any kernel of the layer recorded an error."""
        e = self.error.cpu().tolist()
        if any(e):
            raise RuntimeError(f"MoE kernels reported errors (dispatch, gemm1, gemm2, combine) = {e}")
        self.comm.check()

    def flops(self, routed_rows: int) -> float:
        return routed_rows * (2.0 * self.H * 2 * self.I + 2.0 * self.I * self.H)


def reference_forward(x, logits, w13_all, w2_all):
    """fp32 PyTorch reference of the whole layer on one device.  ``w13_all`` [E, 2I, H] interleaved,
    ``w2_all`` [E, H, I]; intermediate activations are rounded to bf16 where the kernels round them."""
    xf = x.float()
    p = torch.softmax(logits.float(), dim=-1)
    top_p, top_i = torch.topk(p, 2, dim=-1)
    w = top_p / top_p.sum(-1, keepdim=True)
    out = torch.zeros_like(xf)
    for k in range(2):
        for e in torch.unique(top_i[:, k]).tolist():
            rows = (top_i[:, k] == e).nonzero().squeeze(1)
            gu = xf[rows] @ w13_all[e].float().t()
            hmid = (torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]).to(torch.bfloat16).float()
            yv = (hmid @ w2_all[e].float().t()).to(torch.bfloat16).float()
            out[rows] += w[rows, k:k + 1] * yv
    return out, top_i, w
