/* Expert-parallel MoE path: router, dispatch (permute fused with the all-to-all), grouped expert GEMM on
 * the sm_100a tensor cores, combine (return all-to-all fused with the gate-weighted sum).  Nothing of this
 * exists in the reference, which ships only the alltoallv primitive and recorded MoE-like traffic traces
 * (inputs/, examples/MLinputs_example.cpp); it is built on the same symmetric heap and peer mappings as the
 * alltoallv kernels.
 */
#ifndef RBV_MOE_H_
#define RBV_MOE_H_

#include "rbv/rbruckv.h"

#ifdef __cplusplus
namespace rbv { constexpr int kMoeMaxGroups = 64; constexpr int kMoeMaxExperts = 256; }
extern "C" {
#endif

/* C[rows of group g] = epi(A[rows of group g] * B_g^T), bf16 in / bf16 out, fp32 accumulation.
 *   A: [a_rows, K] row-major.  B: [G, N, K] (each expert's weight with K contiguous).  C: rows of ldc elements.
 *   group_start / group_rows: device int32[G].  N % 256 == 0, K % 64 == 0.
 *   epilogue 0: C is [*, N];  epilogue 1 (SwiGLU): B rows interleave gate and up (2j = gate_j, 2j+1 = up_j) and
 *   C is [*, N/2] with C[:, j] = silu(gate_j) * up_j.
 *   error_flag: device int, set non-zero if a bounded wait inside the kernel ran out.
 * Returns 0 or a CUDA error code. */
int rbv_grouped_gemm_bf16(const void* A, long long a_rows, const void* B, void* C, const int* group_start,
                          const int* group_rows, int G, int N, int K, int ldc, int epilogue, int* error_flag,
                          int max_ctas, void* cuda_stream);

/* The kernel behind rbv_grouped_gemm_bf16 when CTA pairs are enabled (the default; RBV_GEMM_PAIR=0 or
 * rbv_grouped_gemm_set_pair(0) selects the one-CTA kernel): clusters of two CTAs share 256 x 256 tiles with
 * tcgen05 cta_group::2 MMAs, each CTA fetching half of the operands.  Same arguments and limits. */
int rbv_grouped_gemm_bf16_pair(const void* A, long long a_rows, const void* B, void* C, const int* group_start,
                               const int* group_rows, int G, int N, int K, int ldc, int epilogue, int* error_flag,
                               int max_ctas, void* cuda_stream);
void rbv_grouped_gemm_set_pair(int on);      /* process-wide switch, not synchronised: set it before launching from */
int rbv_grouped_gemm_pair_enabled(void);      /* several host threads, not while they launch                          */

/* The same with a gated start per group: the loader touches the rows of group g only once ready[g] >= ready_target[g]
 * (device uint64 arrays; the counters are bumped by whoever delivers the rows, e.g. rbv_moe_dispatch_streamed running
 * at the same time on this and on other GPUs).  The wait is bounded by timeout_ms (0: 2 s). */
int rbv_grouped_gemm_bf16_gated(const void* A, long long a_rows, const void* B, void* C, const int* group_start,
                                const int* group_rows, int G, int N, int K, int ldc, int epilogue, int* error_flag,
                                int max_ctas, void* cuda_stream, const unsigned long long* ready,
                                const unsigned long long* ready_target, double timeout_ms);

/* Block-scaled fp8 (e4m3) variant.  A: [a_rows, K] bytes with one fp32 scale per row and 128-wide K block, stored
 * transposed as a_scale_t [K / 128][a_rows]; B: [G, N, K] bytes with one scale per 128 x 128 block, b_scale
 * [G][N / 128][K / 128].  N % 128 == 0, K % 128 == 0.  Output bf16, epilogues as above. */
int rbv_grouped_gemm_fp8(const void* A, const float* a_scale_t, long long a_rows, const void* B, const float* b_scale,
                         void* C, const int* group_start, const int* group_rows, int G, int N, int K, int ldc,
                         int epilogue, int* error_flag, int max_ctas, void* cuda_stream);
/* The kernel behind rbv_grouped_gemm_fp8 when CTA pairs are enabled: 256 x 128 tiles on clusters of two CTAs. */
int rbv_grouped_gemm_fp8_pair(const void* A, const float* a_scale_t, long long a_rows, const void* B,
                              const float* b_scale, void* C, const int* group_start, const int* group_rows, int G,
                              int N, int K, int ldc, int epilogue, int* error_flag, int max_ctas, void* cuda_stream);
/* MXFP8 variant: e4m3 operands with one UE8M0 (power-of-two) scale per 32 elements along K on both operands, applied
 * by the tensor core (tcgen05.mma.kind::mxf8f6f4.block_scale) on CTA pairs.  Scales are packed four to a uint32 (the
 * four 32-blocks of one 128-wide K block, lowest byte first); the words of 128 consecutive rows form one 512-byte atom
 * in which row r sits at word (r % 32) * 4 + (r % 128) / 32:  sfa [K / 128][ceil(a_rows / 128)][128],
 * sfb [G][K / 128][N / 128][128].  Every group with rows must start at a multiple of 128 rows (error flag 5
 * otherwise).  N % 128 == 0, K % 128 == 0.  Output bf16; epilogue 0 plain, 1 SwiGLU. */
int rbv_grouped_gemm_mxfp8(const void* A, const void* sfa, long long a_rows, const void* B, const void* sfb, void* C,
                           const int* group_start, const int* group_rows, int G, int N, int K, int ldc, int epilogue,
                           int* error_flag, int max_ctas, void* cuda_stream);
/* The up/gate GEMM with the SwiGLU epilogue AND the quantiser of the next GEMM fused: Cq is e4m3 [*, N / 2] (row
 * stride ldc_bytes) and sf_out its scale words, [N / 256][ceil(a_rows / 128)][128] in the atom order above, i.e. what
 * rbv_quantize_rows_mxfp8 would make of the bf16 result.  N % 256 == 0. */
int rbv_grouped_gemm_mxfp8_swiglu_q(const void* A, const void* sfa, long long a_rows, const void* B, const void* sfb,
                                    void* Cq, void* sf_out, const int* group_start, const int* group_rows, int G,
                                    int N, int K, int ldc_bytes, int* error_flag, int max_ctas, void* cuda_stream);
/* bf16 [rows, K] (row stride ldx elements) -> e4m3 [rows, K] + sf [K / 128][ceil(rows / 128)][128] as above. */
int rbv_quantize_rows_mxfp8(const void* x_bf16, long long rows, int K, int ldx, void* out_fp8, void* sf,
                            void* cuda_stream);
/* bf16 [rows, K] (row stride ldx elements) -> e4m3 [rows, K] + scale_t [K / 128][rows], scale = amax / 448. */
int rbv_quantize_rows_fp8(const void* x_bf16, long long rows, int K, int ldx, void* out_fp8, float* scale_t,
                          void* cuda_stream);

/* Router: softmax over E logits per token, top-2, weights renormalised to sum to one.
 *   logits [T, E] fp32;  topk_idx [T, 2] int32;  topk_w [T, 2] fp32;  hist [E] int32 (zeroed by the call). */
int rbv_moe_route(const float* logits, int T, int E, int* topk_idx, float* topk_w, int* hist, void* cuda_stream);

/* From the all-gathered histograms hist_all [P, E] computes, for rank `me`:
 *   dst_base [E]   first row of this rank's rows for expert e inside the owner's receive buffer,
 *   group_start / group_rows [E / P]  row ranges of the local experts, cursor [E] zeroed,
 *   totals [2]     rows received by this rank, rows sent by this rank. */
int rbv_moe_layout(const int* hist_all, int P, int E, int me, int* dst_base, int* group_start, int* group_rows,
                   int* cursor, int* totals, void* cuda_stream);
/* The same with every expert's rows starting at a multiple of `align` rows of the owner's buffer (the MXFP8 GEMM wants
 * 128); the buffer then needs up to (E / P - 1) * (align - 1) rows more than it receives. */
int rbv_moe_layout_aligned(const int* hist_all, int P, int E, int me, int* dst_base, int* group_start,
                           int* group_rows, int* cursor, int* totals, int align, void* cuda_stream);

/* Dispatch: every routed (token, k) row of x [T, H] bf16 is stored straight into its expert-sorted row of the
 * owner GPU's receive buffer (`xrecv_off` = byte offset of that buffer inside every process's heap).  slot [T, 2]
 * receives the destination row.  The kernel returns when the rows of ALL ranks have landed here (bounded wait).
 * One logical rank per process. */
int rbv_moe_dispatch(rbv_ctx_t ctx, const void* x, int T, int H, const int* topk_idx, const int* dst_base,
                     int* cursor, int* slot, unsigned long long xrecv_off, long long recv_capacity_rows,
                     int E, int* error_flag, void* cuda_stream);

/* Streamed dispatch (overlaps with the first expert GEMM).  rbv_moe_layout_streamed is rbv_moe_layout plus: loc_off [E]
 * (where this rank's rows for expert e start in an expert-major ordering of its routed rows), order [2 T] (that
 * ordering), and ready_target [E / P] += rows each local expert receives in this call (a running total kept across
 * calls; zero it once).  rbv_moe_dispatch_streamed walks `order`, stores every row into its place on the owner and
 * adds one to the owner's counter ready[e_local] (uint64 [E / P] at byte offset ready_off of every heap, zeroed once,
 * never reset).  It does not wait for anybody: the consumer is rbv_grouped_gemm_bf16_gated(ready, ready_target). */
int rbv_moe_layout_streamed(const int* hist_all, int P, int E, int me, int* dst_base, int* group_start,
                            int* group_rows, int* cursor, int* totals, int* loc_off, unsigned long long* ready_target,
                            const int* topk_idx, int T, int* order, void* cuda_stream);
int rbv_moe_dispatch_streamed(rbv_ctx_t ctx, const void* x, int T, int H, const int* topk_idx, const int* dst_base,
                              const int* loc_off, const int* order, int* slot, unsigned long long xrecv_off,
                              unsigned long long ready_off, long long recv_capacity_rows, int E, int* error_flag,
                              void* cuda_stream);

/* Combine: out[t] = sum_k w[t,k] * Y_owner(k)[slot[t,k]], rows pulled from the owners' `y_off` buffers over
 * NVLink after a bounded cross-GPU barrier ("all expert outputs are complete"). */
int rbv_moe_combine(rbv_ctx_t ctx, void* out, int T, int H, const int* topk_idx, const float* topk_w,
                    const int* slot, unsigned long long y_off, int E, int* error_flag, void* cuda_stream);

/* Dispatch that also leaves, beside every row, where its result has to go: word `pos` of the table at heap offset
 * ret_off on the row's owner becomes (sending process << 24) | (token * 2 + k).  2 T < 2^24. */
int rbv_moe_dispatch_ret(rbv_ctx_t ctx, const void* x, int T, int H, const int* topk_idx, const int* dst_base,
                         int* cursor, int* slot, unsigned long long xrecv_off, unsigned long long ret_off,
                         long long recv_capacity_rows, int E, int* error_flag, void* cuda_stream);

/* Dispatch for the MXFP8 path: rows are quantised where they are read (as rbv_quantize_rows_mxfp8 would) and travel
 * as H bytes + H / 128 scale words: the owner's [capacity, H] e4m3 buffer at heap offset xq_off and its row-major
 * scale words [capacity, H / 128] at sfrow_off; rbv_moe_scale_atoms then makes the GEMM's atom order of them
 * ([H / 128][ceil(rows / 128)][128]).  ret_off as in rbv_moe_dispatch_ret (0: none).  H % 128 == 0. */
int rbv_moe_dispatch_mx(rbv_ctx_t ctx, const void* x, int T, int H, const int* topk_idx, const int* dst_base,
                        int* cursor, int* slot, unsigned long long xq_off, unsigned long long sfrow_off,
                        unsigned long long ret_off, long long recv_capacity_rows, int E, int* error_flag,
                        void* cuda_stream);
int rbv_moe_scale_atoms(const void* sfrow, void* sfa, int rows, int nkb, void* cuda_stream);

/* Down GEMM fused with the return all-to-all: the epilogue stores row `pos` of the result straight into row
 * (token * 2 + k) of the [T, 2, N] bf16 buffer at heap offset y2_off of the process the row came from (`ret`, the
 * table rbv_moe_dispatch_ret filled; `heaps[nheaps]` this process's mappings of every process's heap), so the
 * transfer overlaps the GEMM tile by tile.  Epilogue: plain bf16.  Pair kernel (cta_group::2) in both precisions. */
int rbv_grouped_gemm_bf16_push(const void* A, long long a_rows, const void* B, const int* group_start,
                               const int* group_rows, int G, int N, int K, const unsigned* ret,
                               const void* const* heaps, int nheaps, unsigned long long y2_off, int* error_flag,
                               int max_ctas, void* cuda_stream);
int rbv_grouped_gemm_mxfp8_push(const void* A, const void* sfa, long long a_rows, const void* B, const void* sfb,
                                const int* group_start, const int* group_rows, int G, int N, int K,
                                const unsigned* ret, const void* const* heaps, int nheaps, unsigned long long y2_off,
                                int* error_flag, int max_ctas, void* cuda_stream);

/* Combine after such a GEMM: cross-GPU barrier (every process's GEMM has finished), then
 * out[t] = w[t][0] * y2[t][0] + w[t][1] * y2[t][1] from local memory. */
int rbv_moe_combine_pushed(rbv_ctx_t ctx, void* out, int T, int H, const float* topk_w, const void* y2,
                           int* error_flag, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif
