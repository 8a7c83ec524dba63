// MXFP8 grouped GEMM for the expert FFN: e4m3 operands with one power-of-two (UE8M0) scale per 32 elements along K on
// BOTH operands, applied by the tensor core itself (tcgen05.mma.kind::mxf8f6f4.block_scale), on CTA pairs
// (cta_group::2).  This is the fp8 recipe the hardware scales natively: the accumulator of a tile stays in TMEM for the
// whole K loop and is read out once, where the software-scaled kernel (grouped_gemm_fp8_sm100.cu, fp32 scales per
// 1 x 128 / 128 x 128 block) has to pull it out of TMEM after every K block.  No counterpart in the reference.
//
//   C[rows of g] = epi( sum_k  A[row, k] 2^(sa[row, k / 32] - 127) * B_g[n, k] 2^(sb[g, n, k / 32] - 127) )
//
// Scale storage: one uint32 holds the four scales of one 128-wide K block (lowest byte first); the words of 128
// consecutive rows (of A, or of one expert's weight) sit together as one 512-byte "atom" in the order tcgen05.cp wants,
// word (r % 32) * 4 + (r % 128) / 32 for row r:
//   A: sfa[K / 128][ceil(a_rows / 128)][128]        B: sfb[G][K / 128][N / 128][128]
// so that a tile's scales are one 512-byte TMA box per operand and K block.  For the atoms of A to coincide with tiles,
// every group must start at a multiple of 128 rows (checked in the kernel; the MoE layout pads experts accordingly).
// Two CTAs on neighbouring SMs share a 256 x 128 tile.  Per K block (128 bytes of K) each CTA fetches by TMA (no
// multicast; bytes counted on a barrier of the rank-0 CTA) its own 128 rows of A, its own 64 of the 128 weight rows,
// the scale atom of its A rows and the scale atom of the tile's 128 weight rows.  The rank-0 CTA copies the scales of
// both CTAs from shared memory into TMEM (tcgen05.cp.32x128b.warpx4, 4 + 4 columns per stage) and issues four MMAs
// (M 256, N 128, K 32), each naming its scale byte in the instruction descriptor.  TMEM: two 128-column accumulators
// (the epilogue of tile i overlaps the MMAs of tile i + 1) and 8 columns of scales per pipeline stage.
// Epilogues: bf16; SwiGLU to bf16; SwiGLU followed by the MXFP8 quantiser of the next GEMM's operand (each thread owns a
// row of the tile, so the scale of a 32-block needs no other thread); and, for the down GEMM of the MoE layer, bf16 rows
// stored straight into the buffers of the GPUs the tokens came from (the return all-to-all, overlapped with the MMAs
// of the other tiles).  All waits are bounded; on expiry both CTAs are told, record an error, release their TMEM and
// return.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels/mx_quant.cuh"
#include "kernels/sm100_ptx.cuh"
#include "rbv/moe.h"

namespace rbv {

using namespace sm100;

namespace {

constexpr int XM = 256;                 // tile rows per pair
constexpr int XHM = 128;                // rows per CTA
constexpr int XN = 128;                 // tile columns
constexpr int XHB = 64;                 // weight rows each CTA fetches
constexpr int XK = 128;                 // bytes of K per pipeline stage (one 128-byte swizzle row, four scale blocks)
constexpr int XSTAGES = 8;
constexpr int XA_TILE = XHM * XK;       // 16 KB
constexpr int XB_TILE = XHB * XK;       // 8 KB
constexpr int XSF_TILE = 512;           // 128 scale words
constexpr int XSTAGE = XA_TILE + XB_TILE + 2 * XSF_TILE;   // 25 KB
constexpr int XTHREADS = 192;           // TMA warp, MMA warp, 4 epilogue warps
constexpr int XACC_COLS = 2 * XN;       // two accumulators
constexpr int XSF_COLS = 8;             // TMEM columns of scales per stage: 4 for A, 4 for B
constexpr size_t XSMEM = (size_t)XSTAGES * XSTAGE + 1024;

struct MxParams {
  const int* group_start;
  const int* group_rows;
  int G, N, K, ldc;
  int a_row_blocks;            // ceil(a_rows / 128): scale atoms of A per K block
  void* C;
  uint32_t* sf_out;            // epilogue 3: scale words of the quantised output, [N / 256][a_row_blocks][128]
  int* error;
  int epilogue;                // 0: C = bf16(acc); 1: SwiGLU over interleaved gate / up columns, bf16;
                               // 3: SwiGLU, then MXFP8 again: C is e4m3 [*, N / 2] (ldc in bytes) with sf_out
  // Push mode (ret != null, epilogue 0): row `pos` of the result goes to row (ret[pos] & 0xffffff) of the [*, N] bf16
  // buffer at offset y2_off of the heap of process ret[pos] >> 24: the return all-to-all of the MoE layer.
  const unsigned* ret;
  unsigned long long y2_off;
  char* heap[16];
};

struct XTile { int g, m0, n0, rows; bool valid; };

__device__ __forceinline__ XTile xtile_of(const MxParams& p, int t, const int* s_rows, const int* s_start) {
  const int ntn = p.N / XN;
  XTile r; r.valid = false; r.g = 0; r.m0 = 0; r.n0 = 0; r.rows = 0;
  for (int g = 0; g < p.G; g++) {
    const int ntm = (s_rows[g] + XM - 1) / XM;
    const int cnt = ntm * ntn;
    if (t < cnt) {
      const int n = t / ntm, m = t - n * ntm;
      r.g = g; r.m0 = s_start[g] + m * XM; r.n0 = n * XN; r.rows = s_rows[g] - m * XM; r.valid = true;
      return r;
    }
    t -= cnt;
  }
  return r;
}

__device__ __forceinline__ float silu_x(float x) { return x / (1.0f + __expf(-x)); }

// Instruction descriptor of the block-scaled kinds: e4m3 x e4m3, K-major operands, UE8M0 scales; the scale byte each
// operand uses (0..3 inside its TMEM word) is added per MMA.
__host__ __device__ constexpr uint32_t umma_idesc_block_scaled(int M, int N) {
  return ((uint32_t)(N >> 3) << 17) | (1u << 23) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ uint32_t with_scale_ids(uint32_t idesc, uint32_t a_id, uint32_t b_id) {
  return idesc | (b_id << 4) | (a_id << 29);
}

// Shared-memory descriptor of 32 rows x 16 bytes without swizzle (8-row groups 128 bytes apart): the source of a
// tcgen05.cp.32x128b.
__device__ __forceinline__ uint64_t desc_rows16(const void* smem) {
  const uint64_t addr = (smem_u32(smem) & 0x3FFFFu) >> 4;
  return addr | (8ull << 32) | (1ull << 46);
}

// 32 rows x 128 bits from the shared memory of each CTA of the pair into 4 TMEM columns of that CTA, replicated
// over the four lane quarters.
__device__ __forceinline__ void tmem_cp_scales_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void umma_mxf8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(tsfa), "r"(tsfb), "r"(accumulate)
      : "memory");
}

}  // namespace

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(XTHREADS, 1)
grouped_gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                          const __grid_constant__ CUtensorMap tma_sfa, const __grid_constant__ CUtensorMap tma_sfb,
                          const MxParams p) {
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[XSTAGES];    // rank-0 CTA: operand and scale bytes of both CTAs
  __shared__ __align__(8) uint64_t empty_bar[XSTAGES];   // each CTA: its stage has been read by the MMAs
  __shared__ __align__(8) uint64_t tfull_bar[2];         // each CTA: accumulator b is complete
  __shared__ __align__(8) uint64_t tempty_bar[2];        // rank-0 CTA: both CTAs have drained accumulator b
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_rows[kMoeMaxGroups], s_start[kMoeMaxGroups];
  __shared__ int s_abort, s_bad;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  int npairs = gridDim.x >> 1;

  if (tid == 0) {
    s_bad = 0;
    for (int s = 0; s < XSTAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 8); }
    s_abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  for (int i = tid; i < p.G; i += blockDim.x) {
    s_rows[i] = p.group_rows[i]; s_start[i] = p.group_start[i];
    if (s_rows[i] > 0 && (s_start[i] & 127)) s_bad = 1;   // the scale atoms of A would not coincide with the tiles
  }
  if (warp == 1) { tmem_alloc_pair(&tmem_base_s, 512); tmem_relinquish_pair(); }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  const int num_kb = s_bad ? 0 : p.K / XK;
  if (s_bad) {   // both CTAs see the same arrays: nobody does anything, the error is recorded once
    if (blockIdx.x == 0 && tid == 0) atomicExch(p.error, 5);
    npairs = 1 << 30;
  }
  const int first_tile = s_bad ? (1 << 30) : pair;
  volatile int* abort_flag = &s_abort;
  const uint32_t peer_abort = mapa_u32(smem_u32(&s_abort), rank ^ 1u);

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      tma_prefetch_desc(&tma_sfa);
      tma_prefetch_desc(&tma_sfb);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      const int nb128 = p.N / 128;
      for (int t = first_tile; ok; t += npairs) {
        const XTile tl = xtile_of(p, t, s_rows, s_start);
        if (!tl.valid) break;
        const int a_row = tl.m0 + (int)rank * XHM;
        const int b_row = tl.g * p.N + tl.n0 + (int)rank * XHB;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = tiles + (size_t)stage * XSTAGE;
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * XSTAGE);
          const uint32_t bar0 = mapa_u32(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(sa, &tma_a, kb * XK, a_row, bar0);
          tma_load_2d_pair(sa + XA_TILE, &tma_b, kb * XK, b_row, bar0);
          tma_load_2d_pair(sa + XA_TILE + XB_TILE, &tma_sfa, 0, kb * p.a_row_blocks + a_row / 128, bar0);
          tma_load_2d_pair(sa + XA_TILE + XB_TILE + XSF_TILE, &tma_sfb, 0,
                           (tl.g * num_kb + kb) * nb128 + tl.n0 / 128, bar0);
          if (++stage == XSTAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { s_abort = 1; st_cluster_u32(peer_abort, 1); atomicExch(p.error, 1); }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (rank-0 CTA only) ----------------
    if (leader && elect_one()) {
      const uint32_t idesc = umma_idesc_block_scaled(XM, XN);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      int i = 0;
      for (int t = first_tile; ok; t += npairs, i++) {
        const XTile tl = xtile_of(p, t, s_rows, s_start);
        if (!tl.valid) break;
        const int b = i & 1;
        if (!mbar_wait(&tempty_bar[b], (((uint32_t)i >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)b * XN;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint8_t* sa = tiles + (size_t)stage * XSTAGE;
          const uint64_t adesc = umma_desc_sw128(sa);
          const uint64_t bdesc = umma_desc_sw128(sa + XA_TILE);
          const uint32_t tsfa = tmem_base + XACC_COLS + (uint32_t)stage * XSF_COLS;
          const uint32_t tsfb = tsfa + 4;
          tmem_cp_scales_pair(tsfa, desc_rows16(sa + XA_TILE + XB_TILE));
          tmem_cp_scales_pair(tsfb, desc_rows16(sa + XA_TILE + XB_TILE + XSF_TILE));
          #pragma unroll
          for (int kk = 0; kk < XK / 32; kk++)
            umma_mxf8_pair(d_tmem, adesc + 2u * kk, bdesc + 2u * kk, with_scale_ids(idesc, kk, kk), tsfa, tsfb,
                           (uint32_t)((kb | kk) != 0));
          umma_commit_pair(&empty_bar[stage]);   // frees this stage (operands and scales) in both CTAs
          if (++stage == XSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(&tfull_bar[b]);
      }
      if (!ok) { s_abort = 1; st_cluster_u32(peer_abort, 1); atomicExch(p.error, 2); }
    }
  } else {
    // ---------------- epilogue (both CTAs): warps 2..5, TMEM lane quarter = warp % 4 ----------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    __nv_bfloat16* C = static_cast<__nv_bfloat16*>(p.C);
    const uint32_t tempty0 = mapa_u32(smem_u32(&tempty_bar[0]), 0);
    bool ok = true;
    int i = 0;
    for (int t = first_tile; ok; t += npairs, i++) {
      const XTile tl = xtile_of(p, t, s_rows, s_start);
      if (!tl.valid) break;
      const int b = i & 1;
      if (!mbar_wait(&tfull_bar[b], ((uint32_t)i >> 1) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)b * XN;
      const int my_m0 = tl.m0 + (int)rank * XHM;
      const bool live = row < tl.rows - (int)rank * XHM;
      __nv_bfloat16* crow = C + (size_t)(my_m0 + row) * p.ldc;
      if (p.ret && live) {
        const unsigned rv = __ldg(p.ret + my_m0 + row);
        crow = reinterpret_cast<__nv_bfloat16*>(p.heap[rv >> 24] + p.y2_off) + (size_t)(rv & 0xffffffu) * p.ldc;
      }
      if (p.epilogue == 3) {
        // SwiGLU, then the quantiser of the next GEMM's A operand, fused: the 64 outputs of this thread's row are two
        // blocks of 32; each gets its power-of-two scale from the row's own values (no other thread is involved)
        uint8_t* qrow = static_cast<uint8_t*>(p.C) + (size_t)(my_m0 + row) * p.ldc + tl.n0 / 2;
        uint32_t sbytes = 0;
        #pragma unroll 1
        for (int half = 0; half < 2; half++) {
          float o[32];
          #pragma unroll
          for (int cc = 0; cc < 2; cc++) {
            uint32_t r[32];
            tmem_ld32(taddr + half * 64 + cc * 32, r);
            tmem_ld_wait();
            #pragma unroll
            for (int j = 0; j < 16; j++)
              o[cc * 16 + j] = silu_x(__uint_as_float(r[2 * j])) * __uint_as_float(r[2 * j + 1]);
          }
          float m = 0.0f;
          #pragma unroll
          for (int j = 0; j < 32; j++) m = fmaxf(m, fabsf(o[j]));
          const int e = mx_exponent(m);
          const float inv = mx_inv_scale(e);
          sbytes |= (uint32_t)(e + 127) << (8 * half);
          uint32_t w[8];
          #pragma unroll
          for (int j = 0; j < 8; j++) {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(o[4 * j] * inv, o[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(o[4 * j + 2] * inv, o[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
            w[j] = lo | (hi << 16);
          }
          if (live) {
            uint4* dst = reinterpret_cast<uint4*>(qrow + half * 32);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
          }
        }
        if (live) {
          const unsigned R = (unsigned)(my_m0 + row);
          uint32_t* word = p.sf_out + ((size_t)(tl.n0 / 256) * p.a_row_blocks + R / 128) * 128 + (R % 32) * 4 + (R % 128) / 32;
          *reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(word) + ((tl.n0 / 64) & 3)) = (uint16_t)sbytes;
        }
      } else
      #pragma unroll 1
      for (int c = 0; c < XN; c += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c, r);
        tmem_ld_wait();
        if (p.epilogue & 1) {
          uint32_t o[8];
          #pragma unroll
          for (int j = 0; j < 8; j++) {
            float g0 = __uint_as_float(r[4 * j]), u0 = __uint_as_float(r[4 * j + 1]);
            float g1 = __uint_as_float(r[4 * j + 2]), u1 = __uint_as_float(r[4 * j + 3]);
            __nv_bfloat162 v = __floats2bfloat162_rn(silu_x(g0) * u0, silu_x(g1) * u1);
            o[j] = *reinterpret_cast<uint32_t*>(&v);
          }
          if (live) {
            uint4* dst = reinterpret_cast<uint4*>(crow + (tl.n0 + c) / 2);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        } else {
          uint32_t o[16];
          #pragma unroll
          for (int j = 0; j < 16; j++) {
            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            o[j] = *reinterpret_cast<uint32_t*>(&v);
          }
          if (live) {
            uint4* dst = reinterpret_cast<uint4*>(crow + tl.n0 + c);
            #pragma unroll
            for (int j = 0; j < 4; j++) dst[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty0 + 8u * (uint32_t)b);   // 4 warps x 2 CTAs
    }
    if (!ok && lane == 0) { s_abort = 1; st_cluster_u32(peer_abort, 1); atomicExch(p.error, 3); }
  }

  // ---------------- teardown: nobody leaves while the other CTA may still signal it ----------------
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// Row-wise MXFP8 quantisation of bf16 activations: per (row, 32 columns) a power-of-two scale 2^e >= amax / 448 and
// out = x / 2^e as e4m3.  One half-warp handles one 128-column block: sixteen lanes x 8 bf16 (one 16-byte load
// each), so a block of 32 columns is 4 neighbouring lanes.  The four scale bytes of a 128-column block are packed
// into one word; words are stored in the atom order of the GEMM: sf[K / 128][ceil(rows / 128)][128], word
// (r % 32) * 4 + (r % 128) / 32 of its atom for row r.
__global__ void __launch_bounds__(256)
quantize_rows_mx_kernel(const __nv_bfloat16* __restrict__ x, long long rows, int K, int ldx, uint8_t* __restrict__ out,
                        uint32_t* __restrict__ sf) {
  constexpr int kUnroll = 4;
  const int lane16 = threadIdx.x & 15;
  const unsigned kblocks = (unsigned)(K / 128);
  const unsigned nblk = (unsigned)(rows * kblocks);
  const unsigned groups = (gridDim.x * blockDim.x) >> 4;
  const unsigned g0 = (blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const unsigned which = g0 & 1u;
  for (unsigned base = g0 - which; base < nblk; base += groups * kUnroll) {
    uint4 raw[kUnroll];
    unsigned row[kUnroll], kb[kUnroll];
    #pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const unsigned w = base + which + (unsigned)u * groups;
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      row[u] = w / kblocks;
      kb[u] = w - row[u] * kblocks;
      if (w < nblk)
        raw[u] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)row[u] * ldx + kb[u] * 128 + lane16 * 8));
    }
    #pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const unsigned w = base + which + (unsigned)u * groups;
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
      float2 v[4];
      float m = 0.0f;
      #pragma unroll
      for (int j = 0; j < 4; j++) {
        v[j] = __bfloat1622float2(h[j]);
        m = fmaxf(m, fmaxf(fabsf(v[j].x), fabsf(v[j].y)));
      }
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));   // the 4 lanes of one 32-column block
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      const int e = mx_exponent(m);
      const float inv = mx_inv_scale(e);
      const uint32_t byte = (uint32_t)(e + 127);
      // the four blocks of the 128 columns: lanes 0-3, 4-7, 8-11, 12-15 -> bytes 0..3
      uint32_t word = byte << (8 * (lane16 >> 2));
      word |= __shfl_xor_sync(0xffffffffu, word, 4);
      word |= __shfl_xor_sync(0xffffffffu, word, 8);
      if (w < nblk) {
        uint32_t qv[4];
        #pragma unroll
        for (int j = 0; j < 4; j++)
          qv[j] = __nv_cvt_float2_to_fp8x2(make_float2(v[j].x * inv, v[j].y * inv), __NV_SATFINITE, __NV_E4M3);
        *reinterpret_cast<uint2*>(out + (size_t)row[u] * K + kb[u] * 128 + lane16 * 8) =
            make_uint2(qv[0] | (qv[1] << 16), qv[2] | (qv[3] << 16));
        if (lane16 == 0) {
          const unsigned r = row[u], nrb = (unsigned)((rows + 127) / 128);
          sf[((size_t)kb[u] * nrb + r / 128) * 128 + (r % 32) * 4 + (r % 128) / 32] = word;
        }
      }
    }
  }
}

// ---------------- host side ----------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn_mx() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [rows, K] bytes row-major, box = box_rows x 128 bytes, 128-byte swizzle
bool make_map_mx(CUtensorMap* m, const void* base, unsigned long long rows, unsigned long long K, unsigned box_rows) {
  EncodeTiledFn fn = encode_fn_mx();
  if (!fn) return false;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// scale atoms: [atoms, 128] uint32 row-major, box = one atom (512 bytes), no swizzle
bool make_map_atoms(CUtensorMap* m, const void* base, unsigned long long atoms) {
  EncodeTiledFn fn = encode_fn_mx();
  if (!fn) return false;
  cuuint64_t dims[2] = {128, atoms};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, 1};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace
}  // namespace rbv

static int launch_mxfp8(const void* A, const void* sfa, long long a_rows, const void* B, const void* sfb, void* C,
                        void* sf_out, const int* group_start, const int* group_rows, int G, int N, int K, int ldc,
                        int epilogue, int* error_flag, int max_ctas, void* cuda_stream, const unsigned* ret = nullptr,
                        const void* const* heaps = nullptr, int nheaps = 0, unsigned long long y2_off = 0) {
  using namespace rbv;
  if (ret && (epilogue != 0 || !heaps || nheaps < 1 || nheaps > 16 || (y2_off & 15))) return (int)cudaErrorInvalidValue;
  if (G < 1 || G > kMoeMaxGroups || N % XN || K % XK || a_rows < 1 || (ldc % 8)) return (int)cudaErrorInvalidValue;
  if (epilogue == 3 && (!sf_out || N % 256 || ldc % 16 || (reinterpret_cast<uintptr_t>(sf_out) & 15)))
    return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(sfa) | reinterpret_cast<uintptr_t>(sfb)) & 15) return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)XSMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const unsigned long long nrb = (unsigned long long)((a_rows + 127) / 128), nkb = (unsigned long long)(K / XK);
  CUtensorMap ma, mb, msa, msb;
  if (!make_map_mx(&ma, A, (unsigned long long)a_rows, (unsigned long long)K, XHM)) return (int)cudaErrorUnknown;
  if (!make_map_mx(&mb, B, (unsigned long long)G * N, (unsigned long long)K, XHB)) return (int)cudaErrorUnknown;
  if (!make_map_atoms(&msa, sfa, nkb * nrb)) return (int)cudaErrorUnknown;
  if (!make_map_atoms(&msb, sfb, (unsigned long long)G * nkb * (unsigned long long)(N / 128))) return (int)cudaErrorUnknown;
  MxParams p;
  p.group_start = group_start; p.group_rows = group_rows; p.G = G; p.N = N; p.K = K; p.ldc = ldc;
  p.a_row_blocks = (int)nrb;
  p.C = C; p.sf_out = static_cast<uint32_t*>(sf_out); p.error = error_flag; p.epilogue = epilogue;
  p.ret = ret; p.y2_off = y2_off;
  for (int q = 0; q < 16; q++) p.heap[q] = (ret && q < nheaps) ? static_cast<char*>(const_cast<void*>(heaps[q])) : nullptr;
  int grid = max_ctas;
  if (grid <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&grid, cudaDevAttrMultiProcessorCount, dev);
  }
  grid &= ~1;   // whole pairs
  if (grid < 2) return (int)cudaErrorInvalidValue;
  grouped_gemm_mxfp8_kernel<<<grid, XTHREADS, XSMEM, static_cast<cudaStream_t>(cuda_stream)>>>(ma, mb, msa, msb, p);
  return (int)cudaGetLastError();
}

extern "C" int rbv_grouped_gemm_mxfp8(const void* A, const void* sfa, long long a_rows, const void* B, const void* sfb,
                                      void* C, const int* group_start, const int* group_rows, int G, int N, int K,
                                      int ldc, int epilogue, int* error_flag, int max_ctas, void* cuda_stream) {
  if (epilogue != 0 && epilogue != 1) return (int)cudaErrorInvalidValue;
  return launch_mxfp8(A, sfa, a_rows, B, sfb, C, nullptr, group_start, group_rows, G, N, K, ldc, epilogue, error_flag,
                      max_ctas, cuda_stream);
}

extern "C" int rbv_grouped_gemm_mxfp8_push(const void* A, const void* sfa, long long a_rows, const void* B,
                                           const void* sfb, const int* group_start, const int* group_rows, int G,
                                           int N, int K, const unsigned* ret, const void* const* heaps, int nheaps,
                                           unsigned long long y2_off, int* error_flag, int max_ctas,
                                           void* cuda_stream) {
  if (!ret) return (int)cudaErrorInvalidValue;
  return launch_mxfp8(A, sfa, a_rows, B, sfb, const_cast<void*>(heaps ? heaps[0] : nullptr), nullptr, group_start,
                      group_rows, G, N, K, N, 0, error_flag, max_ctas, cuda_stream, ret, heaps, nheaps, y2_off);
}

extern "C" int rbv_grouped_gemm_mxfp8_swiglu_q(const void* A, const void* sfa, long long a_rows, const void* B,
                                               const void* sfb, void* Cq, void* sf_out, const int* group_start,
                                               const int* group_rows, int G, int N, int K, int ldc_bytes,
                                               int* error_flag, int max_ctas, void* cuda_stream) {
  return launch_mxfp8(A, sfa, a_rows, B, sfb, Cq, sf_out, group_start, group_rows, G, N, K, ldc_bytes, 3, error_flag,
                      max_ctas, cuda_stream);
}

extern "C" int rbv_quantize_rows_mxfp8(const void* x_bf16, long long rows, int K, int ldx, void* out_fp8, void* sf,
                                       void* cuda_stream) {
  using namespace rbv;
  if (K % 128 || rows < 1 || (ldx % 8) || (reinterpret_cast<uintptr_t>(x_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(out_fp8) & 7) || (reinterpret_cast<uintptr_t>(sf) & 15))
    return (int)cudaErrorInvalidValue;
  const long long nblk = rows * (K / 128);
  if (nblk >= (1ll << 31)) return (int)cudaErrorInvalidValue;
  long long grid = (nblk + 63) / 64;
  if (grid > 148 * 8) grid = 148 * 8;
  if (grid < 1) grid = 1;
  quantize_rows_mx_kernel<<<(int)grid, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const __nv_bfloat16*>(x_bf16), rows, K, ldx, static_cast<uint8_t*>(out_fp8),
      static_cast<uint32_t*>(sf));
  return (int)cudaGetLastError();
}
