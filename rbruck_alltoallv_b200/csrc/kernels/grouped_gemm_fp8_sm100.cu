// Block-scaled fp8 (e4m3) grouped GEMM for the expert FFN, sm_100a: the fp8 option of the MoE path.
//
//   C[rows of g] = epi( sum_kb  sa[kb][row] * sb[g][n / 128][kb] * ( A[rows, kb] * B_g[n-tile, kb]^T ) )
//
// Activations carry one fp32 scale per row and 128-wide K block ("1 x 128"), weights one per 128 x 128 block.
// These blocks do not match the 32-element hardware scaling of the MX instruction kinds, so scaling is done in
// software: every K block (128 fp8 = one 128-byte swizzle row) is multiplied on its own by four
// tcgen05.mma.kind::f8f6f4 (K = 32) into one of four 128-column TMEM slots; the four epilogue warps pull each
// finished slot with tcgen05.ld (eight warps: two per TMEM lane quarter, 64 columns each, loaded as two pipelined
// halves), hand the slot back as soon as it sits in registers, and scale and accumulate with packed fp32 FMAs
// (64 fp32 per thread; scales prefetched four K blocks ahead).  MMA of block kb + 1..3 overlaps the scaling of block kb.
// Same structure as the bf16 kernel otherwise: TMA producer warp (plain tiled loads, no multicast), one MMA
// thread, persistent static tile schedule over ragged groups, bounded waits.  No counterpart in the reference.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels/sm100_ptx.cuh"
#include "rbv/moe.h"

namespace rbv {

using namespace sm100;

namespace {

constexpr int BM = 128, BN = 128, BK = 128, STAGES = 6, SLOTS = 4;
constexpr int A_TILE = BM * BK;          // 16 KB (1 byte per element)
constexpr int B_TILE = BN * BK;          // 16 KB
constexpr int STAGE = A_TILE + B_TILE;
constexpr int THREADS = 320;          // TMA warp, MMA warp, 8 scaling / epilogue warps
constexpr int HN = BN / 2;            // columns per epilogue warp (two warps share a TMEM lane quarter)
constexpr size_t SMEM = (size_t)STAGES * STAGE + 1024 + 256;

struct Fp8Params {
  const int* group_start;
  const int* group_rows;
  int G, N, K, ldc;
  long long a_rows;            // rows of A (= leading dimension of the transposed scale array)
  const float* a_scale;        // [K / 128][a_rows]
  const float* b_scale;        // [G][N / 128][K / 128]
  void* C;
  int* error;
  int epilogue;                // bit 0: SwiGLU over interleaved gate / up columns; bit 1: coarse scales (the
                               // scales of K block 0 hold for the whole row / weight block: one TMEM read per tile)
};

struct Tile { int g, m0, n0, rows_left; bool valid; };

__device__ __forceinline__ Tile tile_of(const Fp8Params& p, int t, const int* s_rows, const int* s_start) {
  const int ntn = p.N / BN;
  Tile r; r.valid = false; r.g = 0; r.m0 = 0; r.n0 = 0; r.rows_left = 0;
  for (int g = 0; g < p.G; g++) {
    const int ntm = (s_rows[g] + BM - 1) / BM;
    const int cnt = ntm * ntn;
    if (t < cnt) {
      const int n = t / ntm, m = t - n * ntm;
      r.g = g; r.m0 = s_start[g] + m * BM; r.n0 = n * BN; r.rows_left = s_rows[g] - m * BM; r.valid = true;
      return r;
    }
    t -= cnt;
  }
  return r;
}

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

}  // namespace

__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                        const Fp8Params p) {
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[SLOTS];
  __shared__ __align__(8) uint64_t tempty_bar[SLOTS];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_rows[kMoeMaxGroups], s_start[kMoeMaxGroups];
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < SLOTS; b++) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 8); }
    s_abort = 0;
    mbar_fence_init();
  }
  for (int i = tid; i < p.G; i += blockDim.x) { s_rows[i] = p.group_rows[i]; s_start[i] = p.group_start[i]; }
  if (warp == 1) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  const int num_kb = p.K / BK;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok; t += gridDim.x) {
        const Tile tl = tile_of(p, t, s_rows, s_start);
        if (!tl.valid) break;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = tiles + (size_t)stage * STAGE;
          mbar_arrive_expect_tx(&full_bar[stage], STAGE);
          tma_load_2d(sa, &tma_a, kb * BK, tl.m0, &full_bar[stage]);
          tma_load_2d(sa + A_TILE, &tma_b, kb * BK, tl.g * p.N + tl.n0, &full_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { s_abort = 1; atomicExch(p.error, 1); }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = umma_idesc(BM, BN, 0 /*e4m3*/);
      const bool coarse = (p.epilogue & 2) != 0;
      int stage = 0; uint32_t phase = 0;
      unsigned it = 0;   // running K-block count -> TMEM slot ring
      bool ok = true;
      for (int t = blockIdx.x; ok; t += gridDim.x) {
        const Tile tl = tile_of(p, t, s_rows, s_start);
        if (!tl.valid) break;
        for (int kb = 0; kb < num_kb && ok; kb++) {
          // fine scales: one TMEM slot per K block; coarse scales: one per tile, accumulated over all K blocks
          const int slot = it % SLOTS;
          if (!coarse || kb == 0)
            if (!mbar_wait(&tempty_bar[slot], ((it / SLOTS) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint8_t* sa = tiles + (size_t)stage * STAGE;
          const uint64_t adesc = umma_desc_sw128(sa);
          const uint64_t bdesc = umma_desc_sw128(sa + A_TILE);
          const uint32_t d_tmem = tmem_base + (uint32_t)slot * BN;
          #pragma unroll
          for (int kk = 0; kk < BK / 32; kk++)
            umma_f8(d_tmem, adesc + 2u * kk, bdesc + 2u * kk, idesc, (uint32_t)(coarse ? (kb | kk) != 0 : kk != 0));
          umma_commit(&empty_bar[stage]);
          if (!coarse || kb == num_kb - 1) { umma_commit(&tfull_bar[slot]); it++; }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { s_abort = 1; atomicExch(p.error, 2); }
    }
  } else {
    // warps 2..9: lane quarter = warp % 4, column half = (warp - 2) / 4
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    __nv_bfloat16* C = static_cast<__nv_bfloat16*>(p.C);
    const int nkb = num_kb;
    unsigned it = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok; t += gridDim.x) {
      const Tile tl = tile_of(p, t, s_rows, s_start);
      if (!tl.valid) break;
      float2 acc2[HN / 2];
      #pragma unroll
      for (int j = 0; j < HN / 2; j++) acc2[j] = make_float2(0.0f, 0.0f);
      const long long arow = (long long)tl.m0 + row;
      const bool in_a = arow < p.a_rows;
      const float* sb = p.b_scale + ((size_t)tl.g * (p.N / 128) + tl.n0 / 128) * nkb;
      const float* sa = p.a_scale + (in_a ? arow : 0);
      // Scales are fetched kDepth K blocks ahead, so that their L2 latency never sits between a finished MMA
      // and its scaling.
      constexpr int kDepth = 4;
      float sa_q[kDepth], sb_q[kDepth];
      #pragma unroll
      for (int j = 0; j < kDepth; j++) {
        sa_q[j] = (j < nkb) ? __ldg(sa + (size_t)j * p.a_rows) : 0.0f;
        sb_q[j] = (j < nkb) ? __ldg(sb + j) : 0.0f;
      }
      if (p.epilogue & 2) {
        // coarse scales: the tile was accumulated over all K blocks in one TMEM slot; read it once and scale
        const int slot = it % SLOTS;
        const float scale = in_a ? sa_q[0] * sb_q[0] : 0.0f;
        uint32_t t0[32], t1[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)half * HN + (uint32_t)slot * BN;
        if (!mbar_wait(&tfull_bar[slot], (it / SLOTS) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        tmem_ld32(taddr, t0);
        tmem_ld32(taddr + 32, t1);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[slot]);
        it++;
        #pragma unroll
        for (int c = 0; c < 16; c++) {
          acc2[c] = make_float2(scale * __uint_as_float(t0[2 * c]), scale * __uint_as_float(t0[2 * c + 1]));
          acc2[16 + c] = make_float2(scale * __uint_as_float(t1[2 * c]), scale * __uint_as_float(t1[2 * c + 1]));
        }
      } else {
      // Two 32-column loads per K block, software-pipelined: while one half is multiplied, the other half (or
      // the first half of the next K block) is in flight from TMEM.
      uint32_t r0[32], r1[32];
      const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)half * HN;
      if (!mbar_wait(&tfull_bar[it % SLOTS], (it / SLOTS) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      tmem_ld32(tbase + (uint32_t)(it % SLOTS) * BN, r0);
      for (int kb0 = 0; kb0 < nkb && ok; kb0 += kDepth) {
        #pragma unroll
        for (int j = 0; j < kDepth; j++) {
          const int kb = kb0 + j;
          if (kb >= nkb) break;
          const int slot = it % SLOTS;
          const float scale = in_a ? sa_q[j] * sb_q[j] : 0.0f;
          const float2 s2 = make_float2(scale, scale);
          if (kb + kDepth < nkb) {
            sa_q[j] = __ldg(sa + (size_t)(kb + kDepth) * p.a_rows);
            sb_q[j] = __ldg(sb + kb + kDepth);
          }
          tmem_ld_wait();                                            // first half of this K block has landed
          tmem_ld32(tbase + (uint32_t)slot * BN + 32, r1);
          #pragma unroll
          for (int c = 0; c < 16; c++)
            acc2[c] = __ffma2_rn(s2, make_float2(__uint_as_float(r0[2 * c]), __uint_as_float(r0[2 * c + 1])), acc2[c]);
          tmem_ld_wait();                                            // second half has landed
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[slot]);             // the slot is free once it sits in registers
          it++;
          if (kb + 1 < nkb) {
            if (!mbar_wait(&tfull_bar[it % SLOTS], (it / SLOTS) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            tmem_ld32(tbase + (uint32_t)(it % SLOTS) * BN, r0);
          }
          #pragma unroll
          for (int c = 0; c < 16; c++)
            acc2[16 + c] =
                __ffma2_rn(s2, make_float2(__uint_as_float(r1[2 * c]), __uint_as_float(r1[2 * c + 1])), acc2[16 + c]);
        }
      }
      }
      const float* acc = reinterpret_cast<const float*>(acc2);
      if (!ok) break;
      if (row < tl.rows_left) {
        __nv_bfloat16* crow = C + (size_t)(tl.m0 + row) * p.ldc;
        if (p.epilogue & 1) {
          uint4* dst = reinterpret_cast<uint4*>(crow + (tl.n0 + half * HN) / 2);
          #pragma unroll
          for (int v = 0; v < HN / 16; v++) {
            uint32_t o[4];
            #pragma unroll
            for (int j = 0; j < 4; j++) {
              const int c = v * 16 + j * 4;
              __nv_bfloat162 h = __floats2bfloat162_rn(silu(acc[c]) * acc[c + 1], silu(acc[c + 2]) * acc[c + 3]);
              o[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
          uint4* dst = reinterpret_cast<uint4*>(crow + tl.n0 + half * HN);
          #pragma unroll
          for (int v = 0; v < HN / 8; v++) {
            uint32_t o[4];
            #pragma unroll
            for (int j = 0; j < 4; j++) {
              __nv_bfloat162 h = __floats2bfloat162_rn(acc[v * 8 + 2 * j], acc[v * 8 + 2 * j + 1]);
              o[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
    }
    if (!ok && lane == 0) { s_abort = 1; atomicExch(p.error, 3); }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// Row-wise 1 x 128 quantisation of bf16 activations to e4m3: out[row, k] = x[row, k] / scale, scale = amax / 448.
// Sixteen lanes per (row, 128-column block), eight bf16 (one 16-byte load) per lane, four blocks per half-warp in
// flight before the first reduction; scales are stored transposed, [K / 128][rows].
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, long long rows, int K, int ldx, uint8_t* __restrict__ out,
                     float* __restrict__ scale_t) {
  constexpr int kUnroll = 4;
  const int lane16 = threadIdx.x & 15;
  const unsigned kblocks = (unsigned)(K / 128);
  const unsigned nblk = (unsigned)(rows * kblocks);                       // < 2^31, checked by the caller
  const unsigned groups = (gridDim.x * blockDim.x) >> 4;                  // half-warps in the grid
  const unsigned g0 = (blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const unsigned which = g0 & 1u;   // the two half-warps of a warp take neighbouring blocks; the loop is warp-uniform
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
      #pragma unroll
      for (int o = 8; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));   // stays inside 16 lanes
      if (w < nblk) {
        const float scale = m > 0.0f ? m / 448.0f : 1.0f;
        const float inv = 1.0f / scale;
        uint32_t q[4];
        #pragma unroll
        for (int j = 0; j < 4; j++)
          q[j] = __nv_cvt_float2_to_fp8x2(make_float2(v[j].x * inv, v[j].y * inv), __NV_SATFINITE, __NV_E4M3);
        *reinterpret_cast<uint2*>(out + (size_t)row[u] * K + kb[u] * 128 + lane16 * 8) =
            make_uint2(q[0] | (q[1] << 16), q[2] | (q[3] << 16));
        if (lane16 == 0) scale_t[(size_t)kb[u] * rows + row[u]] = scale;
      }
    }
  }
}

}  // namespace rbv

// ---------------- host side ----------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn8() {
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

// [rows, K] bytes row-major, box = 128 rows x 128 bytes, 128-byte swizzle
bool make_map8(CUtensorMap* m, const void* base, unsigned long long rows, unsigned long long K) {
  EncodeTiledFn fn = encode_fn8();
  if (!fn) return false;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K};
  cuuint32_t box[2] = {128, 128};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" int rbv_grouped_gemm_fp8(const void* A, const float* a_scale_t, long long a_rows, const void* B,
                                    const float* b_scale, void* C, const int* group_start, const int* group_rows,
                                    int G, int N, int K, int ldc, int epilogue, int* error_flag, int max_ctas,
                                    void* cuda_stream) {
  using namespace rbv;
  // CTA pairs (grouped_gemm_fp8_pair_sm100.cu) unless switched off (RBV_GEMM_PAIR=0 / rbv_grouped_gemm_set_pair(0))
  if (rbv_grouped_gemm_pair_enabled())
    return rbv_grouped_gemm_fp8_pair(A, a_scale_t, a_rows, B, b_scale, C, group_start, group_rows, G, N, K, ldc,
                                     epilogue, error_flag, max_ctas, cuda_stream);
  if (G < 1 || G > kMoeMaxGroups || N % BN || K % BK || a_rows < 1 || (ldc % 8)) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap ma, mb;
  if (!make_map8(&ma, A, (unsigned long long)a_rows, (unsigned long long)K)) return (int)cudaErrorUnknown;
  if (!make_map8(&mb, B, (unsigned long long)G * N, (unsigned long long)K)) return (int)cudaErrorUnknown;
  Fp8Params p;
  p.group_start = group_start; p.group_rows = group_rows; p.G = G; p.N = N; p.K = K; p.ldc = ldc;
  p.a_rows = a_rows; p.a_scale = a_scale_t; p.b_scale = b_scale; p.C = C; p.error = error_flag; p.epilogue = epilogue;
  int grid = max_ctas;
  if (grid <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&grid, cudaDevAttrMultiProcessorCount, dev);
  }
  grouped_gemm_fp8_kernel<<<grid, THREADS, SMEM, static_cast<cudaStream_t>(cuda_stream)>>>(ma, mb, p);
  return (int)cudaGetLastError();
}

extern "C" int rbv_quantize_rows_fp8(const void* x_bf16, long long rows, int K, int ldx, void* out_fp8, float* scale_t,
                                     void* cuda_stream) {
  using namespace rbv;
  if (K % 128 || rows < 1 || (ldx % 8) || (reinterpret_cast<uintptr_t>(x_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(out_fp8) & 7))
    return (int)cudaErrorInvalidValue;
  const long long nblk = rows * (K / 128);
  if (nblk >= (1ll << 31)) return (int)cudaErrorInvalidValue;
  long long grid = (nblk + 63) / 64;   // 16 half-warps per block, four blocks of columns each
  if (grid > 148 * 8) grid = 148 * 8;
  if (grid < 1) grid = 1;
  quantize_rows_kernel<<<(int)grid, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const __nv_bfloat16*>(x_bf16), rows, K, ldx, static_cast<uint8_t*>(out_fp8), scale_t);
  return (int)cudaGetLastError();
}
