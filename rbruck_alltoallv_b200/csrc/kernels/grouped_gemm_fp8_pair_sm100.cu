// Block-scaled fp8 (e4m3) grouped GEMM on CTA PAIRS (tcgen05 cta_group::2): the pair version of
// grouped_gemm_fp8_sm100.cu, same operands, scales and epilogues.
//
//   C[rows of g] = epi( sum_kb  sa[kb][row] * sb[g][n / 128][kb] * ( A[rows, kb] * B_g[n-tile, kb]^T ) )
//
// Two CTAs on neighbouring SMs share a 256 x 128 tile: each fetches its own 128 rows of A and its own 64 of the 128
// weight rows per K block (24 KB per SM instead of 32 KB for the same MMAs, 8 stages instead of 6), the rank-0 CTA
// issues four tcgen05.mma.cta_group::2.kind::f8f6f4 (M 256, N 128, K 32) per K block into one of four 128-column TMEM
// slots, and the eight scaling / epilogue warps of EACH CTA pull the 128 accumulator rows of their own TMEM, scale and
// accumulate them in registers (packed fp32 FMAs) and hand the slot back to the rank-0 CTA across the cluster.
// TMA loads carry no cluster multicast.  All waits are bounded; on expiry both CTAs are told, record an error, release
// their TMEM and return.  No counterpart in the reference.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels/sm100_ptx.cuh"
#include "rbv/moe.h"

namespace rbv {

using namespace sm100;

namespace {

constexpr int QM = 256;                 // tile rows per pair
constexpr int QHM = 128;                // rows per CTA
constexpr int QN = 128;                 // tile columns
constexpr int QHB = 64;                 // weight rows each CTA fetches
constexpr int QK = 128;                 // one 128-byte swizzle row of fp8
constexpr int QSTAGES = 8, QSLOTS = 4;
constexpr int QA_TILE = QHM * QK;       // 16 KB
constexpr int QB_TILE = QHB * QK;       // 8 KB
constexpr int QSTAGE = QA_TILE + QB_TILE;
constexpr int QTHREADS = 320;           // TMA warp, MMA warp, 8 scaling / epilogue warps
constexpr int QHN = QN / 2;             // columns per epilogue warp (two warps share a TMEM lane quarter)
constexpr size_t QSMEM = (size_t)QSTAGES * QSTAGE + 1024;

struct Fp8PairParams {
  const int* group_start;
  const int* group_rows;
  int G, N, K, ldc;
  long long a_rows;            // rows of A (= leading dimension of the transposed scale array)
  const float* a_scale;        // [K / 128][a_rows]
  const float* b_scale;        // [G][N / 128][K / 128]
  void* C;
  int* error;
  int epilogue;                // bit 0: SwiGLU over interleaved gate / up columns; bit 1: coarse scales
};

struct QTile { int g, m0, n0, rows; bool valid; };

__device__ __forceinline__ QTile qtile_of(const Fp8PairParams& p, int t, const int* s_rows, const int* s_start) {
  const int ntn = p.N / QN;
  QTile r; r.valid = false; r.g = 0; r.m0 = 0; r.n0 = 0; r.rows = 0;
  for (int g = 0; g < p.G; g++) {
    const int ntm = (s_rows[g] + QM - 1) / QM;
    const int cnt = ntm * ntn;
    if (t < cnt) {
      const int n = t / ntm, m = t - n * ntm;
      r.g = g; r.m0 = s_start[g] + m * QM; r.n0 = n * QN; r.rows = s_rows[g] - m * QM; r.valid = true;
      return r;
    }
    t -= cnt;
  }
  return r;
}

__device__ __forceinline__ float silu_q(float x) { return x / (1.0f + __expf(-x)); }

// fp8 (e4m3 x e4m3 -> fp32) MMA of a CTA pair: M 256, issued by one thread of the rank-0 CTA
__device__ __forceinline__ void umma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

}  // namespace

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(QTHREADS, 1)
grouped_gemm_fp8_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                             const Fp8PairParams p) {
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[QSTAGES];    // used in the rank-0 CTA: bytes of both CTAs' loads
  __shared__ __align__(8) uint64_t empty_bar[QSTAGES];   // in each CTA: its stage has been read by the MMAs
  __shared__ __align__(8) uint64_t tfull_bar[QSLOTS];    // in each CTA: TMEM slot holds a finished K block (or tile)
  __shared__ __align__(8) uint64_t tempty_bar[QSLOTS];   // used in the rank-0 CTA: all 16 scaling warps took the slot
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_rows[kMoeMaxGroups], s_start[kMoeMaxGroups];
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (tid == 0) {
    for (int s = 0; s < QSTAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < QSLOTS; b++) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 16); }
    s_abort = 0;
    mbar_fence_init();
  }
  for (int i = tid; i < p.G; i += blockDim.x) { s_rows[i] = p.group_rows[i]; s_start[i] = p.group_start[i]; }
  if (warp == 1) { tmem_alloc_pair(&tmem_base_s, 512); tmem_relinquish_pair(); }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  const int num_kb = p.K / QK;
  volatile int* abort_flag = &s_abort;
  const uint32_t peer_abort = mapa_u32(smem_u32(&s_abort), rank ^ 1u);

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; ok; t += npairs) {
        const QTile tl = qtile_of(p, t, s_rows, s_start);
        if (!tl.valid) break;
        const int a_row = tl.m0 + (int)rank * QHM;
        const int b_row = tl.g * p.N + tl.n0 + (int)rank * QHB;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = tiles + (size_t)stage * QSTAGE;
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * QSTAGE);
          const uint32_t bar0 = mapa_u32(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(sa, &tma_a, kb * QK, a_row, bar0);
          tma_load_2d_pair(sa + QA_TILE, &tma_b, kb * QK, b_row, bar0);
          if (++stage == QSTAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { s_abort = 1; st_cluster_u32(peer_abort, 1); atomicExch(p.error, 1); }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (rank-0 CTA only) ----------------
    if (leader && elect_one()) {
      const uint32_t idesc = umma_idesc(QM, QN, 0 /*e4m3*/);
      const bool coarse = (p.epilogue & 2) != 0;
      int stage = 0; uint32_t phase = 0;
      unsigned it = 0;   // running K-block count -> TMEM slot ring
      bool ok = true;
      for (int t = pair; ok; t += npairs) {
        const QTile tl = qtile_of(p, t, s_rows, s_start);
        if (!tl.valid) break;
        for (int kb = 0; kb < num_kb && ok; kb++) {
          // fine scales: one TMEM slot per K block; coarse scales: one per tile, accumulated over all K blocks
          const int slot = it % QSLOTS;
          if (!coarse || kb == 0)
            if (!mbar_wait(&tempty_bar[slot], ((it / QSLOTS) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint8_t* sa = tiles + (size_t)stage * QSTAGE;
          const uint64_t adesc = umma_desc_sw128(sa);
          const uint64_t bdesc = umma_desc_sw128(sa + QA_TILE);
          const uint32_t d_tmem = tmem_base + (uint32_t)slot * QN;
          #pragma unroll
          for (int kk = 0; kk < QK / 32; kk++)
            umma_f8_pair(d_tmem, adesc + 2u * kk, bdesc + 2u * kk, idesc,
                         (uint32_t)(coarse ? (kb | kk) != 0 : kk != 0));
          umma_commit_pair(&empty_bar[stage]);
          if (!coarse || kb == num_kb - 1) { umma_commit_pair(&tfull_bar[slot]); it++; }
          if (++stage == QSTAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { s_abort = 1; st_cluster_u32(peer_abort, 1); atomicExch(p.error, 2); }
    }
  } else {
    // ---------------- scaling / epilogue (both CTAs) ----------------
    // warps 2..9: lane quarter = warp % 4, column half = (warp - 2) / 4
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    __nv_bfloat16* C = static_cast<__nv_bfloat16*>(p.C);
    const int nkb = num_kb;
    const uint32_t tempty0 = mapa_u32(smem_u32(&tempty_bar[0]), 0);   // the rank-0 CTA's slot-free barriers
    unsigned it = 0;
    bool ok = true;
    for (int t = pair; ok; t += npairs) {
      const QTile tl = qtile_of(p, t, s_rows, s_start);
      if (!tl.valid) break;
      float2 acc2[QHN / 2];
      #pragma unroll
      for (int j = 0; j < QHN / 2; j++) acc2[j] = make_float2(0.0f, 0.0f);
      const int my_m0 = tl.m0 + (int)rank * QHM;
      const int my_rows = tl.rows - (int)rank * QHM;
      const long long arow = (long long)my_m0 + row;
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
        const int slot = it % QSLOTS;
        const float scale = in_a ? sa_q[0] * sb_q[0] : 0.0f;
        uint32_t t0[32], t1[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)half * QHN + (uint32_t)slot * QN;
        if (!mbar_wait(&tfull_bar[slot], (it / QSLOTS) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        tmem_ld32(taddr, t0);
        tmem_ld32(taddr + 32, t1);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty0 + 8u * (uint32_t)slot);
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
        const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)half * QHN;
        if (!mbar_wait(&tfull_bar[it % QSLOTS], (it / QSLOTS) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        tmem_ld32(tbase + (uint32_t)(it % QSLOTS) * QN, r0);
        for (int kb0 = 0; kb0 < nkb && ok; kb0 += kDepth) {
          #pragma unroll
          for (int j = 0; j < kDepth; j++) {
            const int kb = kb0 + j;
            if (kb >= nkb) break;
            const int slot = it % QSLOTS;
            const float scale = in_a ? sa_q[j] * sb_q[j] : 0.0f;
            const float2 s2 = make_float2(scale, scale);
            if (kb + kDepth < nkb) {
              sa_q[j] = __ldg(sa + (size_t)(kb + kDepth) * p.a_rows);
              sb_q[j] = __ldg(sb + kb + kDepth);
            }
            tmem_ld_wait();                                            // first half of this K block has landed
            tmem_ld32(tbase + (uint32_t)slot * QN + 32, r1);
            #pragma unroll
            for (int c = 0; c < 16; c++)
              acc2[c] = __ffma2_rn(s2, make_float2(__uint_as_float(r0[2 * c]), __uint_as_float(r0[2 * c + 1])), acc2[c]);
            tmem_ld_wait();                                            // second half has landed
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty0 + 8u * (uint32_t)slot);         // the slot is free once it sits in registers
            it++;
            if (kb + 1 < nkb) {
              if (!mbar_wait(&tfull_bar[it % QSLOTS], (it / QSLOTS) & 1u, abort_flag)) { ok = false; break; }
              tc_fence_after_sync();
              tmem_ld32(tbase + (uint32_t)(it % QSLOTS) * QN, r0);
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
      if (row < my_rows) {
        __nv_bfloat16* crow = C + (size_t)(my_m0 + row) * p.ldc;
        if (p.epilogue & 1) {
          uint4* dst = reinterpret_cast<uint4*>(crow + (tl.n0 + half * QHN) / 2);
          #pragma unroll
          for (int v = 0; v < QHN / 16; v++) {
            uint32_t o[4];
            #pragma unroll
            for (int j = 0; j < 4; j++) {
              const int c = v * 16 + j * 4;
              __nv_bfloat162 h = __floats2bfloat162_rn(silu_q(acc[c]) * acc[c + 1], silu_q(acc[c + 2]) * acc[c + 3]);
              o[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
          uint4* dst = reinterpret_cast<uint4*>(crow + tl.n0 + half * QHN);
          #pragma unroll
          for (int v = 0; v < QHN / 8; v++) {
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

// ---------------- host side ----------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn8p() {
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
bool make_map8p(CUtensorMap* m, const void* base, unsigned long long rows, unsigned long long K, unsigned box_rows) {
  EncodeTiledFn fn = encode_fn8p();
  if (!fn) return false;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace
}  // namespace rbv

extern "C" int rbv_grouped_gemm_fp8_pair(const void* A, const float* a_scale_t, long long a_rows, const void* B,
                                         const float* b_scale, void* C, const int* group_start, const int* group_rows,
                                         int G, int N, int K, int ldc, int epilogue, int* error_flag, int max_ctas,
                                         void* cuda_stream) {
  using namespace rbv;
  if (G < 1 || G > kMoeMaxGroups || N % QN || K % QK || a_rows < 1 || (ldc % 8)) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_fp8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)QSMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap ma, mb;
  if (!make_map8p(&ma, A, (unsigned long long)a_rows, (unsigned long long)K, QHM)) return (int)cudaErrorUnknown;
  if (!make_map8p(&mb, B, (unsigned long long)G * N, (unsigned long long)K, QHB)) return (int)cudaErrorUnknown;
  Fp8PairParams p;
  p.group_start = group_start; p.group_rows = group_rows; p.G = G; p.N = N; p.K = K; p.ldc = ldc;
  p.a_rows = a_rows; p.a_scale = a_scale_t; p.b_scale = b_scale; p.C = C; p.error = error_flag; p.epilogue = epilogue;
  int grid = max_ctas;
  if (grid <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&grid, cudaDevAttrMultiProcessorCount, dev);
  }
  grid &= ~1;   // whole pairs
  if (grid < 2) return (int)cudaErrorInvalidValue;
  grouped_gemm_fp8_pair_kernel<<<grid, QTHREADS, QSMEM, static_cast<cudaStream_t>(cuda_stream)>>>(ma, mb, p);
  return (int)cudaGetLastError();
}
