// Grouped (ragged-batch) GEMM for the expert FFN of the MoE path, written for sm_100a:
// TMA-fed shared-memory pipeline, tcgen05.mma with fp32 accumulators in TMEM, epilogue through
// tcgen05.ld.  No counterpart exists in the reference (it has no compute kernels).
//
//   C[rows of group g] = epilogue( A[rows of group g] (M_g x K, K-major) * B_g^T (N x K, K-major) )
//
// Groups are the local experts; their row ranges (start, count) are device-resident because they
// come out of the dispatch kernel.  One persistent CTA per SM walks a static tile schedule:
//   warp 0    TMA producer   (A tile 128 x 64 and B tile 256 x 64 bf16 per stage, 128-byte swizzle)
//   warp 1    MMA issuer     (one elected thread, 4 x tcgen05.mma M128 N256 K16 per stage)
//   warps 2-5 epilogue       (TMEM -> registers -> global; SwiGLU fused for the first FFN GEMM)
// TMEM holds two 128 x 256 fp32 accumulators (all 512 columns), so the epilogue of tile i overlaps
// the MMAs of tile i + 1.  Tiles of one group are ordered n-major / m-minor: CTAs running at the
// same time share a weight tile in L2, and each weight tile is read from HBM once.
//
// TMA loads carry no cluster multicast (the kernel runs on every GPU of a multi-GPU job).
// All waits are bounded; on expiry the CTA records an error, releases its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "kernels/sm100_ptx.cuh"
#include "rbv/moe.h"

namespace rbv {

using namespace sm100;

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_TILE_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_TILE_BYTES = BN * BK * 2;   // 32 KB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr size_t GEMM_SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct GemmParams {
  const int* group_start;   // [G] first row of each group in A / C
  const int* group_rows;    // [G] rows of each group
  int G;
  int N, K;                 // B_g is N x K
  int ldc;                  // elements between rows of C
  void* C;                  // bf16
  int* error;               // set to non-zero when a wait ran out
  int epilogue;             // 0: C = bf16(acc); 1: C[:, j] = bf16(silu(acc[:, 2j]) * acc[:, 2j+1])
  // Gated start (null: none): the rows of group g may be loaded once ready[g] >= ready_target[g].  The counters are
  // bumped by the kernels that deliver the rows, possibly from other GPUs, while this kernel is already running.
  const unsigned long long* ready;
  const unsigned long long* ready_target;
  unsigned long long timeout_ns;
};

struct Tile { int g, m0, n0, rows_left; bool valid; };

// Waits (bounded) until all rows of group g have been delivered.  The deliveries are generic-proxy stores made
// visible by a fence and a relaxed reduction at system scope; the loads that follow go through the TMA unit, hence
// the proxy fence after the acquire.
__device__ bool wait_group_ready(const GemmParams& p, int g, volatile int* abort_flag) {
  const unsigned long long target = p.ready_target[g];
  unsigned long long t0 = 0;
  for (unsigned it = 0;; it++) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p.ready + g) : "memory");
    if (v >= target) break;
    if ((it & 15u) == 15u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (!t0) t0 = now;
      if (*abort_flag || now - t0 > p.timeout_ns) return false;
      __nanosleep(64);
    }
  }
  asm volatile("fence.proxy.async;" ::: "memory");
  return true;
}

// Tile t of the static schedule: groups in order; inside a group n-major, m fastest.
__device__ __forceinline__ Tile tile_of(const GemmParams& p, int t, const int* s_rows, const int* s_start) {
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

__global__ void __launch_bounds__(GEMM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const GemmParams p) {
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_rows[kMoeMaxGroups], s_start[kMoeMaxGroups];
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 4); }
    s_abort = 0;
    mbar_fence_init();
  }
  for (int i = tid; i < p.G; i += blockDim.x) { s_rows[i] = p.group_rows[i]; s_start[i] = p.group_start[i]; }
  if (warp == 1) { tmem_alloc(&tmem_base_s, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  const int num_kb = p.K / BK;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      int ready_g = -1;   // groups up to this one are known to be complete
      for (int t = blockIdx.x; ok; t += gridDim.x) {
        const Tile tl = tile_of(p, t, s_rows, s_start);
        if (!tl.valid) break;
        if (p.ready && tl.g > ready_g) {
          if (!wait_group_ready(p, tl.g, abort_flag)) { ok = false; break; }
          ready_g = tl.g;
        }
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = tiles + (size_t)stage * STAGE_BYTES;
          uint8_t* sb = sa + A_TILE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(sa, &tma_a, kb * BK, tl.m0, &full_bar[stage]);
          tma_load_2d(sb, &tma_b, kb * BK, tl.g * p.N + tl.n0, &full_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { s_abort = 1; atomicExch(p.error, 1); }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      const uint32_t idesc = umma_idesc(BM, BN, 1 /*bf16*/);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      int i = 0;
      for (int t = blockIdx.x; ok; t += gridDim.x, i++) {
        const Tile tl = tile_of(p, t, s_rows, s_start);
        if (!tl.valid) break;
        const int b = i & 1;
        if (!mbar_wait(&tempty_bar[b], (((uint32_t)i >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)b * BN;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint8_t* sa = tiles + (size_t)stage * STAGE_BYTES;
          const uint64_t adesc = umma_desc_sw128(sa);
          const uint64_t bdesc = umma_desc_sw128(sa + A_TILE_BYTES);
          #pragma unroll
          for (int kk = 0; kk < BK / 16; kk++)
            umma_bf16(d_tmem, adesc + 2u * kk, bdesc + 2u * kk, idesc, (uint32_t)((kb | kk) != 0));
          umma_commit(&empty_bar[stage]);   // frees the stage when these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tfull_bar[b]);  // accumulator complete
      }
      if (!ok) { s_abort = 1; atomicExch(p.error, 2); }
    }
  } else {
    // ---------------- epilogue: warps 2..5, TMEM lane quarter = warp % 4 ----------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    __nv_bfloat16* C = static_cast<__nv_bfloat16*>(p.C);
    bool ok = true;
    int i = 0;
    for (int t = blockIdx.x; ok; t += gridDim.x, i++) {
      const Tile tl = tile_of(p, t, s_rows, s_start);
      if (!tl.valid) break;
      const int b = i & 1;
      if (!mbar_wait(&tfull_bar[b], ((uint32_t)i >> 1) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)b * BN;
      const bool live = row < tl.rows_left;
      __nv_bfloat16* crow = C + (size_t)(tl.m0 + row) * p.ldc;
      #pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c, r);
        tmem_ld_wait();
        if (p.epilogue == 1) {
          uint32_t o[8];
          #pragma unroll
          for (int j = 0; j < 8; j++) {
            float g0 = __uint_as_float(r[4 * j]), u0 = __uint_as_float(r[4 * j + 1]);
            float g1 = __uint_as_float(r[4 * j + 2]), u1 = __uint_as_float(r[4 * j + 3]);
            __nv_bfloat162 v = __floats2bfloat162_rn(silu(g0) * u0, silu(g1) * u1);
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
      if (lane == 0) mbar_arrive(&tempty_bar[b]);
    }
    if (!ok && lane == 0) { s_abort = 1; atomicExch(p.error, 3); }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------- host side ----------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

// [rows, K] bf16 row-major, box = box_rows x 64 elements, 128-byte swizzle
bool make_map(CUtensorMap* m, const void* base, unsigned long long rows, unsigned long long K, unsigned box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace
}  // namespace rbv

extern "C" int rbv_grouped_gemm_bf16_gated(const void* A, long long a_rows, const void* B, void* C,
                                           const int* group_start, const int* group_rows, int G, int N, int K, int ldc,
                                           int epilogue, int* error_flag, int max_ctas, void* cuda_stream,
                                           const unsigned long long* ready, const unsigned long long* ready_target,
                                           double timeout_ms);

extern "C" int rbv_grouped_gemm_bf16(const void* A, long long a_rows, const void* B, void* C, const int* group_start,
                                     const int* group_rows, int G, int N, int K, int ldc, int epilogue,
                                     int* error_flag, int max_ctas, void* cuda_stream) {
  return rbv_grouped_gemm_bf16_gated(A, a_rows, B, C, group_start, group_rows, G, N, K, ldc, epilogue, error_flag,
                                     max_ctas, cuda_stream, nullptr, nullptr, 0.0);
}

extern "C" int rbv_grouped_gemm_bf16_gated(const void* A, long long a_rows, const void* B, void* C,
                                           const int* group_start, const int* group_rows, int G, int N, int K, int ldc,
                                           int epilogue, int* error_flag, int max_ctas, void* cuda_stream,
                                           const unsigned long long* ready, const unsigned long long* ready_target,
                                           double timeout_ms) {
  using namespace rbv;
  // Without a gate the CTA-pair kernel (grouped_gemm_pair_sm100.cu) is the default; the gated start stays on this one.
  if (!ready && rbv_grouped_gemm_pair_enabled())
    return rbv_grouped_gemm_bf16_pair(A, a_rows, B, C, group_start, group_rows, G, N, K, ldc, epilogue, error_flag,
                                      max_ctas, cuda_stream);
  if (G < 1 || G > kMoeMaxGroups || N % BN || K % BK || a_rows < 1 || (ldc % 8)) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)GEMM_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap ma, mb;
  if (!make_map(&ma, A, (unsigned long long)a_rows, (unsigned long long)K, BM)) return (int)cudaErrorUnknown;
  if (!make_map(&mb, B, (unsigned long long)G * N, (unsigned long long)K, BN)) return (int)cudaErrorUnknown;
  GemmParams p;
  p.group_start = group_start; p.group_rows = group_rows; p.G = G; p.N = N; p.K = K; p.ldc = ldc; p.C = C;
  p.error = error_flag; p.epilogue = epilogue;
  p.ready = ready; p.ready_target = ready ? ready_target : nullptr;
  p.timeout_ns = (unsigned long long)((timeout_ms > 0 ? timeout_ms : 2000.0) * 1e6);
  int grid = max_ctas;
  if (grid <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&grid, cudaDevAttrMultiProcessorCount, dev);
  }
  grouped_gemm_kernel<<<grid, GEMM_THREADS, GEMM_SMEM, static_cast<cudaStream_t>(cuda_stream)>>>(ma, mb, p);
  return (int)cudaGetLastError();
}
