// Grouped GEMM for the expert FFN on CTA PAIRS (tcgen05 cta_group::2): two CTAs on neighbouring SMs share one
// 256 x 256 output tile.  Each CTA fetches its own 128 rows of A and its own half (128 of 256 rows) of the B tile, so a
// k-block costs 32 KB of shared-memory fill per SM instead of the 48 KB of the one-CTA kernel
// (grouped_gemm_sm100.cu) for the same number of MMAs: a third less traffic between L2 and the SMs, and a pipeline of
// 6 stages instead of 4 in the same shared memory.  No counterpart exists in the reference (it has no compute kernels).
//
//   C[rows of group g] = epilogue( A[rows of group g] (M_g x K, K-major) * B_g^T (N x K, K-major) )
//
// One persistent cluster of two CTAs per SM pair walks a static tile schedule (groups in order, n-major, m fastest):
//   warp 0    TMA producer, in both CTAs (own A rows, own half of B; bytes counted on a barrier of the rank-0 CTA)
//   warp 1    TMEM allocation in both CTAs; in the rank-0 CTA one elected thread issues the M256 N256 K16 MMAs
//   warps 2-5 epilogue, in both CTAs (each drains the 128 accumulator rows in its own TMEM)
// TMEM holds two 128 x 256 fp32 accumulators per CTA, so the epilogue of tile i overlaps the MMAs of tile i + 1.
// TMA loads carry no cluster multicast.  All waits are bounded; on expiry both CTAs are told, record an error,
// release their TMEM and return.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>

#include "kernels/sm100_ptx.cuh"
#include "rbv/moe.h"

namespace rbv {

using namespace sm100;

namespace {

constexpr int PM = 256;            // tile rows per pair
constexpr int HM = 128;            // rows per CTA
constexpr int PN = 256;            // tile columns
constexpr int HN = 128;            // rows of the B tile each CTA fetches
constexpr int PK = 64;             // one 128-byte swizzle atom of bf16
constexpr int PSTAGES = 6;
constexpr int PA_BYTES = HM * PK * 2;   // 16 KB
constexpr int PB_BYTES = HN * PK * 2;   // 16 KB
constexpr int PSTAGE_BYTES = PA_BYTES + PB_BYTES;
constexpr int PAIR_THREADS = 192;
constexpr int PAIR_TMEM_COLS = 512;
constexpr size_t PAIR_SMEM = (size_t)PSTAGES * PSTAGE_BYTES + 1024 /*alignment slack*/;

struct PairParams {
  const int* group_start;
  const int* group_rows;
  int G;
  int N, K;
  int ldc;
  void* C;
  int* error;
  int epilogue;   // 0: C = bf16(acc); 1: C[:, j] = bf16(silu(acc[:, 2j]) * acc[:, 2j+1])
  // Push mode (ret != null, epilogue 0): row `pos` of the result goes to row (ret[pos] & 0xffffff) of the [*, N] bf16
  // buffer at offset y2_off of the heap of process ret[pos] >> 24 (a peer mapping over NVLink when that is another
  // GPU): the return all-to-all of the MoE layer, done by the epilogue.
  const unsigned* ret;
  unsigned long long y2_off;
  char* heap[16];
};

struct PairTile { int m0, n0, b_row, rows; bool valid; };

// Tile t of the pair schedule: groups in order; inside a group n-major, m fastest.  `rows` = rows of the group from m0 on.
__device__ __forceinline__ PairTile pair_tile_of(const PairParams& p, int t, const int* s_rows, const int* s_start) {
  const int ntn = p.N / PN;
  PairTile r; r.valid = false; r.m0 = 0; r.n0 = 0; r.b_row = 0; r.rows = 0;
  for (int g = 0; g < p.G; g++) {
    const int ntm = (s_rows[g] + PM - 1) / PM;
    const int cnt = ntm * ntn;
    if (t < cnt) {
      const int n = t / ntm, m = t - n * ntm;
      r.m0 = s_start[g] + m * PM; r.n0 = n * PN; r.b_row = g * p.N + n * PN; r.rows = s_rows[g] - m * PM;
      r.valid = true;
      return r;
    }
    t -= cnt;
  }
  return r;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

}  // namespace

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                         const PairParams p) {
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[PSTAGES];    // used in the rank-0 CTA: bytes of both CTAs' loads
  __shared__ __align__(8) uint64_t empty_bar[PSTAGES];   // in each CTA: its stage has been read by the MMAs
  __shared__ __align__(8) uint64_t tfull_bar[2];         // in each CTA: accumulator b is complete
  __shared__ __align__(8) uint64_t tempty_bar[2];        // used in the rank-0 CTA: both CTAs have drained accumulator b
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_rows[kMoeMaxGroups], s_start[kMoeMaxGroups];
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (tid == 0) {
    for (int s = 0; s < PSTAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 8); }
    s_abort = 0;
    mbar_fence_init();
  }
  for (int i = tid; i < p.G; i += blockDim.x) { s_rows[i] = p.group_rows[i]; s_start[i] = p.group_start[i]; }
  if (warp == 1) { tmem_alloc_pair(&tmem_base_s, PAIR_TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // barriers of both CTAs are initialised before anything is signalled across
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  const int num_kb = p.K / PK;
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
        const PairTile tl = pair_tile_of(p, t, s_rows, s_start);
        if (!tl.valid) break;
        const int a_row = tl.m0 + (int)rank * HM;
        const int b_row = tl.b_row + (int)rank * HN;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = tiles + (size_t)stage * PSTAGE_BYTES;
          uint8_t* sb = sa + PA_BYTES;
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * PSTAGE_BYTES);
          const uint32_t bar0 = mapa_u32(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(sa, &tma_a, kb * PK, a_row, bar0);
          tma_load_2d_pair(sb, &tma_b, kb * PK, b_row, bar0);
          if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { s_abort = 1; st_cluster_u32(peer_abort, 1); atomicExch(p.error, 1); }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (rank-0 CTA only) ----------------
    if (leader && elect_one()) {
      const uint32_t idesc = umma_idesc(PM, PN, 1 /*bf16*/);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      int i = 0;
      for (int t = pair; ok; t += npairs, i++) {
        const PairTile tl = pair_tile_of(p, t, s_rows, s_start);
        if (!tl.valid) break;
        const int b = i & 1;
        if (!mbar_wait(&tempty_bar[b], (((uint32_t)i >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)b * PN;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint8_t* sa = tiles + (size_t)stage * PSTAGE_BYTES;
          const uint64_t adesc = umma_desc_sw128(sa);
          const uint64_t bdesc = umma_desc_sw128(sa + PA_BYTES);
          #pragma unroll
          for (int kk = 0; kk < PK / 16; kk++)
            umma_bf16_pair(d_tmem, adesc + 2u * kk, bdesc + 2u * kk, idesc, (uint32_t)((kb | kk) != 0));
          umma_commit_pair(&empty_bar[stage]);   // frees this stage in both CTAs
          if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(&tfull_bar[b]);   // accumulator complete, both CTAs
      }
      if (!ok) { s_abort = 1; st_cluster_u32(peer_abort, 1); atomicExch(p.error, 2); }
    }
  } else {
    // ---------------- epilogue (both CTAs): warps 2..5, TMEM lane quarter = warp % 4 ----------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    __nv_bfloat16* C = static_cast<__nv_bfloat16*>(p.C);
    bool ok = true;
    int i = 0;
    for (int t = pair; ok; t += npairs, i++) {
      const PairTile tl = pair_tile_of(p, t, s_rows, s_start);
      if (!tl.valid) break;
      const int b = i & 1;
      if (!mbar_wait(&tfull_bar[b], ((uint32_t)i >> 1) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)b * PN;
      const bool live = row < tl.rows - (int)rank * HM;
      __nv_bfloat16* crow = C + (size_t)(tl.m0 + (int)rank * HM + row) * p.ldc;
      if (p.ret && live) {
        const unsigned rv = __ldg(p.ret + tl.m0 + (int)rank * HM + row);
        crow = reinterpret_cast<__nv_bfloat16*>(p.heap[rv >> 24] + p.y2_off) + (size_t)(rv & 0xffffffu) * p.ldc;
      }
      #pragma unroll 1
      for (int c = 0; c < PN; c += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c, r);
        tmem_ld_wait();
        if (p.epilogue == 1) {
          uint32_t o[8];
          #pragma unroll
          for (int j = 0; j < 8; j++) {
            float g0 = __uint_as_float(r[4 * j]), u0 = __uint_as_float(r[4 * j + 1]);
            float g1 = __uint_as_float(r[4 * j + 2]), u1 = __uint_as_float(r[4 * j + 3]);
            __nv_bfloat162 v = __floats2bfloat162_rn(silu_f(g0) * u0, silu_f(g1) * u1);
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
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty_bar[b]), 0));   // 4 warps x 2 CTAs
    }
    if (!ok && lane == 0) { s_abort = 1; st_cluster_u32(peer_abort, 1); atomicExch(p.error, 3); }
  }

  // ---------------- teardown: nobody leaves while the other CTA may still signal it ----------------
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, PAIR_TMEM_COLS);
  }
}

// ---------------- host side ----------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn pair_encode_fn() {
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

// [rows, K] bf16 row-major, box = 128 rows x 64 elements, 128-byte swizzle
bool pair_make_map(CUtensorMap* m, const void* base, unsigned long long rows, unsigned long long K) {
  EncodeTiledFn fn = pair_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K * 2};
  cuuint32_t box[2] = {(cuuint32_t)PK, (cuuint32_t)HM};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int g_pair_mode = -1;   // -1: not decided yet (environment), 0: one-CTA kernel, 1: CTA pairs

}  // namespace
}  // namespace rbv

extern "C" void rbv_grouped_gemm_set_pair(int on) { rbv::g_pair_mode = on ? 1 : 0; }

extern "C" int rbv_grouped_gemm_pair_enabled() {
  if (rbv::g_pair_mode < 0) {
    const char* e = std::getenv("RBV_GEMM_PAIR");
    rbv::g_pair_mode = (e && e[0] == '0') ? 0 : 1;
  }
  return rbv::g_pair_mode;
}

static int launch_bf16_pair(const void* A, long long a_rows, const void* B, void* C, const int* group_start,
                            const int* group_rows, int G, int N, int K, int ldc, int epilogue, int* error_flag,
                            int max_ctas, void* cuda_stream, const unsigned* ret, const void* const* heaps, int nheaps,
                            unsigned long long y2_off) {
  using namespace rbv;
  if (G < 1 || G > kMoeMaxGroups || N % PN || K % PK || a_rows < 1 || (ldc % 8)) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return (int)cudaErrorInvalidValue;
  if (ret && (epilogue != 0 || !heaps || nheaps < 1 || nheaps > 16 || (y2_off & 15))) return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)PAIR_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap ma, mb;
  if (!pair_make_map(&ma, A, (unsigned long long)a_rows, (unsigned long long)K)) return (int)cudaErrorUnknown;
  if (!pair_make_map(&mb, B, (unsigned long long)G * N, (unsigned long long)K)) return (int)cudaErrorUnknown;
  PairParams p;
  p.group_start = group_start; p.group_rows = group_rows; p.G = G; p.N = N; p.K = K; p.ldc = ldc; p.C = C;
  p.error = error_flag; p.epilogue = epilogue;
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
  grouped_gemm_pair_kernel<<<grid, PAIR_THREADS, PAIR_SMEM, static_cast<cudaStream_t>(cuda_stream)>>>(ma, mb, p);
  return (int)cudaGetLastError();
}

extern "C" int rbv_grouped_gemm_bf16_pair(const void* A, long long a_rows, const void* B, void* C,
                                          const int* group_start, const int* group_rows, int G, int N, int K, int ldc,
                                          int epilogue, int* error_flag, int max_ctas, void* cuda_stream) {
  return launch_bf16_pair(A, a_rows, B, C, group_start, group_rows, G, N, K, ldc, epilogue, error_flag, max_ctas,
                          cuda_stream, nullptr, nullptr, 0, 0ull);
}

extern "C" int rbv_grouped_gemm_bf16_push(const void* A, long long a_rows, const void* B, const int* group_start,
                                          const int* group_rows, int G, int N, int K, const unsigned* ret,
                                          const void* const* heaps, int nheaps, unsigned long long y2_off,
                                          int* error_flag, int max_ctas, void* cuda_stream) {
  if (!ret) return (int)cudaErrorInvalidValue;
  // C is only a base for rows that are not pushed (there are none): any aligned address of this process will do
  return launch_bf16_pair(A, a_rows, B, const_cast<void*>(heaps ? heaps[0] : nullptr), group_start, group_rows, G, N, K,
                          N, 0, error_flag, max_ctas, cuda_stream, ret, heaps, nheaps, y2_off);
}
