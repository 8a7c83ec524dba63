// MoE expert-parallel kernels around the grouped GEMM: router, layout, dispatch (permute fused with the
// all-to-all: every routed row is stored straight into its expert-sorted position on the owner GPU over
// NVLink) and combine (the return all-to-all fused with the gate-weighted sum: rows are pulled from the
// owners' output buffers).  The reference has no counterpart; the cross-GPU synchronisation follows the
// same rules as the alltoallv kernel (monotonic counters, bounded waits, no reset between calls).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "api/ctx_internal.h"
#include "kernels/mx_quant.cuh"
#include "kernels/primitives.cuh"
#include "rbv/device_types.h"
#include "rbv/moe.h"

namespace rbv {
namespace {

constexpr int kMoeThreads = 512;

// ---------------------------------------------------------------------------------------------
// Router: one warp per token.
// ---------------------------------------------------------------------------------------------
__global__ void moe_route_kernel(const float* __restrict__ logits, int T, int E, int* __restrict__ topk_idx,
                                 float* __restrict__ topk_w, int* __restrict__ hist) {
  __shared__ int s_hist[kMoeMaxExperts];
  for (int i = threadIdx.x; i < E; i += blockDim.x) s_hist[i] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    const float* row = logits + (size_t)t * E;
    float v[kMoeMaxExperts / 32];
    float mx = -INFINITY;
    #pragma unroll
    for (int j = 0; j < kMoeMaxExperts / 32; j++) {
      int e = j * 32 + lane;
      v[j] = e < E ? row[e] : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
    #pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    // top-2 by (value, lower index wins ties)
    float best[2]; int bi[2];
    #pragma unroll
    for (int k = 0; k < 2; k++) {
      float bv = -INFINITY; int be = 0x7fffffff;
      #pragma unroll
      for (int j = 0; j < kMoeMaxExperts / 32; j++) {
        int e = j * 32 + lane;
        bool taken = (k == 1 && e == bi[0]);
        if (e < E && !taken && (v[j] > bv || (v[j] == bv && e < be))) { bv = v[j]; be = e; }
      }
      #pragma unroll
      for (int o = 16; o; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
      }
      best[k] = bv; bi[k] = be;
    }
    // softmax probabilities of the two winners, renormalised: p_k / (p_0 + p_1)
    const float p0 = __expf(best[0] - mx), p1 = __expf(best[1] - mx);
    const float inv = 1.0f / (p0 + p1);
    if (lane == 0) {
      topk_idx[2 * t] = bi[0]; topk_idx[2 * t + 1] = bi[1];
      topk_w[2 * t] = p0 * inv; topk_w[2 * t + 1] = p1 * inv;
      atomicAdd(&s_hist[bi[0]], 1);
      atomicAdd(&s_hist[bi[1]], 1);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x)
    if (s_hist[i]) atomicAdd(&hist[i], s_hist[i]);
}

// ---------------------------------------------------------------------------------------------
// Layout: one CTA.  Receive buffer of a rank = its local experts in order; inside an expert the
// rows of source rank 0, then 1, ...
// ---------------------------------------------------------------------------------------------
// loc_off (optional): first index of this rank's rows for expert e in an expert-major ordering of its routed rows;
// ready_target (optional): running totals of rows each local expert has been promised over all calls so far.
// align: every expert's rows start at a multiple of `align` rows in the owner's buffer (1: packed).
__global__ void moe_layout_kernel(const int* __restrict__ hist_all, int P, int E, int me, int* dst_base,
                                  int* group_start, int* group_rows, int* cursor, int* totals, int* loc_off,
                                  unsigned long long* ready_target, int align) {
  __shared__ int s_tot[kMoeMaxExperts];      // rows of expert e over all sources
  __shared__ int s_before[kMoeMaxExperts];   // rows of expert e from sources < me
  const int El = E / P;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int s = 0; s < P; s++) {
      int c = hist_all[s * E + e];
      if (s < me) before += c;
      tot += c;
    }
    s_tot[e] = tot; s_before[e] = before;
    cursor[e] = 0;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int owner = e / El;
    int base = 0;
    for (int e2 = owner * El; e2 < e; e2++) base += (s_tot[e2] + align - 1) / align * align;
    dst_base[e] = base + s_before[e];
    if (owner == me) {
      group_start[e - owner * El] = base; group_rows[e - owner * El] = s_tot[e];
      if (ready_target) ready_target[e - owner * El] += (unsigned long long)s_tot[e];
    }
    if (loc_off) {
      int off = 0;
      for (int e2 = 0; e2 < e; e2++) off += hist_all[me * E + e2];
      loc_off[e] = off;
    }
  }
  if (threadIdx.x == 0) {
    int recv = 0, sent = 0;
    for (int e = me * El; e < (me + 1) * El; e++) recv += s_tot[e];
    for (int e = 0; e < E; e++) sent += hist_all[me * E + e];
    totals[0] = recv; totals[1] = sent;
  }
}

struct MoeComm {
  int nproc, proc;
  unsigned long long ctrl_off;
  unsigned long long timeout_ns;
  int* error;               // device flag: 0 ok, else (site << 8 | detail)
  unsigned long long* aux_self;   // arrival counters of the auxiliary barriers in the NVLS buffer (null: in the
  unsigned long long* aux_mc;     // control blocks); aux_mc is the multicast address that reaches every GPU's copy
  char* heap[kMaxProcs];
};

// This process has reached auxiliary barrier `slot`: one multimem.red through NVSwitch, or one relaxed reduction
// per process.  The caller has fenced.
__device__ __forceinline__ void aux_arrive(const MoeComm& c, int slot) {
  if (c.aux_mc) { dev::multimem_red_add(c.aux_mc + slot, 1ull); return; }
  for (int q = 0; q < c.nproc; q++)
    dev::red_relaxed_add(&reinterpret_cast<CtrlBlock*>(c.heap[q] + c.ctrl_off)->aux_arrivals[slot], 1ull, q != c.proc);
}
__device__ __forceinline__ const unsigned long long* aux_counter(const MoeComm& c, int slot) {
  return c.aux_mc ? c.aux_self + slot : &reinterpret_cast<CtrlBlock*>(c.heap[c.proc] + c.ctrl_off)->aux_arrivals[slot];
}

__device__ __forceinline__ CtrlBlock* ctrl_of(const MoeComm& c, int q) {
  return reinterpret_cast<CtrlBlock*>(c.heap[q] + c.ctrl_off);
}

__device__ void moe_fail(const MoeComm& c, int site, int detail) {
  atomicCAS(c.error, 0, (site << 8) | (detail & 0xff));
}

}  // namespace
}  // namespace rbv

namespace rbv {
namespace {

// ---------------------------------------------------------------------------------------------
// Dispatch: one warp per routed row.
// ---------------------------------------------------------------------------------------------
struct DispatchArgs {
  MoeComm comm;
  const char* x;            // [T, H] bf16
  int T, H, E, El;
  const int* topk_idx;      // [T, 2]
  const int* dst_base;      // [E]
  int* cursor;              // [E], zero on entry
  int* slot;                // [T, 2] out
  unsigned long long xrecv_off;
  long long capacity_rows;
  unsigned long long ret_off;   // != 0: heap offset of the owner's table of return addresses, one word per row:
                                // (sending process << 24) | (token * 2 + k), for GEMMs that push their result back
};

__global__ void __launch_bounds__(kMoeThreads) moe_dispatch_kernel(const __grid_constant__ DispatchArgs a) {
  const MoeComm& c = a.comm;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const size_t row_bytes = (size_t)a.H * 2;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < 2 * a.T; r += warps) {
    const int e = a.topk_idx[r];
    int pos = 0;
    if (lane == 0) pos = a.dst_base[e] + atomicAdd(&a.cursor[e], 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (lane == 0) a.slot[r] = pos;
    if (pos >= a.capacity_rows) { if (lane == 0) moe_fail(c, 4, e); continue; }
    const int owner = e / a.El;
    char* dst = c.heap[owner] + a.xrecv_off + (size_t)pos * row_bytes;
    if (a.ret_off && lane == 0)
      reinterpret_cast<unsigned*>(c.heap[owner] + a.ret_off)[pos] = ((unsigned)c.proc << 24) | (unsigned)r;
    dev::group_copy(dst, a.x + (size_t)(r >> 1) * row_bytes, row_bytes, lane, 32);
  }
  // completion: the last CTA tells every process that this rank's rows are in place, then waits for all ranks
  __syncthreads();
  if (threadIdx.x == 0) {
    CtrlBlock* my = ctrl_of(c, c.proc);
    dev::fence_acq_rel(c.nproc > 1);
    if (atomicAdd(&my->aux_exit[0], 1u) == gridDim.x - 1) {
      my->aux_exit[0] = 0;
      const unsigned seq = my->aux_seq[0];
      dev::fence_acq_rel(c.nproc > 1);   // one fence publishes every CTA's rows (each fenced before its exit count)
      aux_arrive(c, 0);
      dev::WaitCfg wc{&my->abort_flag, c.timeout_ns};
      const unsigned long long target = ((unsigned long long)seq + 1ull) * (unsigned long long)c.nproc;
      if (dev::wait_ge(aux_counter(c, 0), target, wc, c.nproc > 1) != dev::WAIT_OK) moe_fail(c, 1, 0);
      my->aux_seq[0] = seq + 1u;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Dispatch for the MXFP8 expert GEMMs: the row is quantised where it is read (e4m3, one power-of-two scale per 32
// columns, as rbv_quantize_rows_mxfp8 does) and travels as H bytes plus H / 128 scale words instead of 2 H bytes, so
// half as much crosses NVLink and the owner needs no quantiser pass.  Scale words land row-major
// ([capacity][H / 128], one coalesced store per row); moe_scale_atoms_kernel puts them into the GEMM's atom order.
// ---------------------------------------------------------------------------------------------
struct DispatchMxArgs {
  MoeComm comm;
  const char* x;            // [T, H] bf16
  int T, H, E, El;
  const int* topk_idx;
  const int* dst_base;
  int* cursor;
  int* slot;
  unsigned long long xq_off;      // heap offset of the owner's [capacity, H] e4m3 rows
  unsigned long long sfrow_off;   // heap offset of the owner's [capacity, H / 128] scale words
  unsigned long long ret_off;     // as in DispatchArgs
  long long capacity_rows;
};

__global__ void __launch_bounds__(kMoeThreads, 2) moe_dispatch_mx_kernel(const __grid_constant__ DispatchMxArgs a) {
  const MoeComm& c = a.comm;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int nkb = a.H / 128;                    // scale words per row (<= 32 handled per pass of the word exchange)
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < 2 * a.T; r += warps) {
    const int e = a.topk_idx[r];
    int pos = 0;
    if (lane == 0) pos = a.dst_base[e] + atomicAdd(&a.cursor[e], 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (lane == 0) a.slot[r] = pos;
    if (pos >= a.capacity_rows) { if (lane == 0) moe_fail(c, 4, e); continue; }
    const int owner = e / a.El;
    if (a.ret_off && lane == 0)
      reinterpret_cast<unsigned*>(c.heap[owner] + a.ret_off)[pos] = ((unsigned)c.proc << 24) | (unsigned)r;
    const uint4* src = reinterpret_cast<const uint4*>(a.x + (size_t)(r >> 1) * a.H * 2);
    uint2* dst = reinterpret_cast<uint2*>(c.heap[owner] + a.xq_off + (size_t)pos * a.H);
    unsigned* sfdst = reinterpret_cast<unsigned*>(c.heap[owner] + a.sfrow_off) + (size_t)pos * nkb;
    // 256 columns per pass: lane l holds columns 8 l .. 8 l + 7, a 32-column block is 4 lanes, a 128-column block
    // (one scale word) 16 lanes
    for (int base = 0; base < nkb; base += 32) {
      unsigned myword = 0;
      const int passes = min(16, (nkb - base + 1) / 2);
      // four loads (1024 columns) in flight per lane at a time, two CTAs per SM: a quarter of the trips to memory
      // that one load per 256 columns would take
      #pragma unroll 1
      for (int i0 = 0; i0 < passes; i0 += 4) {
      uint4 rawv[4];
      #pragma unroll
      for (int j = 0; j < 4; j++) {
        const int vec = (base / 2 + i0 + j) * 32 + lane;
        rawv[j] = make_uint4(0u, 0u, 0u, 0u);
        if (i0 + j < passes && vec * 8 < a.H) rawv[j] = __ldg(src + vec);
      }
      #pragma unroll
      for (int j = 0; j < 4; j++) {
        const int i = i0 + j;
        if (i >= passes) break;
        const int vec = (base / 2 + i) * 32 + lane;             // 16-byte vector of the row
        const bool in = vec * 8 < a.H;
        const uint4 raw = rawv[j];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float2 v[4];
        float m = 0.0f;
        #pragma unroll
        for (int j = 0; j < 4; j++) {
          v[j] = __bfloat1622float2(h[j]);
          m = fmaxf(m, fmaxf(fabsf(v[j].x), fabsf(v[j].y)));
        }
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        const int ex = mx_exponent(m);
        const float inv = mx_inv_scale(ex);
        unsigned word = (unsigned)(ex + 127) << (8 * ((lane & 15) >> 2));
        word |= __shfl_xor_sync(0xffffffffu, word, 4);
        word |= __shfl_xor_sync(0xffffffffu, word, 8);
        // word of K block base + 2 i sits in lanes 0-15, of base + 2 i + 1 in lanes 16-31; lane j keeps word j
        const unsigned w = __shfl_sync(0xffffffffu, word, (lane & 1) * 16);
        if ((lane >> 1) == i) myword = w;
        if (in) {
          unsigned q[4];
          #pragma unroll
          for (int j = 0; j < 4; j++)
            q[j] = __nv_cvt_float2_to_fp8x2(make_float2(v[j].x * inv, v[j].y * inv), __NV_SATFINITE, __NV_E4M3);
          dst[vec] = make_uint2(q[0] | (q[1] << 16), q[2] | (q[3] << 16));
        }
      }
      }
      if (base + lane < nkb) sfdst[base + lane] = myword;
    }
  }
  // completion: as moe_dispatch_kernel
  __syncthreads();
  if (threadIdx.x == 0) {
    CtrlBlock* my = ctrl_of(c, c.proc);
    dev::fence_acq_rel(c.nproc > 1);
    if (atomicAdd(&my->aux_exit[0], 1u) == gridDim.x - 1) {
      my->aux_exit[0] = 0;
      const unsigned seq = my->aux_seq[0];
      dev::fence_acq_rel(c.nproc > 1);
      aux_arrive(c, 0);
      dev::WaitCfg wc{&my->abort_flag, c.timeout_ns};
      const unsigned long long target = ((unsigned long long)seq + 1ull) * (unsigned long long)c.nproc;
      if (dev::wait_ge(aux_counter(c, 0), target, wc, c.nproc > 1) != dev::WAIT_OK) moe_fail(c, 1, 0);
      my->aux_seq[0] = seq + 1u;
    }
  }
}

// Scale words [rows][nkb] (row-major) -> the atom order of the MXFP8 GEMM, [nkb][ceil(rows / 128)][128].
__global__ void moe_scale_atoms_kernel(const unsigned* __restrict__ sfrow, unsigned* __restrict__ sfa, int rows, int nkb) {
  const long long n = (long long)rows * nkb;
  const int nrb = (rows + 127) / 128;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    // consecutive threads walk the rows of one K block: reads are strided by nkb words, writes fill whole atoms
    const int kb = (int)(i / rows), r = (int)(i - (long long)kb * rows);
    sfa[((size_t)kb * nrb + r / 128) * 128 + (r % 32) * 4 + (r % 128) / 32] = sfrow[(size_t)r * nkb + kb];
  }
}

// ---------------------------------------------------------------------------------------------
// Combine: cross-GPU barrier, then one warp per token pulls its two expert rows.
// ---------------------------------------------------------------------------------------------
struct CombineArgs {
  MoeComm comm;
  char* out;                // [T, H] bf16
  int T, H, E, El;
  const int* topk_idx;
  const float* topk_w;
  const int* slot;
  unsigned long long y_off;
};

__device__ __forceinline__ void bf16x8_fma(float (&acc)[8], const uint4& v, float w) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
  #pragma unroll
  for (int i = 0; i < 4; i++) {
    float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] = fmaf(w, f.x, acc[2 * i]);
    acc[2 * i + 1] = fmaf(w, f.y, acc[2 * i + 1]);
  }
}

__global__ void __launch_bounds__(kMoeThreads) moe_combine_kernel(const __grid_constant__ CombineArgs a) {
  const MoeComm& c = a.comm;
  __shared__ int s_ok;
  CtrlBlock* my = ctrl_of(c, c.proc);
  if (threadIdx.x == 0) {
    const unsigned seq = __ldcg(&my->aux_seq[1]);
    if (blockIdx.x == 0) {
      dev::fence_acq_rel(c.nproc > 1);
      aux_arrive(c, 1);
    }
    dev::WaitCfg wc{&my->abort_flag, c.timeout_ns};
    const unsigned long long target = ((unsigned long long)seq + 1ull) * (unsigned long long)c.nproc;
    int r = dev::wait_ge(aux_counter(c, 1), target, wc, c.nproc > 1);
    if (r != dev::WAIT_OK) moe_fail(c, 2, 0);
    s_ok = (r == dev::WAIT_OK);
  }
  __syncthreads();
  if (s_ok) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int nvec = a.H / 8;   // 16-byte vectors per row
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < a.T; t += warps) {
      const int e0 = a.topk_idx[2 * t], e1 = a.topk_idx[2 * t + 1];
      const float w0 = a.topk_w[2 * t], w1 = a.topk_w[2 * t + 1];
      const uint4* r0 = reinterpret_cast<const uint4*>(c.heap[e0 / a.El] + a.y_off + (size_t)a.slot[2 * t] * a.H * 2);
      const uint4* r1 = reinterpret_cast<const uint4*>(c.heap[e1 / a.El] + a.y_off + (size_t)a.slot[2 * t + 1] * a.H * 2);
      uint4* o = reinterpret_cast<uint4*>(a.out + (size_t)t * a.H * 2);
      for (int i = lane; i < nvec; i += 32) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        bf16x8_fma(acc, dev::ld_cg_v4(r0 + i), w0);
        bf16x8_fma(acc, dev::ld_cg_v4(r1 + i), w1);
        uint4 v;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
        #pragma unroll
        for (int j = 0; j < 4; j++) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        o[i] = v;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&my->aux_exit[1], 1u) == gridDim.x - 1) {
      my->aux_exit[1] = 0;
      my->aux_seq[1] = my->aux_seq[1] + 1u;
    }
  }
}

// Combine after a down GEMM that pushed every result row back to the GPU of its token (row (token, k) of a
// [T, 2, H] buffer there): a cross-GPU barrier says that every GEMM has finished, then the gate-weighted sum reads
// local memory only.
struct CombinePushedArgs {
  MoeComm comm;
  char* out;                // [T, H] bf16
  const char* y2;           // [T, 2, H] bf16, local
  int T, H;
  const float* topk_w;
};

__global__ void __launch_bounds__(kMoeThreads) moe_combine_pushed_kernel(const __grid_constant__ CombinePushedArgs a) {
  const MoeComm& c = a.comm;
  __shared__ int s_ok;
  CtrlBlock* my = ctrl_of(c, c.proc);
  if (threadIdx.x == 0) {
    const unsigned seq = __ldcg(&my->aux_seq[1]);
    if (blockIdx.x == 0) {
      dev::fence_acq_rel(c.nproc > 1);
      aux_arrive(c, 1);
    }
    dev::WaitCfg wc{&my->abort_flag, c.timeout_ns};
    const unsigned long long target = ((unsigned long long)seq + 1ull) * (unsigned long long)c.nproc;
    int r = dev::wait_ge(aux_counter(c, 1), target, wc, c.nproc > 1);
    if (r != dev::WAIT_OK) moe_fail(c, 2, 0);
    s_ok = (r == dev::WAIT_OK);
  }
  __syncthreads();
  if (s_ok) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int nvec = a.H / 8;
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < a.T; t += warps) {
      const float w0 = a.topk_w[2 * t], w1 = a.topk_w[2 * t + 1];
      const uint4* r0 = reinterpret_cast<const uint4*>(a.y2 + (size_t)(2 * t) * a.H * 2);
      const uint4* r1 = r0 + nvec;
      uint4* o = reinterpret_cast<uint4*>(a.out + (size_t)t * a.H * 2);
      for (int i = lane; i < nvec; i += 32) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        bf16x8_fma(acc, dev::ld_cg_v4(r0 + i), w0);   // the rows were written by other GPUs: not through L1
        bf16x8_fma(acc, dev::ld_cg_v4(r1 + i), w1);
        uint4 v;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
        #pragma unroll
        for (int j = 0; j < 4; j++) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        o[i] = v;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&my->aux_exit[1], 1u) == gridDim.x - 1) {
      my->aux_exit[1] = 0;
      my->aux_seq[1] = my->aux_seq[1] + 1u;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Streamed dispatch.  The routed rows are visited expert by expert (`order` lists them expert-major), every GPU
// therefore fills expert 0 of every owner first, then expert 1, ...; each landed row bumps a counter of its expert
// on the owner, and the grouped GEMM's loader starts an expert's tiles as soon as the counter says that all its
// rows are there (rbv_grouped_gemm_bf16_gated).  The first expert is complete after about one El-th of the
// dispatch, and the GEMM of an expert takes far longer than its dispatch, so all but the head of the dispatch
// disappears behind the GEMM.  No barrier at the end: nothing but the counters says when data is usable.
// ---------------------------------------------------------------------------------------------
__global__ void moe_order_kernel(const int* __restrict__ topk_idx, int n_rows, const int* __restrict__ loc_off,
                                 int* __restrict__ cursor, int* __restrict__ order) {
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += gridDim.x * blockDim.x) {
    const int e = topk_idx[r];
    order[loc_off[e] + atomicAdd(&cursor[e], 1)] = r;
  }
}

struct StreamedArgs {
  MoeComm comm;
  const char* x;
  int T, H, E, El;
  const int* topk_idx;
  const int* dst_base;
  const int* loc_off;
  const int* order;
  int* slot;
  unsigned long long xrecv_off, ready_off;
  long long capacity_rows;
};

__global__ void __launch_bounds__(kMoeThreads) moe_dispatch_streamed_kernel(const __grid_constant__ StreamedArgs a) {
  const MoeComm& c = a.comm;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const size_t row_bytes = (size_t)a.H * 2;
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < 2 * a.T; i += warps) {
    const int r = a.order[i];
    const int e = a.topk_idx[r];
    const int pos = a.dst_base[e] + (i - a.loc_off[e]);
    const int owner = e / a.El;
    if (lane == 0) a.slot[r] = pos;
    if (pos < a.capacity_rows)
      dev::group_copy(c.heap[owner] + a.xrecv_off + (size_t)pos * row_bytes, a.x + (size_t)(r >> 1) * row_bytes, row_bytes,
                      lane, 32);
    else if (lane == 0) moe_fail(c, 4, e);
    __syncwarp();
    // the row counts as landed once its stores are visible on the owner (a row that did not fit is counted too,
    // so that the consumer's target is met and the error flag, not a time-out, tells the story)
    if (lane == 0) {
      const bool far = owner != c.proc;
      dev::fence_acq_rel(far);
      dev::red_relaxed_add(reinterpret_cast<unsigned long long*>(c.heap[owner] + a.ready_off) + (e - owner * a.El), 1ull, far);
    }
  }
}

MoeComm make_comm(rbv_ctx_t ctx, int* error) {
  MoeComm m;
  const Context& c = *ctx->c;
  m.nproc = c.nproc(); m.proc = c.proc();
  m.ctrl_off = c.layout().ctrl_off;
  m.timeout_ns = c.timeout_ns();
  m.error = error;
  m.aux_self = c.nvls_aux_self();
  m.aux_mc = c.nvls_aux_mc();
  for (int q = 0; q < kMaxProcs; q++) m.heap[q] = q < c.nproc() ? c.peer_heap(q) : nullptr;
  return m;
}

}  // namespace
}  // namespace rbv

using namespace rbv;

extern "C" {

int rbv_moe_route(const float* logits, int T, int E, int* topk_idx, float* topk_w, int* hist, void* stream) {
  if (E < 2 || E > kMoeMaxExperts) return (int)cudaErrorInvalidValue;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(hist, 0, sizeof(int) * E, st);
  if (e != cudaSuccess) return (int)e;
  const int warps_per_cta = 8;
  int grid = (T + warps_per_cta - 1) / warps_per_cta;
  grid = grid < 1 ? 1 : (grid > 1184 ? 1184 : grid);
  moe_route_kernel<<<grid, warps_per_cta * 32, 0, st>>>(logits, T, E, topk_idx, topk_w, hist);
  return (int)cudaGetLastError();
}

int rbv_moe_layout_aligned(const int* hist_all, int P, int E, int me, int* dst_base, int* group_start,
                           int* group_rows, int* cursor, int* totals, int align, void* stream) {
  if (E > kMoeMaxExperts || E % P || align < 1) return (int)cudaErrorInvalidValue;
  moe_layout_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(hist_all, P, E, me, dst_base, group_start,
                                                                        group_rows, cursor, totals, nullptr, nullptr,
                                                                        align);
  return (int)cudaGetLastError();
}

int rbv_moe_layout(const int* hist_all, int P, int E, int me, int* dst_base, int* group_start, int* group_rows,
                   int* cursor, int* totals, void* stream) {
  return rbv_moe_layout_aligned(hist_all, P, E, me, dst_base, group_start, group_rows, cursor, totals, 1, stream);
}

int rbv_moe_layout_streamed(const int* hist_all, int P, int E, int me, int* dst_base, int* group_start,
                            int* group_rows, int* cursor, int* totals, int* loc_off, unsigned long long* ready_target,
                            const int* topk_idx, int T, int* order, void* stream) {
  if (E > kMoeMaxExperts || E % P) return (int)cudaErrorInvalidValue;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  moe_layout_kernel<<<1, 256, 0, st>>>(hist_all, P, E, me, dst_base, group_start, group_rows, cursor, totals, loc_off,
                                       ready_target, 1);
  int grid = (2 * T + 255) / 256;
  grid = grid < 1 ? 1 : (grid > 592 ? 592 : grid);
  moe_order_kernel<<<grid, 256, 0, st>>>(topk_idx, 2 * T, loc_off, cursor, order);
  return (int)cudaGetLastError();
}

}  // extern "C"

extern "C" {

int rbv_moe_dispatch(rbv_ctx_t ctx, const void* x, int T, int H, const int* topk_idx, const int* dst_base,
                     int* cursor, int* slot, unsigned long long xrecv_off, long long recv_capacity_rows,
                     int E, int* error_flag, void* stream) {
  return rbv_moe_dispatch_ret(ctx, x, T, H, topk_idx, dst_base, cursor, slot, xrecv_off, 0ull, recv_capacity_rows, E,
                              error_flag, stream);
}

int rbv_moe_dispatch_ret(rbv_ctx_t ctx, const void* x, int T, int H, const int* topk_idx, const int* dst_base,
                         int* cursor, int* slot, unsigned long long xrecv_off, unsigned long long ret_off,
                         long long recv_capacity_rows, int E, int* error_flag, void* stream) {
  const Context& c = *ctx->c;
  if (2ll * T >= (1ll << 24)) return (int)cudaErrorInvalidValue;
  if (c.L() != 1 || E % c.P() || (H % 8)) return (int)cudaErrorInvalidValue;
  DispatchArgs a;
  a.comm = make_comm(ctx, error_flag);
  a.x = static_cast<const char*>(x);
  a.T = T; a.H = H; a.E = E; a.El = E / c.P();
  a.topk_idx = topk_idx; a.dst_base = dst_base; a.cursor = cursor; a.slot = slot;
  a.xrecv_off = xrecv_off; a.capacity_rows = recv_capacity_rows; a.ret_off = ret_off;
  const int warps_per_cta = kMoeThreads / 32;
  int grid = (2 * T + warps_per_cta - 1) / warps_per_cta;
  const int cap = c.sm_count() * 2;
  grid = grid < 1 ? 1 : (grid > cap ? cap : grid);
  moe_dispatch_kernel<<<grid, kMoeThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}

int rbv_moe_dispatch_mx(rbv_ctx_t ctx, const void* x, int T, int H, const int* topk_idx, const int* dst_base,
                        int* cursor, int* slot, unsigned long long xq_off, unsigned long long sfrow_off,
                        unsigned long long ret_off, long long recv_capacity_rows, int E, int* error_flag,
                        void* stream) {
  const Context& c = *ctx->c;
  if (c.L() != 1 || E % c.P() || (H % 128) || 2ll * T >= (1ll << 24)) return (int)cudaErrorInvalidValue;
  DispatchMxArgs a;
  a.comm = make_comm(ctx, error_flag);
  a.x = static_cast<const char*>(x);
  a.T = T; a.H = H; a.E = E; a.El = E / c.P();
  a.topk_idx = topk_idx; a.dst_base = dst_base; a.cursor = cursor; a.slot = slot;
  a.xq_off = xq_off; a.sfrow_off = sfrow_off; a.ret_off = ret_off; a.capacity_rows = recv_capacity_rows;
  const int warps_per_cta = kMoeThreads / 32;
  int grid = (2 * T + warps_per_cta - 1) / warps_per_cta;
  const int cap = c.sm_count() * 2;
  grid = grid < 1 ? 1 : (grid > cap ? cap : grid);
  moe_dispatch_mx_kernel<<<grid, kMoeThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}

int rbv_moe_scale_atoms(const void* sfrow, void* sfa, int rows, int nkb, void* stream) {
  if (rows < 1 || nkb < 1) return (int)cudaErrorInvalidValue;
  long long n = (long long)rows * nkb;
  int grid = (int)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
  moe_scale_atoms_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned*>(sfrow), static_cast<unsigned*>(sfa), rows, nkb);
  return (int)cudaGetLastError();
}

int rbv_moe_dispatch_streamed(rbv_ctx_t ctx, const void* x, int T, int H, const int* topk_idx, const int* dst_base,
                              const int* loc_off, const int* order, int* slot, unsigned long long xrecv_off,
                              unsigned long long ready_off, long long recv_capacity_rows, int E, int* error_flag,
                              void* stream) {
  const Context& c = *ctx->c;
  if (c.L() != 1 || E % c.P() || (H % 8)) return (int)cudaErrorInvalidValue;
  StreamedArgs a;
  a.comm = make_comm(ctx, error_flag);
  a.x = static_cast<const char*>(x);
  a.T = T; a.H = H; a.E = E; a.El = E / c.P();
  a.topk_idx = topk_idx; a.dst_base = dst_base; a.loc_off = loc_off; a.order = order; a.slot = slot;
  a.xrecv_off = xrecv_off; a.ready_off = ready_off; a.capacity_rows = recv_capacity_rows;
  // One CTA per SM: the grouped GEMM that consumes the rows runs at the same time and needs its share of every SM.
  // That kernel configures its SMs for the largest shared memory; an SM takes CTAs of two kernels only under one
  // configuration, so this kernel asks for the same one although it uses no shared memory itself.
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(moe_dispatch_streamed_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  const int warps_per_cta = kMoeThreads / 32;
  int grid = (2 * T + warps_per_cta - 1) / warps_per_cta;
  grid = grid < 1 ? 1 : (grid > c.sm_count() ? c.sm_count() : grid);
  moe_dispatch_streamed_kernel<<<grid, kMoeThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}

int rbv_moe_combine(rbv_ctx_t ctx, void* out, int T, int H, const int* topk_idx, const float* topk_w,
                    const int* slot, unsigned long long y_off, int E, int* error_flag, void* stream) {
  const Context& c = *ctx->c;
  if (c.L() != 1 || E % c.P() || (H % 8)) return (int)cudaErrorInvalidValue;
  CombineArgs a;
  a.comm = make_comm(ctx, error_flag);
  a.out = static_cast<char*>(out);
  a.T = T; a.H = H; a.E = E; a.El = E / c.P();
  a.topk_idx = topk_idx; a.topk_w = topk_w; a.slot = slot; a.y_off = y_off;
  const int warps_per_cta = kMoeThreads / 32;
  int grid = (T + warps_per_cta - 1) / warps_per_cta;
  // every CTA waits on the barrier, so all of them must be able to run without waiting for each other:
  // only CTA 0 signals and the signal does not depend on any other CTA, which keeps any grid size safe
  const int cap = c.sm_count() * 2;
  grid = grid < 1 ? 1 : (grid > cap ? cap : grid);
  moe_combine_kernel<<<grid, kMoeThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}

int rbv_moe_combine_pushed(rbv_ctx_t ctx, void* out, int T, int H, const float* topk_w, const void* y2,
                           int* error_flag, void* stream) {
  const Context& c = *ctx->c;
  if (c.L() != 1 || (H % 8)) return (int)cudaErrorInvalidValue;
  CombinePushedArgs a;
  a.comm = make_comm(ctx, error_flag);
  a.out = static_cast<char*>(out);
  a.y2 = static_cast<const char*>(y2);
  a.T = T; a.H = H; a.topk_w = topk_w;
  const int warps_per_cta = kMoeThreads / 32;
  int grid = (T + warps_per_cta - 1) / warps_per_cta;
  const int cap = c.sm_count() * 2;   // every CTA waits on the barrier and only CTA 0 signals: any grid size is safe
  grid = grid < 1 ? 1 : (grid > cap ? cap : grid);
  moe_combine_pushed_kernel<<<grid, kMoeThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}

}  // extern "C"
