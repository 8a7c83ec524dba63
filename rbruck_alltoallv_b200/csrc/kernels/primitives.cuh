// Device primitives: system-scope signal / bounded wait, CTA-wide byte copy for arbitrary alignment.
//
// Every wait is bounded by a %globaltimer deadline and also leaves when the context's abort flag
// is raised; it never traps.  On expiry the caller records a status and the kernel runs to its
// normal end, so the CUDA context stays usable.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "rbv/device_types.h"

namespace rbv {
namespace dev {

__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_relaxed_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(unsigned* p, unsigned v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Result of a bounded wait.
enum WaitResult : int { WAIT_OK = 0, WAIT_TIMEOUT = 1, WAIT_ABORTED = 2 };

struct WaitCfg {
  const unsigned* abort_flag;        // local
  unsigned long long timeout_ns;
};

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_acquire_gpu(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
template <typename T>
__device__ __forceinline__ T ld_acquire(const T* p, bool sys) {
  return sys ? ld_acquire_sys(p) : ld_acquire_gpu(p);
}

// `sys` = the value may be written by another GPU (system-scope acquire); otherwise gpu scope.
template <typename T>
__device__ __forceinline__ WaitResult wait_ge(const T* p, T target, const WaitCfg& cfg, bool sys = true) {
  if (ld_acquire(p, sys) >= target) return WAIT_OK;
  unsigned long long t0 = globaltimer();
  unsigned it = 0;
  for (;;) {
    if (ld_acquire(p, sys) >= target) return WAIT_OK;
    if ((++it & 31u) == 0) {
      if (ld_relaxed_sys(cfg.abort_flag)) return WAIT_ABORTED;
      if (globaltimer() - t0 > cfg.timeout_ns) return WAIT_TIMEOUT;
      __nanosleep(32);
    }
  }
}

// ---- CTA-wide copy ---------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_cg_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_v4(uint4* p, const uint4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ unsigned char ld_cg_u8(const unsigned char* p) {
  unsigned v;
  asm volatile("ld.global.cg.u8 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return (unsigned char)v;
}

template <int WO>
__device__ __forceinline__ uint4 shift_words(const uint4& a, const uint4& b, unsigned bits) {
  // the 16 bytes that start WO words + bits/8 bytes into the 32-byte pair (a, b)
  const unsigned w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  uint4 o;
  o.x = __funnelshift_r(w[WO + 0], w[WO + 1], bits);
  o.y = __funnelshift_r(w[WO + 1], w[WO + 2], bits);
  o.z = __funnelshift_r(w[WO + 2], w[WO + 3], bits);
  o.w = __funnelshift_r(w[WO + 3], w[WO + 4], bits);
  return o;
}

// Source and destination differ in their phase inside a 16-byte vector: output vector i is cut out of the
// aligned source vectors i and i + 1.  Vector i + 1 is what the next lane loads as its own vector i, so it comes
// by shuffle; only the last lane of a warp (and the lane that holds the last vector) loads it.  That keeps the
// traffic from L2 at one vector per vector written.  All lanes of a warp must call this together, with
// consecutive `tid` in consecutive lanes and `nt` a multiple of 32.
template <int WO>
__device__ __forceinline__ void copy_shifted(uint4* d, const uint4* s, size_t nvec, unsigned bits,
                                             unsigned tid, unsigned nt) {
  constexpr int U = 4;
  const bool last_lane = (tid & 31u) == 31u;
  for (size_t base = 0; base < nvec; base += (size_t)U * nt) {   // same trip count for every lane
    uint4 a[U], b[U];
    #pragma unroll
    for (int j = 0; j < U; j++) {
      const size_t i = base + (size_t)j * nt + tid;
      a[j] = make_uint4(0u, 0u, 0u, 0u);
      b[j] = a[j];
      if (i < nvec) {
        a[j] = ld_cg_v4(s + i);
        if (last_lane || i + 1 >= nvec) b[j] = ld_cg_v4(s + i + 1);
      }
    }
    #pragma unroll
    for (int j = 0; j < U; j++) {
      const size_t i = base + (size_t)j * nt + tid;
      uint4 n;
      n.x = __shfl_down_sync(0xffffffffu, a[j].x, 1);
      n.y = __shfl_down_sync(0xffffffffu, a[j].y, 1);
      n.z = __shfl_down_sync(0xffffffffu, a[j].z, 1);
      n.w = __shfl_down_sync(0xffffffffu, a[j].w, 1);
      if (!(last_lane || i + 1 >= nvec)) b[j] = n;
      if (i < nvec) st_v4(d + i, shift_words<WO>(a[j], b[j], bits));
    }
  }
}

// Copies n bytes with a group of nt threads (tid = index in the group: a warp or a whole CTA).
// dst and src may have any alignment, relative to each other too: stores are 16-byte aligned
// vectors, loads are aligned vectors re-assembled with funnel shifts when the two phases differ.
// Loads bypass L1 (the source may have been written by another GPU).  The caller synchronises.
__device__ __forceinline__ void group_copy(char* dst, const char* src, size_t n, unsigned tid, unsigned nt) {
  if (n == 0) return;
  size_t head = (16 - ((uintptr_t)dst & 15)) & 15;
  if (head > n) head = n;
  if (tid < head) dst[tid] = (char)ld_cg_u8((const unsigned char*)src + tid);
  dst += head; src += head; n -= head;
  const size_t nvec = n >> 4;
  if (nvec) {
    uint4* d = reinterpret_cast<uint4*>(dst);
    const unsigned sh = (unsigned)((uintptr_t)src & 15);
    // Vectors in front of the first 128-byte line boundary of the destination go first, so that every store
    // instruction of the main loops covers whole lines.  A peer GPU receives a line that is written in two pieces
    // as two NVLink packets with one header each, which costs a fifth of the link when 512-byte warp stores start
    // in the middle of a line.
    size_t hv = ((128 - ((uintptr_t)dst & 127)) & 127) >> 4;
    if (hv > nvec || nvec < 64) hv = 0;
    if (sh == 0) {
      const uint4* s = reinterpret_cast<const uint4*>(src);
      if (tid < hv) st_v4(d + tid, ld_cg_v4(s + tid));
      size_t i = hv + tid;
      // 8 independent 16-byte loads in flight per thread (4 KB per warp) before the first store
      for (; i + 7 * (size_t)nt < nvec; i += 8 * (size_t)nt) {
        uint4 v[8];
        #pragma unroll
        for (int j = 0; j < 8; j++) v[j] = ld_cg_v4(s + i + j * (size_t)nt);
        #pragma unroll
        for (int j = 0; j < 8; j++) st_v4(d + i + j * (size_t)nt, v[j]);
      }
      for (; i + 3 * (size_t)nt < nvec; i += 4 * (size_t)nt) {
        uint4 v0 = ld_cg_v4(s + i), v1 = ld_cg_v4(s + i + nt);
        uint4 v2 = ld_cg_v4(s + i + 2 * nt), v3 = ld_cg_v4(s + i + 3 * nt);
        st_v4(d + i, v0); st_v4(d + i + nt, v1);
        st_v4(d + i + 2 * nt, v2); st_v4(d + i + 3 * nt, v3);
      }
      for (; i < nvec; i += nt) st_v4(d + i, ld_cg_v4(s + i));
    } else {
      const uint4* s = reinterpret_cast<const uint4*>(src - sh);
      const unsigned bits = (sh & 3u) * 8u;
      switch (sh >> 2) {
        case 0: if (hv) copy_shifted<0>(d, s, hv, bits, tid, nt); copy_shifted<0>(d + hv, s + hv, nvec - hv, bits, tid, nt); break;
        case 1: if (hv) copy_shifted<1>(d, s, hv, bits, tid, nt); copy_shifted<1>(d + hv, s + hv, nvec - hv, bits, tid, nt); break;
        case 2: if (hv) copy_shifted<2>(d, s, hv, bits, tid, nt); copy_shifted<2>(d + hv, s + hv, nvec - hv, bits, tid, nt); break;
        default: if (hv) copy_shifted<3>(d, s, hv, bits, tid, nt); copy_shifted<3>(d + hv, s + hv, nvec - hv, bits, tid, nt); break;
      }
    }
  }
  const size_t done = nvec << 4, tail = n - done;
  if (tid < tail) dst[done + tid] = (char)ld_cg_u8((const unsigned char*)src + done + tid);
}

__device__ __forceinline__ void cta_copy(char* dst, const char* src, size_t n) {
  group_copy(dst, src, n, threadIdx.x, blockDim.x);
}

// Index of the op that owns work item c: the largest i in [lo, n) with prefix[i] <= c (prefix is an exclusive scan
// over n ops in shared memory, prefix[n] > c).  A warp's first item can belong to any op, and walking there op by
// op costs a dependent shared-memory load per step (measured: 2 us for the warps that own the last of 900
// items); later items of the same warp continue from the previous answer.
__device__ __forceinline__ int find_op(const unsigned* prefix, int lo, int n, unsigned c) {
  int hi = n;                       // invariant: prefix[lo] <= c < prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= c) lo = mid; else hi = mid;
  }
  return lo;
}

// ---- scope-selectable signals: gpu scope when producer and consumer share the GPU ----------------
// A signal is a fence followed by a relaxed store or reduction by the same thread, which is a release pattern.
// Measured on B200 over NVLink: `red.release.sys` took about 9 us longer than `fence.acq_rel.sys` followed by
// `red.relaxed.sys` (30.7 -> 21.3 us for a 1 MB exchange between two GPUs), so the fused forms are not used.
__device__ __forceinline__ void red_relaxed_add(unsigned long long* p, unsigned long long v, bool sys) {
  if (sys) asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
  else asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// One reduction that NVSwitch applies to the copy of the counter on every GPU of the multicast group (NVLS).
__device__ __forceinline__ void multimem_red_add(unsigned long long* mc, unsigned long long v) {
  asm volatile("multimem.red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(mc), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed(unsigned* p, unsigned v, bool sys) {
  if (sys) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
  else asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel(bool sys) {
  if (sys) asm volatile("fence.acq_rel.sys;" ::: "memory");
  else asm volatile("fence.acq_rel.gpu;" ::: "memory");
}
__device__ __forceinline__ void signal_store(unsigned* p, unsigned v, bool sys) {
  fence_acq_rel(sys);
  st_relaxed(p, v, sys);
}
__device__ __forceinline__ void signal_add(unsigned long long* p, unsigned long long v, bool sys) {
  fence_acq_rel(sys);
  red_relaxed_add(p, v, sys);
}

// ---- call bookkeeping shared by the three alltoallv kernels ---------------------------------------------------
// The call number lives in device memory (kernel arguments of a repeated call stay constant).  Every CTA (or warp)
// reads it with an acquire load and then adds itself to CtrlBlock::start_count; whoever completes the count knows
// that all others have read the number and advances it for the next call.  Doing this when the kernel starts
// rather than when it ends takes an atomic round trip and the stores that follow it off the tail of every call.
__device__ __forceinline__ unsigned read_call_seq(const CtrlBlock* c) { return ld_acquire_gpu(&c->call_seq); }
__device__ __forceinline__ void advance_call_seq(CtrlBlock* c, unsigned seq) {
  c->start_count = 0;
  c->call_seq = seq + 1u;
}
// The same when the call number came from the host: true if memory agrees with it (it must, unless launches that
// the host did not count, such as graph replays, ran on this context).
__device__ __forceinline__ bool advance_call_seq_checked(CtrlBlock* c, unsigned seq) {
  const bool ok = __ldcg(&c->call_seq) == seq;
  advance_call_seq(c, seq);
  return ok;
}

// First failure of a call: kept in the control block (first one wins) and handed to the host at once, so that no
// end-of-kernel pass is needed to publish it.  The abort flag makes every other wait on this process leave, and the
// peers are told to stop waiting as well.  `heap` / `nproc` / `proc` / `ctrl_off` locate the peers' control blocks.
__device__ inline void note_failure(char* const* heap, int nproc, int proc, unsigned long long ctrl_off,
                                    StatusBlock* host, int code, int site, int d0, int d1) {
  CtrlBlock* c = reinterpret_cast<CtrlBlock*>(heap[proc] + ctrl_off);
  if (atomicCAS(&c->status.code, 0, code) == 0) {
    c->status.site = site;
    c->status.detail0 = d0;
    c->status.detail1 = d1;
    c->last_code = code;
  }
  __threadfence();
  if (host && *reinterpret_cast<volatile int*>(&host->code) == 0) {   // sticky on the host until it has been read
    host->site = site;
    host->detail0 = d0;
    host->detail1 = d1;
    __threadfence_system();
    *reinterpret_cast<volatile int*>(&host->code) = code;
  }
  if (code != RBV_ERR_ABORTED) {
    st_relaxed_sys(&c->abort_flag, 1u);
    for (int q = 0; q < nproc; q++)
      if (q != proc) st_relaxed_sys(&reinterpret_cast<CtrlBlock*>(heap[q] + ctrl_off)->abort_flag, 1u);
  }
}

// End of a traced call: the last CTA to get here copies the per-key stamps and the status block to the host and
// clears the stamps.  All threads of the CTA must call it; `s_last` is a shared-memory word.
__device__ inline void publish_trace(CtrlBlock* c, TraceBlock* tb, TraceBlock* host_trace, StatusBlock* host_status,
                                     int* s_last) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    *s_last = atomicAdd(&c->exit_count, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!*s_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < kMaxTraceKeys; i += blockDim.x) {
    if (host_trace) { host_trace->kstart[i] = __ldcg(&tb->kstart[i]); host_trace->kend[i] = __ldcg(&tb->kend[i]); }
    tb->kstart[i] = ~0ull;
    tb->kend[i] = 0ull;
  }
  if (threadIdx.x == 0) {
    c->exit_count = 0;
    if (host_status) {
      for (int i = 0; i < 8; i++) host_status->trace[i] = c->status.trace[i];
    }
  }
}

}  // namespace dev
}  // namespace rbv
