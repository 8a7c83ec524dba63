// Low-latency ("eager") protocol of the alltoallv kernel for small blocks.
//
// The rendezvous kernel (a2av_kernel.cu) needs two dependent trips over NVLink per hop: the receiver's
// displacement row must arrive before the sender can store, and every completion signal has to wait for the
// acknowledgements of the stores before it.  Here a block travels as a stream of self-validating 16-byte units
//     { payload word 0, flag, payload word 1, flag }        flag = call number + 1
// into a cell owned by the library on the destination rank: a unit is valid as soon as both flags show the
// current call number, so no separate signal and no metadata phase exist; the block's byte count travels in
// the cell's first unit (this is the reference's "metadata then data" two-phase exchange of every round,
// e.g. src/tuna2.cpp:160-185, folded into one stream).  The destination rank copies the payload from its
// arrival cell into recvbuf[rdispls[source]] itself, so only the owner ever writes a receive buffer and no
// "receiver ready" handshake is needed.  Relay hops of the Bruck schedules forward a cell unit by unit as it
// arrives.  Cells live in arenas of their own (never touched by the rendezvous protocol, zero when the context
// is created or reset) and alternate with the call parity, like staging cells do.
//
// Work items (one warp each, walked in list order): the plan's send ops, cut into chunks, followed by one unpack
// op per (local rank, source).  Block sizes of relay and unpack items are not known before the header arrives;
// they get as many chunk items as the cell (or the receiver's recvcount) allows and idle ones leave after
// reading the header.
#include <cuda_runtime.h>

#include "kernels/primitives.cuh"
#include "rbv/device_types.h"

namespace rbv {

namespace {

constexpr int kOpTileE = 1024;
constexpr unsigned kBadSize = 0xffffffffu;   // header value: the sender refused the block (too large for a cell)

__device__ __forceinline__ CtrlBlock* ctrl_of(const KernelArgs& a, int proc) {
  return reinterpret_cast<CtrlBlock*>(a.heap[proc] + a.lay.ctrl_off);
}
__device__ __forceinline__ size_t cell_stride(const KernelArgs& a) { return 16 + 2 * (size_t)a.eager_payload; }
__device__ __forceinline__ uint4* cell_of(const KernelArgs& a, int proc, int parity, int lr, int cell) {
  return reinterpret_cast<uint4*>(a.heap[proc] + a.lay.eager_off + (size_t)(lr * 2 + parity) * a.lay.arena_bytes +
                                  (size_t)cell * cell_stride(a));
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_unit(uint4* p, unsigned w0, unsigned w1, unsigned flag) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(w0), "r"(flag), "r"(w1), "r"(flag) : "memory");
}

struct EagerCtx {
  const unsigned* abort_flag;
  unsigned long long timeout_ns;
  unsigned flag;
};

// Polls one unit until both flags carry the current call number.  false on time-out / abort.
__device__ __forceinline__ bool poll_unit(const uint4* p, const EagerCtx& c, uint4& v) {
  v = ld_volatile_v4(p);
  if (v.y == c.flag && v.w == c.flag) return true;
  const unsigned long long t0 = dev::globaltimer();
  unsigned it = 0;
  for (;;) {
    v = ld_volatile_v4(p);
    if (v.y == c.flag && v.w == c.flag) return true;
    if ((++it & 63u) == 0) {
      if (dev::ld_relaxed_sys(c.abort_flag)) return false;
      if (dev::globaltimer() - t0 > c.timeout_ns) return false;
    }
  }
}

__device__ void eager_error(const KernelArgs& a, int code, int site, int d0, int d1) {
  dev::note_failure(a.heap, a.nproc, a.proc, a.lay.ctrl_off, a.host_status, code, site, d0, d1);
}

// payload word i (4 bytes) of a block that starts at `src` (any alignment), zero beyond `bytes`
__device__ __forceinline__ unsigned load_word(const char* src, size_t i, size_t bytes) {
  const size_t o = i * 4;
  if (o + 4 <= bytes && ((reinterpret_cast<uintptr_t>(src) & 3) == 0))
    return __ldcg(reinterpret_cast<const unsigned*>(src + o));
  unsigned w = 0;
  #pragma unroll
  for (int b = 0; b < 4; b++)
    if (o + b < bytes) w |= (unsigned)(unsigned char)__ldcg(src + o + b) << (8 * b);
  return w;
}
__device__ __forceinline__ void store_words(char* dst, size_t unit, unsigned w0, unsigned w1, size_t bytes) {
  const size_t o = unit * 8;
  if (o + 8 <= bytes && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0)) {
    *reinterpret_cast<uint2*>(dst + o) = make_uint2(w0, w1);
  } else if (o + 8 <= bytes && ((reinterpret_cast<uintptr_t>(dst) & 3) == 0)) {
    *reinterpret_cast<unsigned*>(dst + o) = w0;
    *reinterpret_cast<unsigned*>(dst + o + 4) = w1;
  } else {
    #pragma unroll
    for (int b = 0; b < 8; b++)
      if (o + b < bytes) dst[o + b] = (char)((b < 4 ? w0 >> (8 * b) : w1 >> (8 * (b - 4))) & 0xff);
  }
}

}  // namespace

__global__ void __launch_bounds__(kThreads, 1) a2av_eager_kernel(const __grid_constant__ KernelArgs a) {
  __shared__ unsigned s_prefix[kOpTileE + 1];
  __shared__ unsigned s_total, s_seq;
  __shared__ int s_last;
  const bool trace = (a.flags & CALL_TRACE) != 0;
  TraceBlock* tb = reinterpret_cast<TraceBlock*>(a.heap[a.proc] + a.lay.trace_off);
  const int P = a.P, L = a.L, ts = a.type_size;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned warps_per_cta = blockDim.x >> 5;
  const unsigned nwarps = gridDim.x * warps_per_cta;
  const unsigned gwarp = (a.flags & CALL_SPREAD) ? warp * gridDim.x + blockIdx.x : blockIdx.x * warps_per_cta + warp;
  CtrlBlock* my = ctrl_of(a, a.proc);
  const bool inl = (a.flags & CALL_META_INLINE) != 0;
  const int* sendcounts = inl ? a.inl.sendcounts : a.sendcounts;
  const int* recvcounts = inl ? a.inl.recvcounts : a.recvcounts;
  const long long* sdispls = inl ? a.inl.sdispls : a.sdispls;
  const long long* rdispls = inl ? a.inl.rdispls : a.rdispls;
  const size_t chunk = a.chunk_bytes;          // payload bytes per work item, a multiple of 8
  const size_t emax = a.eager_payload;

  // the call number is fetched while the first tile of work items is being sized (one barrier less on the
  // critical path of small calls)
  // Whoever completes CtrlBlock::start_count knows that everybody has read the call number and advances it for the
  // next call: CTAs count when the work items are sized in the kernel (thread 0 reads the number for its CTA), warps
  // count when the call brings its item table (every warp reads the number itself).
  const bool pre = a.items != nullptr;
  const bool hinted = a.use_seq_hint != 0;   // the host passed the call number: nobody reads it from memory
  unsigned seq_early = a.seq_hint;
  unsigned cta_rank = 0;     // thread 0, without an item table: CTAs that had read the call number before this one
  if (tid == 0) {
    if (!hinted) seq_early = dev::read_call_seq(my);
    if (blockIdx.x == 0) my->status.trace[0] = dev::globaltimer();
    if (a.flags & CALL_TRACE) atomicMax(&my->status.trace[5], dev::globaltimer());   // latest CTA start
    if (!pre) cta_rank = atomicAdd(&my->start_count, 1u);   // looked at when the CTA is done
  }
  unsigned seq = 0;
  int parity = 0;
  EagerCtx ec{&my->abort_flag, a.timeout_ns, 0u};
  bool alive = true;

  // Persistent calls with host-side counts bring a table of their work items: no sizing pass, no block-wide
  // barrier before the first byte moves; every warp fetches the call number itself.
  unsigned start_rank = 0;   // lane 0: how many warps had read the call number before this one
  if (pre) {
    unsigned sq = 0;
    if (lane == 0) {
      sq = (tid == 0 || hinted) ? seq_early : dev::read_call_seq(my);
      start_rank = atomicAdd(&my->start_count, 1u);   // the result is looked at after the warp's items
    }
    seq = hinted ? a.seq_hint : __shfl_sync(0xffffffffu, sq, 0);
    parity = seq & 1;
    ec.flag = seq + 1u;
    if (blockIdx.x == 0 && tid == 0) my->status.trace[1] = dev::globaltimer();
  }

  unsigned base = 0;
  for (int t0 = 0; t0 < (pre ? 1 : a.nops); t0 += kOpTileE) {
    const int tn = min(kOpTileE, a.nops - t0);
    if (!pre) {
    for (int i = tid; i < tn; i += blockDim.x) {
      const Op o = a.ops[t0 + i];
      const int lsrc = o.src - a.proc * L;
      size_t b;
      if (o.flags & 2u) {                     // unpack: bounded by the receiver's recvcount when it is known
        const int cap = recvcounts ? recvcounts[(size_t)lsrc * P + o.origin] : -1;
        b = cap >= 0 ? min((size_t)cap * ts, emax) : emax;
      } else if (o.src_cell < 0) {            // first hop (or self copy): size known locally
        b = (size_t)sendcounts[(size_t)lsrc * P + o.dest] * ts;
        // Small blocks: start fetching the block now.  By the time a warp picks the item up (two barriers and a
        // scan later) the lines are in L2, which takes one DRAM round trip off the path of a small call.
        if (b != 0 && b <= 1024) {
          const char* src = a.sendbuf[lsrc] + (size_t)sdispls[(size_t)lsrc * P + o.dest] * ts;
          for (size_t off = 0; off < b; off += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + off));
        }
      } else {
        b = emax;                             // relay: size arrives with the block
      }
      unsigned nch = (unsigned)((b + chunk - 1) / chunk);
      s_prefix[i + 1] = nch ? nch : 1u;
    }
    if (t0 == 0 && tid == 0) s_seq = seq_early;
    __syncthreads();
    if (t0 == 0) { seq = hinted ? a.seq_hint : s_seq; parity = seq & 1; ec.flag = seq + 1u; }
    if (tid < 32) {
      unsigned carry = 0;
      if (tid == 0) s_prefix[0] = 0;
      for (int i0 = 0; i0 < tn; i0 += 32) {
        int i = i0 + tid;
        unsigned v = (i < tn) ? s_prefix[i + 1] : 0u, s = v;
        #pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          unsigned n = __shfl_up_sync(0xffffffffu, s, d);
          if (tid >= d) s += n;
        }
        if (i < tn) s_prefix[i + 1] = s + carry;
        carry += __shfl_sync(0xffffffffu, s, 31);
      }
      if (tid == 0) s_total = carry;
    }
    __syncthreads();
    if (t0 == 0 && blockIdx.x == 0 && tid == 0) my->status.trace[1] = dev::globaltimer();   // work items sized
    }
    const unsigned total = pre ? a.nitems : s_total;
    unsigned c = (gwarp + nwarps - (base % nwarps)) % nwarps;
    int oi = 0;
    for (; c < total && alive; c += nwarps) {
      unsigned k;
      Op o;
      if (pre) {
        // the item brings its op along: one 32-byte fetch (none when the table fits the kernel parameters),
        // nothing that depends on it but the data itself
        union { uint4 q[2]; EagerItem it; } u;
        if (c < (unsigned)kInlineEagerItems) {
          u.it = a.inl_items[c];
        } else {
          const uint4* ip = reinterpret_cast<const uint4*>(a.items + c);
          u.q[0] = __ldg(ip);
          u.q[1] = __ldg(ip + 1);
        }
        o = u.it.op;
        k = u.it.k;
        oi = (int)u.it.index;
      } else {
        oi = dev::find_op(s_prefix, oi, tn, c);
        k = c - s_prefix[oi];
        o = a.ops[t0 + oi];
      }
      const int lsrc = o.src - a.proc * L;
      const unsigned kidx = min(op_key_index(o), (unsigned)kMaxTraceKeys - 1);
      if (trace && lane == 0) atomicMin(&tb->kstart[kidx], dev::globaltimer());
      const size_t u0 = (size_t)k * (chunk / 8);           // first payload unit of this item
      const size_t cu = chunk / 8;

      if (o.flags & 1u) {
        // ---- self copy: plain local copy, chunked ----
        const size_t bytes = (size_t)sendcounts[(size_t)lsrc * P + o.dest] * ts;
        const size_t off = (size_t)k * chunk;
        if (off < bytes) {
          const size_t len = min(chunk, bytes - off);
          dev::group_copy(a.heap[a.proc] + a.recvoff[lsrc] + (size_t)rdispls[(size_t)lsrc * P + o.origin] * ts + off,
                          a.sendbuf[lsrc] + (size_t)sdispls[(size_t)lsrc * P + o.dest] * ts + off, len, lane, 32);
        }
        if (trace && lane == 0) atomicMax(&tb->kend[kidx], dev::globaltimer());
        continue;
      }
      if (o.flags & 2u) {
        // ---- unpack: arrival cell -> receive buffer ----
        const uint4* cell = cell_of(a, a.proc, parity, lsrc, o.src_cell);
        uint4 h;
        bool ok = true;
        if (lane == 0) ok = poll_unit(cell, ec, h);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        unsigned bytes = __shfl_sync(0xffffffffu, h.x, 0);
        if (!ok) { if (lane == 0 && k == 0) eager_error(a, RBV_ERR_TIMEOUT, WAIT_CELL, t0 + oi, o.origin); alive = false; break; }
        if (bytes == kBadSize) { alive = false; break; }
        const int cap = recvcounts ? recvcounts[(size_t)lsrc * P + o.origin] : -1;
        if (cap >= 0 && (size_t)bytes > (size_t)cap * ts) {
          if (lane == 0 && k == 0) eager_error(a, RBV_ERR_TRUNCATE, 0, o.origin, o.src);
          continue;
        }
        const size_t nunits = ((size_t)bytes + 7) / 8;
        char* dst = a.heap[a.proc] + a.recvoff[lsrc] + (size_t)rdispls[(size_t)lsrc * P + o.origin] * ts;
        const size_t uend = min(nunits, u0 + cu);
        if (((reinterpret_cast<uintptr_t>(dst) & 15) | (u0 & 1)) == 0) {
          // two units per lane, written as one 16-byte vector (full 32-byte sectors; larger packets when the
          // receive buffer is pinned host memory)
          for (size_t u = u0 + 2 * lane; u < uend; u += 64) {
            uint4 v0, v1 = make_uint4(0u, 0u, 0u, 0u);
            bool got = poll_unit(cell + 1 + u, ec, v0);
            const bool two = u + 1 < uend;
            if (got && two) got = poll_unit(cell + 2 + u, ec, v1);
            if (!got) { eager_error(a, RBV_ERR_TIMEOUT, WAIT_CELL, t0 + oi, (int)u); alive = false; break; }
            if (two && (u + 2) * 8 <= bytes) {
              *reinterpret_cast<uint4*>(dst + u * 8) = make_uint4(v0.x, v0.z, v1.x, v1.z);
            } else {
              store_words(dst, u, v0.x, v0.z, bytes);
              if (two) store_words(dst, u + 1, v1.x, v1.z, bytes);
            }
          }
        } else {
          for (size_t u = u0 + lane; u < uend; u += 32) {
            uint4 v;
            if (!poll_unit(cell + 1 + u, ec, v)) { eager_error(a, RBV_ERR_TIMEOUT, WAIT_CELL, t0 + oi, (int)u); alive = false; break; }
            store_words(dst, u, v.x, v.z, bytes);
          }
        }
        alive = __all_sync(0xffffffffu, alive);
        if (trace && lane == 0) atomicMax(&tb->kend[kidx], dev::globaltimer());
        continue;
      }
      // ---- send: send buffer or staging cell -> cell on the destination rank ----
      const int dproc = o.dst / L, ldst = o.dst - dproc * L;
      uint4* dcell = cell_of(a, dproc, parity, ldst, o.dst_cell);
      if (o.src_cell < 0) {
        size_t bytes = (size_t)sendcounts[(size_t)lsrc * P + o.dest] * ts;
        if (bytes > emax) {
          if (lane == 0 && k == 0) { eager_error(a, RBV_ERR_CAPACITY, 0, o.src, o.dest); st_unit(dcell, kBadSize, 0u, ec.flag); }
          continue;
        }
        if (k == 0 && lane == 0) st_unit(dcell, (unsigned)bytes, 0u, ec.flag);
        const char* src = a.sendbuf[lsrc] + (size_t)sdispls[(size_t)lsrc * P + o.dest] * ts;
        const size_t nunits = (bytes + 7) / 8;
        const size_t uend = min(nunits, u0 + cu);
        if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
          // 16-byte loads, two units each; up to four loads per lane are issued before the first store so that
          // their DRAM latencies overlap
          for (size_t ub = u0; ub < uend; ub += 256) {
            uint4 v[4];
            bool full[4];
            #pragma unroll
            for (int j = 0; j < 4; j++) {
              const size_t u = ub + 64 * j + 2 * lane;
              full[j] = (u + 2 <= uend) && ((u + 2) * 8 <= bytes);
              if (full[j]) v[j] = dev::ld_cg_v4(reinterpret_cast<const uint4*>(src + u * 8));
            }
            #pragma unroll
            for (int j = 0; j < 4; j++) {
              const size_t u = ub + 64 * j + 2 * lane;
              if (full[j]) {
                st_unit(dcell + 1 + u, v[j].x, v[j].y, ec.flag);
                st_unit(dcell + 2 + u, v[j].z, v[j].w, ec.flag);
              } else if (u < uend) {
                st_unit(dcell + 1 + u, load_word(src, 2 * u, bytes), load_word(src, 2 * u + 1, bytes), ec.flag);
                if (u + 1 < uend)
                  st_unit(dcell + 2 + u, load_word(src, 2 * u + 2, bytes), load_word(src, 2 * u + 3, bytes), ec.flag);
              }
            }
          }
        } else {
          for (size_t u = u0 + lane; u < uend; u += 32)
            st_unit(dcell + 1 + u, load_word(src, 2 * u, bytes), load_word(src, 2 * u + 1, bytes), ec.flag);
        }
      } else {
        const uint4* scell = cell_of(a, a.proc, parity, lsrc, o.src_cell);
        uint4 h;
        bool ok = true;
        if (lane == 0) ok = poll_unit(scell, ec, h);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        const unsigned bytes = __shfl_sync(0xffffffffu, h.x, 0);
        if (!ok) { if (lane == 0 && k == 0) eager_error(a, RBV_ERR_TIMEOUT, WAIT_CELL, t0 + oi, o.src_cell); alive = false; break; }
        if (k == 0 && lane == 0) st_unit(dcell, bytes, 0u, ec.flag);
        if (bytes == kBadSize) continue;
        const size_t nunits = ((size_t)bytes + 7) / 8;
        const size_t uend = min(nunits, u0 + cu);
        for (size_t u = u0 + lane; u < uend; u += 32) {
          uint4 v;
          if (!poll_unit(scell + 1 + u, ec, v)) { eager_error(a, RBV_ERR_TIMEOUT, WAIT_CELL, t0 + oi, (int)u); alive = false; break; }
          st_unit(dcell + 1 + u, v.x, v.z, ec.flag);
        }
        alive = __all_sync(0xffffffffu, alive);
      }
      if (trace && lane == 0) atomicMax(&tb->kend[kidx], dev::globaltimer());
    }
    if (blockIdx.x == 0 && tid == 0) my->status.trace[2] = dev::globaltimer();   // first warp's items done
    base += total;
    __syncthreads();
  }

  // No end-of-call pass.  With an item table the warp that completed the start count advances the call number now
  // (its own items are done, so the atomic's result has long arrived); it also reports a communicator that was
  // told to stop.  (The rendezvous protocol keeps no per-call counter targets here, so the protocols mix freely.)
  if ((pre && lane == 0 && start_rank == nwarps - 1) || (!pre && tid == 0 && cta_rank == gridDim.x - 1)) {
    if (!hinted) dev::advance_call_seq(my, seq);
    else if (!dev::advance_call_seq_checked(my, seq)) eager_error(a, RBV_ERR_BAD_ARG, 0, (int)seq, -1);
    if (dev::ld_relaxed_sys(&my->abort_flag)) eager_error(a, RBV_ERR_ABORTED, 0, 0, 0);
  }
  if (trace) {
    __syncthreads();
    if (tid == 0) {
      const unsigned long long now = dev::globaltimer();
      if (blockIdx.x == 0) my->status.trace[3] = now;                            // first CTA done
      if (atomicMax(&my->status.trace[6], now) < now) my->status.trace[7] = blockIdx.x;   // latest CTA done, and which
      atomicMax(&my->status.trace[4], now);
    }
    dev::publish_trace(my, tb, a.host_trace, a.host_status, &s_last);
  }
}

cudaError_t a2av_eager_launch(const KernelArgs& args, int grid, bool cooperative, cudaStream_t stream) {
  void* params[] = {(void*)&args};
  if (cooperative)
    return cudaLaunchCooperativeKernel((const void*)a2av_eager_kernel, dim3(grid), dim3(kThreads), params, 0, stream);
  return cudaLaunchKernel((const void*)a2av_eager_kernel, dim3(grid), dim3(kThreads), params, 0, stream);
}

}  // namespace rbv
