// The alltoallv kernel: one persistent cooperative launch per call and per process that performs
//   (1) the metadata phase  -- every rank stores its sendcounts / recvcounts / rdispls row and its
//       receive-buffer offset into every process's metadata table as self-validating 16-byte units
//       (this replaces the host-side MPI_Alltoall of counts in the reference's drivers, the
//       MPI_Allreduce(MAX) and the per-round metadata MPI_Sendrecv, e.g. src/tuna2.cpp:45,160),
//   (2) the data phase      -- an interpreter of the plan's op list: each op copies one block from
//       the executing rank's send buffer or staging cell straight into the destination rank's
//       receive buffer or staging cell (a peer mapping over NVLink when the destination lives on
//       another GPU); rotation, pack, unpack and final placement are folded into the addressing,
//   (3) completion          -- waits until every chunk bound for a local rank's receive buffer has landed
//       (chunks of final hops are tallied per CTA in shared memory and added to the receivers' arrival counters
//       once per op tile, behind one fence; the receiver knows all sizes and therefore the count to wait for).
//
// Work distribution: ops are cut into chunks of `chunk_bytes`; chunk c of the process-wide
// sequence is handled by WARP c mod (warps in the grid).  A warp copies its chunk with 16-byte
// vectors (512 contiguous bytes per warp instruction; optionally with cp.async.bulk through a
// shared-memory ring, see bulk_copy.cuh).  A chunk that lands in a staging cell raises that chunk's own flag on the
// destination, and the relay hop that forwards chunk k waits for chunk k only, so the hops of a store-and-forward
// schedule overlap chunk by chunk (the reference keeps all rounds of a digit in flight and unpacks after the
// digit, src/tuna2.cpp:184-223; here the pipeline is per chunk).  Small blocks thus proceed in parallel, one warp
// each, and large blocks are spread over all warps of all SMs.  Warps walk their chunks in plan order, so a wait
// on a staging chunk only ever depends on chunks of an earlier plan key, which rules out cycles as long as all
// CTAs are resident (cooperative launch).
//
// This kernel serves calls whose counts are not all known on the host (device-resident counts, one-shot calls of
// a multi-process communicator) and in-place calls; persistent calls with host-side counts run the static kernel
// (a2av_static.cu).  A block that a plan sends in slices (split_alltoallv) travels whole here, with its first slice.
//
// Signals use gpu scope when producer and consumer are on the same GPU and system scope across
// GPUs.  The call number lives in device memory (CtrlBlock::call_seq), so the kernel arguments of
// a repeated call are constant.
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include "kernels/bulk_copy.cuh"
#include "kernels/primitives.cuh"
#include "rbv/device_types.h"

namespace cg = cooperative_groups;

namespace rbv {

namespace {

constexpr int kOpTile = 1024;

// Tiles per warp of the bulk-copy ring: three where the tables of the communicator leave room in shared memory.
__host__ __device__ constexpr int a2av_bulk_stages(int P) { return P <= 16 ? dev::kBulkMaxStages : 2; }

struct Smem {
  int* counts;
  int* caps;
  long long* rdispl;
  unsigned long long* recvoff;
  unsigned* schunk;     // chunk size used by each sending rank
  unsigned* prefix;
};

__device__ __forceinline__ CtrlBlock* ctrl_of(const KernelArgs& a, int proc) {
  return reinterpret_cast<CtrlBlock*>(a.heap[proc] + a.lay.ctrl_off);
}
__device__ __forceinline__ unsigned* chunk_flag_of(const KernelArgs& a, int proc, int parity, int lr, size_t f) {
  return reinterpret_cast<unsigned*>(a.heap[proc] + a.lay.flags_off) +
         ((size_t)(parity * a.L + lr) * a.lay.flags_per_rank + f);
}
__device__ __forceinline__ TraceBlock* trace_of(const KernelArgs& a) {
  return reinterpret_cast<TraceBlock*>(a.heap[a.proc] + a.lay.trace_off);
}
__device__ __forceinline__ char* meta_of(const KernelArgs& a, int proc, int parity) {
  return a.heap[proc] + a.lay.meta_off + (size_t)parity * a.lay.meta_bytes;
}
// One store that NVSwitch replicates into the tables of every process (NVLS multicast mapping).
__device__ __forceinline__ void st_unit_mc(uint4* mc, unsigned w0, unsigned w1, unsigned flag) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc), "f"(__uint_as_float(w0)), "f"(__uint_as_float(flag)), "f"(__uint_as_float(w1)),
                 "f"(__uint_as_float(flag)) : "memory");
}
__device__ __forceinline__ char* stage_of(const KernelArgs& a, int proc, int parity, int lr) {
  return a.heap[proc] + a.lay.stage_off + (size_t)(lr * 2 + parity) * a.lay.arena_bytes;
}

__device__ void report_error(const KernelArgs& a, int code, int site, int d0, int d1) {
  dev::note_failure(a.heap, a.nproc, a.proc, a.lay.ctrl_off, a.host_status, code, site, d0, d1);
}

__device__ __forceinline__ const int* in_sendcounts(const KernelArgs& a) {
  return (a.flags & CALL_META_INLINE) ? a.inl.sendcounts : a.sendcounts;
}
__device__ __forceinline__ const int* in_recvcounts(const KernelArgs& a) {
  return (a.flags & CALL_META_INLINE) ? a.inl.recvcounts : a.recvcounts;
}
__device__ __forceinline__ const long long* in_sdispls(const KernelArgs& a) {
  return (a.flags & CALL_META_INLINE) ? a.inl.sdispls : a.sdispls;
}
__device__ __forceinline__ const long long* in_rdispls(const KernelArgs& a) {
  return (a.flags & CALL_META_INLINE) ? a.inl.rdispls : a.rdispls;
}

__device__ __forceinline__ void st_unit(uint4* p, unsigned w0, unsigned w1, unsigned flag) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(w0), "r"(flag), "r"(w1), "r"(flag) : "memory");
}
__device__ __forceinline__ uint4 ld_unit(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Metadata rows of local rank lr go to process q: one warp per (lr, q) pair.  Every unit carries the call
// number, so nothing else has to be signalled.
__device__ void publish_metadata(const KernelArgs& a, int parity, unsigned flag) {
  const int P = a.P;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int* rc = in_recvcounts(a);
  if (a.meta_mc) {
    // NVLS: each local rank writes its rows once; the switch delivers them to every process
    for (int lr = warp; lr < a.L; lr += nwarps) {
      if (lr == a.absent_rank) continue;
      const int me = a.proc * a.L + lr;
      char* mt = a.meta_mc + (size_t)parity * a.lay.meta_bytes;
      uint4* ct = reinterpret_cast<uint4*>(mt + meta_ct_off(P)) + (size_t)me * P;
      uint4* rt = reinterpret_cast<uint4*>(mt + meta_rt_off(P)) + (size_t)me * P * 2;
      uint4* ro = reinterpret_cast<uint4*>(mt + meta_ro_off(P)) + me;
      const int* sc = in_sendcounts(a) + (size_t)lr * P;
      const long long* rdi = in_rdispls(a) + (size_t)lr * P;
      for (int i = lane; i < P; i += 32) {
        const unsigned long long rd = (unsigned long long)rdi[i];
        st_unit_mc(ct + i, (unsigned)sc[i], (unsigned)a.chunk_bytes, flag);
        st_unit_mc(rt + 2 * i, rc ? (unsigned)rc[(size_t)lr * P + i] : 0xffffffffu, 0u, flag);
        st_unit_mc(rt + 2 * i + 1, (unsigned)rd, (unsigned)(rd >> 32), flag);
      }
      if (lane == 0) st_unit_mc(ro, (unsigned)a.recvoff[lr], (unsigned)(a.recvoff[lr] >> 32), flag);
    }
    return;
  }
  for (int pair = warp; pair < a.L * a.nproc; pair += nwarps) {
    const int lr = pair / a.nproc, q = pair % a.nproc;
    if (lr == a.absent_rank) continue;  // host-injected fault: the rank "never joins"
    const int me = a.proc * a.L + lr;
    char* mt = meta_of(a, q, parity);
    uint4* ct = reinterpret_cast<uint4*>(mt + meta_ct_off(P)) + (size_t)me * P;
    uint4* rt = reinterpret_cast<uint4*>(mt + meta_rt_off(P)) + (size_t)me * P * 2;
    uint4* ro = reinterpret_cast<uint4*>(mt + meta_ro_off(P)) + me;
    const int* sc = in_sendcounts(a) + (size_t)lr * P;
    const long long* rdi = in_rdispls(a) + (size_t)lr * P;
    for (int i = lane; i < P; i += 32) {
      const unsigned long long rd = (unsigned long long)rdi[i];
      st_unit(ct + i, (unsigned)sc[i], (unsigned)a.chunk_bytes, flag);
      st_unit(rt + 2 * i, rc ? (unsigned)rc[(size_t)lr * P + i] : 0xffffffffu, 0u, flag);
      st_unit(rt + 2 * i + 1, (unsigned)rd, (unsigned)(rd >> 32), flag);
    }
    if (lane == 0) st_unit(ro, (unsigned)a.recvoff[lr], (unsigned)(a.recvoff[lr] >> 32), flag);
  }
}

// Bytes the op moves: the whole block; a block that the plan cuts into slices travels with its first slice.
__device__ __forceinline__ size_t op_bytes(const Op& o, const Smem& sm, int P, int ts) {
  if (op_nparts(o) && op_part(o)) return 0;
  return (size_t)sm.counts[(size_t)o.origin * P + o.dest] * (size_t)ts;
}
__device__ __forceinline__ bool op_skipped(const Op& o) { return op_nparts(o) && op_part(o); }

}  // namespace

__global__ void __launch_bounds__(kThreads, 1) a2av_kernel(const __grid_constant__ KernelArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int s_flag;
  __shared__ unsigned s_total;
  __shared__ unsigned s_seq;
  __shared__ int s_last;
  __shared__ unsigned s_arrived[kMaxRanks];   // chunks this CTA delivered to each rank's receive buffer, not yet reported
  const int P = a.P, L = a.L, ts = a.type_size;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned warps_per_cta = blockDim.x >> 5;
  const unsigned gwarp = blockIdx.x * warps_per_cta + warp, nwarps = gridDim.x * warps_per_cta;
  const bool multi = a.nproc > 1;   // some producers are on other GPUs
  CtrlBlock* my = ctrl_of(a, a.proc);
  dev::WaitCfg wc{&my->abort_flag, a.timeout_ns};

  Smem sm;
  unsigned char* bulk_region;
  {
    unsigned char* p = smem_raw;
    sm.rdispl = reinterpret_cast<long long*>(p); p += 8ull * P * P;
    sm.recvoff = reinterpret_cast<unsigned long long*>(p); p += 8ull * P;
    sm.counts = reinterpret_cast<int*>(p); p += 4ull * P * P;
    sm.caps = reinterpret_cast<int*>(p); p += 4ull * P * P;
    sm.schunk = reinterpret_cast<unsigned*>(p); p += 4ull * P;
    sm.prefix = reinterpret_cast<unsigned*>(p); p += 4ull * (kOpTile + 1);
    bulk_region = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(p) + 127) & ~uintptr_t(127));
  }
  const bool bulk = (a.flags & CALL_BULK) != 0;
  dev::BulkPipe bp{0u, 0u, 0u, 2u};
  if (bulk) dev::bulk_pipe_init(bp, bulk_region, warp, (int)warps_per_cta, lane, a2av_bulk_stages(P));   // published by the barrier below

  if (tid < kMaxRanks) s_arrived[tid] = 0;
  // The CTA that completes the start count advances the call number for the next call (checked at the end).
  unsigned start_rank = 0;
  if (tid == 0) {
    if (!a.use_seq_hint) s_seq = dev::read_call_seq(my);
    if (blockIdx.x == 0) my->status.trace[0] = dev::globaltimer();
    start_rank = atomicAdd(&my->start_count, 1u);
  }
  __syncthreads();
  const unsigned seq = a.use_seq_hint ? a.seq_hint : s_seq;
  const int parity = seq & 1;

  // ---- in-place calls: move the send data out of recvbuf before anyone may write into it ----
  if (a.flags & CALL_INPLACE) {
    for (int lr = 0; lr < L; lr++) {
      const size_t n = a.sendcopy_bytes[lr];
      const size_t per = ((n + gridDim.x - 1) / gridDim.x + 15) & ~(size_t)15;
      const size_t lo = (size_t)blockIdx.x * per;
      if (lo < n) {
        const size_t len = (lo + per <= n) ? per : n - lo;
        dev::cta_copy(a.heap[a.proc] + a.sendcopy_off[lr] + lo, a.heap[a.proc] + a.recvoff[lr] + lo, len);
      }
    }
    __threadfence();
    cg::this_grid().sync();
  }

  // ---- (1) metadata phase ----
  if (blockIdx.x == 0) {
    publish_metadata(a, parity, seq + 1u);
    if (tid == 0) my->status.trace[1] = dev::globaltimer();
  }
  // every CTA polls the table units until they carry this call's number and keeps a copy in shared memory
  bool alive = true;
  int mx = 0;
  {
    const char* mt = a.meta_self + (size_t)parity * a.lay.meta_bytes;
    const uint4* ct = reinterpret_cast<const uint4*>(mt + meta_ct_off(P));
    const uint4* rt = reinterpret_cast<const uint4*>(mt + meta_rt_off(P));
    const uint4* ro = reinterpret_cast<const uint4*>(mt + meta_ro_off(P));
    const unsigned flag = seq + 1u;
    const int nunits = 3 * P * P + P;
    unsigned long long t_start = 0;
    bool failed = false;
    for (int u = tid; u < nunits && !failed; u += blockDim.x) {
      const uint4* src = u < P * P ? ct + u : (u < 3 * P * P ? rt + (u - P * P) : ro + (u - 3 * P * P));
      uint4 v = ld_unit(src);
      unsigned it = 0;
      while (v.y != flag || v.w != flag) {
        if ((++it & 63u) == 0) {
          if (!t_start) t_start = dev::globaltimer();
          if (dev::ld_relaxed_sys(&my->abort_flag) || dev::globaltimer() - t_start > a.timeout_ns) { failed = true; break; }
        }
        v = ld_unit(src);
      }
      if (failed) {
        if (!dev::ld_relaxed_sys(&my->abort_flag)) report_error(a, RBV_ERR_TIMEOUT, WAIT_META, u, nunits);
        break;
      }
      if (u < P * P) {
        sm.counts[u] = (int)v.x;
        if (u % P == 0) sm.schunk[u / P] = v.z;
        mx = max(mx, (int)v.x);
      } else if (u < 3 * P * P) {
        const int e = (u - P * P) >> 1;
        if (((u - P * P) & 1) == 0) sm.caps[e] = (int)v.x;
        else sm.rdispl[e] = (long long)((unsigned long long)v.x | ((unsigned long long)v.z << 32));
      } else {
        sm.recvoff[u - 3 * P * P] = (unsigned long long)v.x | ((unsigned long long)v.z << 32);
      }
    }
    alive = !__syncthreads_or(failed ? 1 : 0);
  }

  // Chunking must be the same on every rank (receivers count chunks): use the largest proposal.
  unsigned long long chunk_b = a.chunk_bytes;
  if (alive) {
    for (int s = 0; s < P; s++) chunk_b = max(chunk_b, (unsigned long long)sm.schunk[s]);
  }
  size_t stride = 0;
  unsigned long long fpc = 1;   // chunk flags per staging cell
  const bool trace = (a.flags & CALL_TRACE) != 0;
  if (alive) {
    // global max block -> staging cell stride (the reference's max_send_count allreduce)
    if (a.ncells > 0) {
      mx = __reduce_max_sync(0xffffffffu, mx);
      if (tid == 0) s_flag = 0;
      __syncthreads();
      if (lane == 0) atomicMax(&s_flag, mx);
      __syncthreads();
      stride = (((size_t)s_flag * ts) + 15) & ~(size_t)15;
      if (stride * (size_t)a.ncells > a.lay.arena_bytes) {
        if (blockIdx.x == 0 && tid == 0) report_error(a, RBV_ERR_CAPACITY, 0, a.ncells, (int)(stride >> 10));
        alive = false;
      }
      // every chunk of a staging cell has a flag of its own: chunks must be large enough for the flags to suffice
      // (same inputs on every rank, hence the same result)
      fpc = a.lay.flags_per_rank / (unsigned long long)a.ncells;
      const unsigned long long need = ((stride + fpc - 1) / fpc + 15) & ~15ull;
      chunk_b = max(chunk_b, need);
    }
    // the owner of a receive buffer adds the chunks it expects in this call to its running target
    if (blockIdx.x == 0 && tid < L) {
      const int me = a.proc * L + tid;
      unsigned long long expect = 0;
      for (int s = 0; s < P; s++) {
        const unsigned long long b = (unsigned long long)sm.counts[s * P + me] * (unsigned long long)ts;
        const unsigned long long n = (b + chunk_b - 1) / chunk_b;
        expect += n ? n : 1ull;
      }
      my->recv_target[tid] += expect;
    }
    if (blockIdx.x == 0 && tid == 0) my->status.trace[2] = dev::globaltimer();
  }

  // ---- (2) data phase ----
  unsigned base = 0;  // chunks before the current tile
  for (int t0 = 0; t0 < a.nops; t0 += kOpTile) {
    const int tn = min(kOpTile, a.nops - t0);
    for (int i = tid; i < tn; i += blockDim.x) {
      const Op o = a.ops[t0 + i];
      size_t b = alive ? op_bytes(o, sm, P, ts) : 0;
      unsigned nch = (unsigned)((b + chunk_b - 1) / chunk_b);
      sm.prefix[i + 1] = op_skipped(o) ? 0u : (nch ? nch : 1u);   // empty blocks still signal their arrival
    }
    __syncthreads();
    if (tid < 32) {
      unsigned carry = 0;
      if (tid == 0) sm.prefix[0] = 0;
      for (int i0 = 0; i0 < tn; i0 += 32) {
        int i = i0 + tid;
        unsigned v = (i < tn) ? sm.prefix[i + 1] : 0u;
        unsigned s = v;
        #pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          unsigned n = __shfl_up_sync(0xffffffffu, s, d);
          if (tid >= d) s += n;
        }
        if (i < tn) sm.prefix[i + 1] = s + carry;
        carry += __shfl_sync(0xffffffffu, s, 31);
      }
      if (tid == 0) s_total = carry;
    }
    __syncthreads();
    const unsigned total = s_total;

    // first chunk of this tile owned by this warp
    unsigned c = (gwarp + nwarps - (base % nwarps)) % nwarps;
    int oi = 0;
    for (; c < total; c += nwarps) {
      oi = dev::find_op(sm.prefix, oi, tn, c);   // chunks are visited in order: the search resumes at the last op
      const Op o = a.ops[t0 + oi];
      const unsigned k = c - sm.prefix[oi];
      if (trace && lane == 0) atomicMin(&trace_of(a)->kstart[min(op_key_index(o), (unsigned)kMaxTraceKeys - 1)], dev::globaltimer());
      const int lsrc = o.src - a.proc * L;
      const int dproc = o.dst / L, ldst = o.dst - dproc * L;
      const bool remote = dproc != a.proc;
      bool ok = alive;
      size_t bytes = ok ? op_bytes(o, sm, P, ts) : 0;

      // truncation check for blocks that go to a receive buffer
      if (ok && o.dst_cell < 0) {
        const int cap = sm.caps[(size_t)o.dst * P + o.origin];
        if (cap >= 0 && sm.counts[(size_t)o.origin * P + o.dest] > cap) {
          if (lane == 0 && k == 0) report_error(a, RBV_ERR_TRUNCATE, 0, o.origin, o.dest);
          bytes = 0;
        }
      }
      // wait for this chunk of the source cell
      if (ok && o.src_cell >= 0) {
        int r = 0;
        if (lane == 0) {
          r = dev::wait_ge(chunk_flag_of(a, a.proc, parity, lsrc, (size_t)o.src_cell * fpc + k), seq + 1u, wc, multi);
          if (r == dev::WAIT_TIMEOUT) report_error(a, RBV_ERR_TIMEOUT, WAIT_CELL, t0 + oi, o.src_cell);
        }
        r = __shfl_sync(0xffffffffu, r, 0);
        if (r != dev::WAIT_OK) { ok = false; alive = false; }
      }
      if (ok && bytes) {
        const size_t off = (size_t)k * chunk_b;
        const size_t len = (off + chunk_b <= bytes) ? (size_t)chunk_b : bytes - off;
        const char* src;
        if (o.src_cell < 0) {
          const char* sb = (a.flags & CALL_INPLACE) ? (a.heap[a.proc] + a.sendcopy_off[lsrc]) : a.sendbuf[lsrc];
          src = sb + (size_t)in_sdispls(a)[(size_t)lsrc * P + o.dest] * ts;
        } else {
          src = stage_of(a, a.proc, parity, lsrc) + (size_t)o.src_cell * stride;
        }
        char* dst;
        if (o.dst_cell < 0)
          dst = a.heap[dproc] + sm.recvoff[o.dst] + (size_t)sm.rdispl[(size_t)o.dst * P + o.origin] * ts;
        else
          dst = stage_of(a, dproc, parity, ldst) + (size_t)o.dst_cell * stride;
        if (bulk && len >= dev::kBulkMinBytes &&
            ((reinterpret_cast<uintptr_t>(dst + off) | reinterpret_cast<uintptr_t>(src + off)) & 15u) == 0) {
          // one thread drives the copy engine; a tail shorter than 16 bytes goes through the vector path
          const size_t body = len & ~(size_t)15;
          int r = 0;
          if (lane == 0) {
            r = dev::bulk_copy(dst + off, src + off, body, bp, wc);
            if (r == dev::WAIT_TIMEOUT) report_error(a, RBV_ERR_TIMEOUT, WAIT_BULK, t0 + oi, (int)k);
          }
          r = __shfl_sync(0xffffffffu, r, 0);
          if (r != dev::WAIT_OK) { ok = false; alive = false; }
          else if (len > body) dev::group_copy(dst + off + body, src + off + body, len - body, lane, 32);
        } else {
          dev::group_copy(dst + off, src + off, len, lane, 32);
        }
      }
      __syncwarp();
      // completion.  Final hops: every chunk counts towards the receiver's arrival counter (the receiver knows
      // how many to expect); nobody looks at that counter before the end of the call, so the chunks are tallied
      // per CTA and reported once per op tile, which spares a fence and a remote atomic per chunk.
      // Staging cells: the chunk's own flag on the destination goes up as soon as the chunk has been stored.
      if (lane == 0) {
        if (o.dst_cell < 0) atomicAdd(&s_arrived[o.dst], 1u);
        else if (ok) dev::signal_store(chunk_flag_of(a, dproc, parity, ldst, (size_t)o.dst_cell * fpc + k), seq + 1u, remote);
        if (trace) atomicMax(&trace_of(a)->kend[min(op_key_index(o), (unsigned)kMaxTraceKeys - 1)], dev::globaltimer());
      }
    }
    // this warp's stores are performed before the CTA reports them
    __syncwarp();
    base += total;
    __syncthreads();
    if (blockIdx.x == 0 && tid == 0) my->status.trace[5] = dev::globaltimer();
    if (tid < P) {
      const unsigned n = atomicExch(&s_arrived[tid], 0u);
      const int dproc = tid / L;
      const bool far = dproc != a.proc;
      // the barrier above orders every warp's stores before this fence, which publishes them (cumulativity)
      if (n) dev::fence_acq_rel(far);
      if (blockIdx.x == 0 && tid == 0) my->status.trace[6] = dev::globaltimer();
      if (n) dev::red_relaxed_add(&ctrl_of(a, dproc)->recv_arrivals[tid - dproc * L], (unsigned long long)n, far);
    }
    if (blockIdx.x == 0 && tid == 0) my->status.trace[7] = dev::globaltimer();
  }

  if (tid == 0 && start_rank == gridDim.x - 1) {
    if (!a.use_seq_hint) dev::advance_call_seq(my, seq);
    else if (!dev::advance_call_seq_checked(my, seq)) report_error(a, RBV_ERR_BAD_ARG, 0, (int)seq, -1);
  }
  // ---- (3) completion ----
  if (blockIdx.x == 0) {
    if (tid == 0) my->status.trace[3] = dev::globaltimer();
    if (tid < L) {
      const unsigned long long target = my->recv_target[tid];
      int r = alive ? dev::wait_ge(&my->recv_arrivals[tid], target, wc, multi) : (int)dev::WAIT_ABORTED;
      if (r == dev::WAIT_TIMEOUT)
        report_error(a, RBV_ERR_TIMEOUT, WAIT_RECV, tid, (int)(target - my->recv_arrivals[tid]));
    }
    // a process that was told to stop (or runs on a communicator that failed earlier and was not reset) says so;
    // the load overlaps with the wait above
    if (tid == 32 && dev::ld_relaxed_sys(&my->abort_flag)) report_error(a, RBV_ERR_ABORTED, 0, 0, 0);
    __syncthreads();
    if (tid == 0) my->status.trace[4] = dev::globaltimer();
  }
  // No end-of-call pass: the call number was advanced at the start and failures are reported where they happen.
  // Only traced calls gather their stamps here.
  if (trace) dev::publish_trace(my, trace_of(a), a.host_trace, a.host_status, &s_last);
}

size_t a2av_smem_bytes(int P) {
  return 8ull * P * P + 8ull * P + 4ull * P * P * 2 + 4ull * P + 4ull * (kOpTile + 1) + 16;
}

// Dynamic shared memory of a launch that uses the bulk-copy engine: the tables plus one tile ring per warp.
size_t a2av_smem_bytes_bulk(int P) {
  return a2av_smem_bytes(P) + 128 + dev::bulk_smem_bytes(kThreads / 32, a2av_bulk_stages(P));
}

cudaError_t a2av_configure(int P, int* max_ctas_per_sm) {
  size_t smem = a2av_smem_bytes(P);
  // The attribute belongs to the kernel, not to a context: size it for the largest communicator so
  // that contexts with different rank counts can coexist in one process.
  cudaError_t e = cudaFuncSetAttribute(a2av_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)a2av_smem_bytes_bulk(kMaxRanks));
  if (e != cudaSuccess) return e;
  int nb = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, a2av_kernel, kThreads, smem);
  if (max_ctas_per_sm) *max_ctas_per_sm = nb;
  return e;
}

int a2av_bulk_ctas_per_sm(int P) {
  int nb = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, a2av_kernel, kThreads, a2av_smem_bytes_bulk(P)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return nb;
}

cudaError_t a2av_launch(const KernelArgs& args, int grid, bool cooperative, cudaStream_t stream) {
  void* params[] = {(void*)&args};
  const size_t smem = (args.flags & CALL_BULK) ? a2av_smem_bytes_bulk(args.P) : a2av_smem_bytes(args.P);
  // An in-place call synchronises the whole grid after moving the send data aside, which is defined for
  // cooperative launches only: such a call is launched cooperatively whatever the caller's preference.
  if (cooperative || (args.flags & CALL_INPLACE))
    return cudaLaunchCooperativeKernel((const void*)a2av_kernel, dim3(grid), dim3(kThreads), params, smem, stream);
  return cudaLaunchKernel((const void*)a2av_kernel, dim3(grid), dim3(kThreads), params, smem, stream);
}

}  // namespace rbv
