// Static rendezvous kernel: the alltoallv of a persistent call whose counts were all known on the host.
//
// The reference learns the sizes of a round's blocks by exchanging them before the data
// (src/tuna2.cpp:160 and the MPI_Alltoall of counts in its drivers, examples/rbruckv_example.cpp:76) and sizes
// its staging by an MPI_Allreduce(MAX) per call (src/tuna2.cpp:45).  A persistent call repeats the same counts,
// so that exchange is done once, on the host, when the call is prepared; what is left for the device is a list
// of resolved copies ("items"): source address, destination address (a peer mapping over NVLink when the
// destination lives on another GPU), length, the chunk flag to wait for and the chunk flag to raise.  The kernel
// has no metadata phase, no tables and no sizing pass: a warp fetches an item (32 bytes), waits if the item
// forwards a staged chunk, copies, and signals.  Items are listed in plan order; inside one plan key (a round or
// a batch) the chunks of the different blocks alternate, so that a rank writes to all peers of the round at the
// same time instead of one after the other, and a relay hop forwards chunk k as soon as chunk k has landed.
//
// What remains of the metadata phase is one word per peer: at its start a process tells every other process which
// call it has entered, and a warp stores into another process's memory only after that process has entered the
// same call.  Otherwise a rank that runs ahead could overwrite a receive buffer, or a staging cell of the same
// parity, that its peer still uses for the previous call.  The wait costs one NVLink trip after the slowest peer
// has started and overlaps with the fetch of the first items.
//
// Completion is the same as in the dynamic kernel (a2av_kernel.cu): chunks that land in a receive buffer are
// tallied per CTA and added to the receiver's arrival counter behind one fence; the receiver's target for the
// call was counted on the host.  When one process hosts every rank nothing is tallied or waited for: every delivery
// is a store of this very launch, so the end of the kernel is the completion.  All waits are bounded.
#include <cuda_runtime.h>

#include "kernels/primitives.cuh"
#include "rbv/context.h"
#include "rbv/device_types.h"

namespace rbv {

namespace {

__device__ __forceinline__ CtrlBlock* ctrl_of(const StaticArgs& a, int proc) {
  return reinterpret_cast<CtrlBlock*>(a.heap[proc] + a.lay.ctrl_off);
}
__device__ __forceinline__ unsigned* flag_of(const StaticArgs& a, int proc, int parity, unsigned idx) {
  return reinterpret_cast<unsigned*>(a.heap[proc] + a.lay.flags_off) +
         ((size_t)parity * a.L * a.lay.flags_per_rank + idx);
}

__device__ void static_error(const StaticArgs& a, int code, int site, int d0, int d1) {
  dev::note_failure(a.heap, a.nproc, a.proc, a.lay.ctrl_off, a.host_status, code, site, d0, d1);
}

}  // namespace

// MINB = CTAs per SM the register budget is cut for: 1 keeps everything in registers (16 warps per SM), 2 trades a
// few spilled words for twice the warps, hence twice the loads in flight per SM.
template <int MINB>
__global__ void __launch_bounds__(kThreads, MINB) a2av_static_kernel(const __grid_constant__ StaticArgs a) {
  __shared__ unsigned s_arrived[kMaxRanksStatic];
  __shared__ unsigned s_seq;
  __shared__ int s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned warps_per_cta = blockDim.x >> 5;
  const bool multi = a.nproc > 1;
  // One process: items are dealt CTA by CTA (item c to warp c / grid of CTA c % grid), so the few items of a small
  // call run on as many SMs.  Several processes: 16 consecutive items per CTA, because every CTA that delivers to
  // another GPU pays a system-scope fence and a reduction per destination at its end (measured on 2 GPUs: spreading
  // the items cost 1-3 us per call).
  const unsigned nwarps = gridDim.x * warps_per_cta;
  const unsigned gwarp = multi ? blockIdx.x * warps_per_cta + warp : warp * gridDim.x + blockIdx.x;
  const bool trace = (a.flags & CALL_TRACE) != 0;
  CtrlBlock* my = ctrl_of(a, a.proc);
  TraceBlock* tb = reinterpret_cast<TraceBlock*>(a.heap[a.proc] + a.lay.trace_off);
  dev::WaitCfg wc{&my->abort_flag, a.timeout_ns};

  // The first items travel in the kernel parameters: the source of such an item is requested from memory before
  // anything else happens (with a call number that has to be read from memory, the two trips to DRAM overlap).
  if (gwarp < a.nitems && gwarp < (unsigned)kInlineItems) {
    const StaticItem& f = a.inl[gwarp];
    if (!(f.flags & ITEM_SRC_STAGE))
      for (unsigned off = lane * 128u; off < f.len; off += 32u * 128u)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(f.src + off));
  }
  // The CTA that completes the start count advances the call number for the next call; the count's result is only
  // looked at when the CTA is done, so the atomic's round trip is off the path of the data.
  unsigned start_rank = 0;
  if (tid == 0) {
    if (!a.use_seq_hint) s_seq = dev::read_call_seq(my);
    if (blockIdx.x == 0) my->status.trace[0] = dev::globaltimer();
    start_rank = atomicAdd(&my->start_count, 1u);
  }
  for (int i = tid; i < a.P; i += blockDim.x) s_arrived[i] = 0;
  __syncthreads();
  const unsigned seq = a.use_seq_hint ? a.seq_hint : s_seq;
  const int parity = seq & 1;
  const unsigned flagv = seq + 1u;
  if (multi && blockIdx.x == 0 && tid < a.nproc && tid != a.proc)
    dev::st_relaxed_sys(&ctrl_of(a, tid)->entered[a.proc], flagv);
  // the owner of a receive buffer adds the chunks this call brings to its running target
  if (multi && blockIdx.x == 0)
    for (int i = tid; i < a.L; i += blockDim.x) my->recv_target[i] += a.expect[i];

  bool alive = true;
  unsigned ready = 1u << a.proc;   // processes known to have entered this call
  for (unsigned c = gwarp; c < a.nitems; c += nwarps) {
    union { uint4 q[2]; StaticItem it; } u;
    if (c < (unsigned)kInlineItems) {
      u.it = a.inl[c];
    } else {
      const uint4* ip = reinterpret_cast<const uint4*>(a.items + c);
      u.q[0] = __ldg(ip);
      u.q[1] = __ldg(ip + 1);
    }
    const StaticItem& it = u.it;
    const unsigned kidx = min((unsigned)(it.flags >> 8), (unsigned)kMaxTraceKeys - 1);
    if (trace && lane == 0) atomicMin(&tb->kstart[kidx], dev::globaltimer());
    const int dproc = it.dst_rank / a.L;
    const bool remote = (it.flags & ITEM_REMOTE) != 0;
    bool ok = alive;
    if (ok && !((ready >> dproc) & 1u)) {
      int r = 0;
      if (lane == 0) {
        r = dev::wait_ge(&my->entered[dproc], flagv, wc, true);
        if (r == dev::WAIT_TIMEOUT) static_error(a, RBV_ERR_TIMEOUT, WAIT_META, (int)c, dproc);
      }
      r = __shfl_sync(0xffffffffu, r, 0);
      if (r == dev::WAIT_OK) ready |= 1u << dproc;
      else { ok = false; alive = false; }
    }
    if (ok && it.wait_flag != kNoFlag) {
      int r = 0;
      if (lane == 0) {
        r = dev::wait_ge(flag_of(a, a.proc, parity, it.wait_flag), flagv, wc, multi);
        if (r == dev::WAIT_TIMEOUT) static_error(a, RBV_ERR_TIMEOUT, WAIT_CELL, (int)c, (int)it.wait_flag);
      }
      r = __shfl_sync(0xffffffffu, r, 0);
      if (r != dev::WAIT_OK) { ok = false; alive = false; }
    }
    if (ok && it.len) {
      const char* src = reinterpret_cast<const char*>(it.src) + ((it.flags & ITEM_SRC_STAGE) ? (size_t)parity * a.lay.arena_bytes : 0);
      char* dst = reinterpret_cast<char*>(it.dst) + ((it.flags & ITEM_DST_STAGE) ? (size_t)parity * a.lay.arena_bytes : 0);
      dev::group_copy(dst, src, it.len, lane, 32);
    }
    __syncwarp();
    if (lane == 0) {
      if (it.signal_flag == kNoFlag) { if (multi) atomicAdd(&s_arrived[it.dst_rank], 1u); }
      else if (ok) dev::signal_store(flag_of(a, dproc, parity, it.signal_flag), flagv, remote);
      if (trace) atomicMax(&tb->kend[kidx], dev::globaltimer());
    }
  }
  __syncwarp();
  __syncthreads();
  if (tid == 0 && start_rank == gridDim.x - 1) {
    if (!a.use_seq_hint) dev::advance_call_seq(my, seq);
    else if (!dev::advance_call_seq_checked(my, seq)) static_error(a, RBV_ERR_BAD_ARG, 0, (int)seq, -1);
  }
  // report this CTA's deliveries: the barrier orders every warp's stores before the fence, which publishes them
  if (blockIdx.x == 0 && tid == 0) my->status.trace[5] = dev::globaltimer();
  for (int d = tid; multi && d < a.P; d += blockDim.x) {
    const unsigned n = s_arrived[d];
    const int dproc = d / a.L;
    const bool far = dproc != a.proc;
    if (n) {
      dev::fence_acq_rel(far);
      dev::red_relaxed_add(&ctrl_of(a, dproc)->recv_arrivals[d - dproc * a.L], (unsigned long long)n, far);
    }
  }
  if (blockIdx.x == 0) {
    if (tid == 0) my->status.trace[3] = my->status.trace[6] = dev::globaltimer();
    for (int i = tid; multi && i < a.L; i += blockDim.x) {
      const unsigned long long target = my->recv_target[i];
      int r = alive ? dev::wait_ge(&my->recv_arrivals[i], target, wc, multi) : (int)dev::WAIT_ABORTED;
      if (r == dev::WAIT_TIMEOUT)
        static_error(a, RBV_ERR_TIMEOUT, WAIT_RECV, i, (int)(target - my->recv_arrivals[i]));
      if (r != dev::WAIT_OK) alive = false;
    }
    // a process that was told to stop (or runs on a communicator that failed earlier and was not reset) says so;
    // where fewer than all threads wait above, the load overlaps with that wait
    if (tid == (int)blockDim.x - 1 && dev::ld_relaxed_sys(&my->abort_flag)) static_error(a, RBV_ERR_ABORTED, 0, 0, 0);
    // Everything has arrived: received blocks the caller wants elsewhere (pinned host memory, say) are copied on by
    // this CTA, whose 16 warps outrun a PCIe link; the end of the kernel then is the end of the whole transfer.
    if (a.ndrain) {
      const int all_ok = __syncthreads_and(alive ? 1 : 0);
      if (all_ok)
        for (unsigned c = warp; c < a.ndrain; c += warps_per_cta) {
          const DrainItem di = a.drain[c];
          dev::group_copy(reinterpret_cast<char*>(di.dst), reinterpret_cast<const char*>(di.src), di.len, lane, 32);
        }
    }
    __syncthreads();
    if (tid == 0) my->status.trace[4] = my->status.trace[7] = dev::globaltimer();
  }
  // No end-of-call pass: the call number was advanced at the start and failures are reported where they happen.
  // Only traced calls gather their stamps here.
  if (trace) dev::publish_trace(my, tb, a.host_trace, a.host_status, &s_last);
}

cudaError_t a2av_static_configure(int occupancy, int* max_ctas_per_sm) {
  int nb = 0;
  cudaError_t e = occupancy >= 2
      ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, a2av_static_kernel<2>, kThreads, 0)
      : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, a2av_static_kernel<1>, kThreads, 0);
  if (max_ctas_per_sm) *max_ctas_per_sm = nb;
  return e;
}

cudaError_t a2av_static_launch(const StaticArgs& args, int grid, int occupancy, bool cooperative, cudaStream_t stream) {
  void* params[] = {(void*)&args};
  const void* fn = occupancy >= 2 ? (const void*)a2av_static_kernel<2> : (const void*)a2av_static_kernel<1>;
  if (cooperative) return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kThreads), params, 0, stream);
  return cudaLaunchKernel(fn, dim3(grid), dim3(kThreads), params, 0, stream);
}

}  // namespace rbv
