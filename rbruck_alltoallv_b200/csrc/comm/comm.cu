// Context implementation: heap layout, CUDA IPC peer mapping, symmetric allocator, plan cache and
// the launch path of the alltoallv kernel.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

#include <cuda.h>

#include "rbv/context.h"

namespace rbv {

namespace {
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

#define RBV_CUDA_THROW(expr)                                                              \
  do {                                                                                    \
    cudaError_t e__ = (expr);                                                             \
    if (e__ != cudaSuccess) {                                                             \
      char buf__[512];                                                                    \
      std::snprintf(buf__, sizeof buf__, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
      throw std::runtime_error(buf__);                                                    \
    }                                                                                     \
  } while (0)
}  // namespace

Context::Context(int P, int nproc, int proc, int device, size_t user_bytes, size_t arena_bytes)
    : P_(P), L_(nproc > 0 ? P / nproc : 0), nproc_(nproc), proc_(proc), device_(device) {
  if (P < 1 || P > kMaxRanksStatic) throw std::runtime_error("rank count must be in 1..1024");
  if (nproc < 1 || nproc > kMaxProcs || P % nproc != 0) throw std::runtime_error("process count must divide the rank count (max 16)");
  if (proc < 0 || proc >= nproc) throw std::runtime_error("process index out of range");
  RBV_CUDA_THROW(cudaSetDevice(device));
  cudaDeviceProp prop;
  RBV_CUDA_THROW(cudaGetDeviceProperties(&prop, device));
  sm_count_ = prop.multiProcessorCount;
  int per_sm = 1;
  RBV_CUDA_THROW(a2av_configure(std::min(P, kMaxRanks), &per_sm));
  per_sm = std::max(1, std::min(per_sm, 2));
  max_ctas_ = sm_count_ * per_sm;
  bulk_ctas_ = sm_count_ * std::max(0, std::min(a2av_bulk_ctas_per_sm(std::min(P, kMaxRanks)), 1));
  if (const char* e = std::getenv("RBV_BULK")) bulk_mode_ = std::atoi(e);
  if (const char* e = std::getenv("RBV_COOPERATIVE")) cooperative_mode_ = std::atoi(e) != 0 ? 1 : 0;
  if (const char* e = std::getenv("RBV_STATIC_OCC")) static_occ_ = std::atoi(e) >= 2 ? 2 : 1;
  if (const char* e = std::getenv("RBV_STATIC_SPREAD")) static_spread_ = std::atoi(e) != 0;
  if (const char* e = std::getenv("RBV_EAGER_SPREAD")) eager_spread_ = std::atoi(e);
  if (const char* e = std::getenv("RBV_SEQ_HINT")) seq_hints_ = std::atoi(e) != 0;
  int st_per_sm = 1;
  RBV_CUDA_THROW(a2av_static_configure(static_occ_, &st_per_sm));
  static_max_ctas_ = sm_count_ * std::max(1, std::min(st_per_sm, 2));

  lay_.ctrl_off = 0;
  lay_.trace_off = align_up(sizeof(CtrlBlock), 256);
  lay_.flags_off = lay_.trace_off + align_up(sizeof(TraceBlock), 256);
  lay_.flags_per_rank = L_ <= kMaxRanks ? kMaxFlagsPerRank : kMaxCellsPerRank;   // many ranks per GPU: fewer chunk flags each
  lay_.meta_off = lay_.flags_off + align_up(sizeof(unsigned) * 2ull * L_ * lay_.flags_per_rank, 256);
  lay_.meta_bytes = P <= kMaxRanks ? meta_table_bytes(P) : 256;   // larger communicators run static calls only: no tables
  lay_.stage_off = align_up(lay_.meta_off + 2 * lay_.meta_bytes, 4096);
  lay_.arena_bytes = align_up(arena_bytes, 4096);
  lay_.eager_off = lay_.stage_off + 2ull * L_ * lay_.arena_bytes;
  lay_.user_off = lay_.eager_off + 2ull * L_ * lay_.arena_bytes;
  lay_.total_bytes = lay_.user_off + align_up(user_bytes, 4096);

  RBV_CUDA_THROW(cudaMalloc(&heap_, lay_.total_bytes));
  RBV_CUDA_THROW(clear_library_regions());
  peer_[proc] = heap_;
  opened_[proc] = false;
  free_[lay_.user_off] = lay_.total_bytes - lay_.user_off;

  RBV_CUDA_THROW(cudaHostAlloc(&host_status_, sizeof(StatusBlock), cudaHostAllocMapped));
  std::memset(host_status_, 0, sizeof(StatusBlock));
  RBV_CUDA_THROW(cudaHostGetDevicePointer(&host_status_dev_, host_status_, 0));
  RBV_CUDA_THROW(cudaHostAlloc(&host_trace_, sizeof(TraceBlock), cudaHostAllocMapped));
  std::memset(host_trace_, 0, sizeof(TraceBlock));
  RBV_CUDA_THROW(cudaHostGetDevicePointer(&host_trace_dev_, host_trace_, 0));
  RBV_CUDA_THROW(cudaDeviceSynchronize());
}

// Everything in front of the user region starts at zero: counters, chunk flags, metadata tables, and both kinds of
// arena.  The eager cells in particular must not show flag words of an earlier life of this memory (a heap from
// cudaMalloc can be the memory of a context that was destroyed, and reset() restarts the call numbers).
cudaError_t Context::clear_library_regions() {
  cudaError_t e = cudaMemset(heap_, 0, lay_.user_off);
  if (e != cudaSuccess) return e;
  return cudaMemset(heap_ + lay_.trace_off + offsetof(TraceBlock, kstart), 0xff, sizeof(TraceBlock::kstart));
}

Context::~Context() {
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  nvls_teardown();
  for (auto& kv : plans_) {
    if (kv.second->d_ops) cudaFree(kv.second->d_ops);
    if (kv.second->d_done) cudaFree(kv.second->d_done);
    if (kv.second->d_eops) cudaFree(kv.second->d_eops);
  }
  for (int q = 0; q < nproc_; q++)
    if (opened_[q] && peer_[q]) cudaIpcCloseMemHandle(peer_[q]);
  for (int i = 0; i < kRing; i++) {
    if (ring_host_[i]) cudaFreeHost(ring_host_[i]);
    if (ring_dev_[i]) cudaFree(ring_dev_[i]);
    if (ring_ev_[i]) cudaEventDestroy(ring_ev_[i]);
  }
  if (host_status_) cudaFreeHost(host_status_);
  if (host_trace_) cudaFreeHost(host_trace_);
  if (heap_) cudaFree(heap_);
}

cudaError_t Context::ipc_handle(void* out64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, heap_);
  if (e == cudaSuccess) std::memcpy(out64, &h, 64);
  return e;
}

cudaError_t Context::connect(const void* handles) {
  cudaError_t e = cudaSetDevice(device_);
  if (e != cudaSuccess) return e;
  for (int q = 0; q < nproc_; q++) {
    if (q == proc_) continue;
    if (opened_[q]) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const char*>(handles) + 64 * q, 64);
    void* p = nullptr;
    e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return e;
    peer_[q] = static_cast<char*>(p);
    opened_[q] = true;
  }
  return cudaSuccess;
}

void* Context::symm_alloc(size_t bytes) {
  bytes = align_up(std::max<size_t>(bytes, 1), 256);
  for (auto it = free_.begin(); it != free_.end(); ++it) {
    if (it->second >= bytes) {
      size_t off = it->first, rest = it->second - bytes;
      free_.erase(it);
      if (rest) free_[off + bytes] = rest;
      used_[off] = bytes;
      return heap_ + off;
    }
  }
  return nullptr;
}

int Context::symm_free(void* p) {
  size_t off = static_cast<char*>(p) - heap_;
  auto it = used_.find(off);
  if (it == used_.end()) return -1;
  size_t bytes = it->second;
  used_.erase(it);
  auto ins = free_.emplace(off, bytes).first;
  auto next = std::next(ins);
  if (next != free_.end() && ins->first + ins->second == next->first) {
    ins->second += next->second;
    free_.erase(next);
  }
  if (ins != free_.begin()) {
    auto prev = std::prev(ins);
    if (prev->first + prev->second == ins->first) {
      prev->second += ins->second;
      free_.erase(ins);
    }
  }
  return 0;
}

bool Context::in_heap(const void* p, size_t bytes) const {
  const char* c = static_cast<const char*>(p);
  return c >= heap_ + lay_.user_off && c + bytes <= heap_ + lay_.total_bytes;
}

const DevPlan* Context::plan_for(const AlgoSpec& s) {
  auto key = std::make_tuple(s.algo, s.P, s.n, s.r, s.r2, s.b, s.b2);
  auto it = plans_.find(key);
  last_plan_build_s_ = 0;
  if (it != plans_.end()) return it->second.get();
  auto dp = std::make_unique<DevPlan>();
  const auto t_build = std::chrono::steady_clock::now();
  dp->plan = build_plan(s);
  last_plan_build_s_ = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_build).count();
  if (!dp->plan.err) {
    if (dp->plan.ncells > kMaxCellsPerRank) {
      dp->plan.err = -3;
      dp->plan.errmsg = "plan needs more staging cells than the communicator provides";
    } else {
      std::vector<int> mine(L_);
      for (int i = 0; i < L_; i++) mine[i] = proc_ * L_ + i;
      std::vector<Op> ops = ops_for_ranks(dp->plan, mine);
      dp->nops = (int)ops.size();
      dp->h_ops = ops;
      for (const Op& o : dp->plan.ops) if (op_nparts(o)) dp->has_parts = true;
      if (dp->nops) {
        RBV_CUDA_THROW(cudaMalloc(&dp->d_ops, ops.size() * sizeof(Op)));
        RBV_CUDA_THROW(cudaMemcpy(dp->d_ops, ops.data(), ops.size() * sizeof(Op), cudaMemcpyHostToDevice));
        RBV_CUDA_THROW(cudaMalloc(&dp->d_done, ops.size() * sizeof(unsigned)));
        RBV_CUDA_THROW(cudaMemset(dp->d_done, 0, ops.size() * sizeof(unsigned)));
      }
      // eager variant of the op list (communicators of more than 64 ranks run static calls only)
      std::vector<Op> eops;
      if (P_ > kMaxRanks) ops.clear();
      eops.reserve(ops.size() + (size_t)L_ * P_);
      for (Op o : ops) {
        if (!(o.flags & 1u)) {
          if (o.src_cell >= 0) o.src_cell += P_;
          o.dst_cell = o.dst_cell >= 0 ? o.dst_cell + P_ : (int)o.origin;
        }
        eops.push_back(o);
      }
      for (int lr = 0; lr < L_ && P_ <= kMaxRanks; lr++) {
        const int d = proc_ * L_ + lr;
        for (int s = 0; s < P_; s++) {
          if (s == d) continue;
          Op u{};
          u.src = u.dst = u.dest = (uint16_t)d; u.origin = (uint16_t)s;
          u.src_cell = s; u.dst_cell = -1; u.key = 0xffffffffu;
          u.flags = kOpUnpack | ((uint32_t)dp->plan.keys.size() << 16);   // unpacking is timed as a key of its own
          eops.push_back(u);
        }
      }
      dp->n_eops = (int)eops.size();
      dp->h_eops = eops;
      if (dp->n_eops) {
        RBV_CUDA_THROW(cudaMalloc(&dp->d_eops, eops.size() * sizeof(Op)));
        RBV_CUDA_THROW(cudaMemcpy(dp->d_eops, eops.data(), eops.size() * sizeof(Op), cudaMemcpyHostToDevice));
      }
    }
  }
  const DevPlan* out = dp.get();
  plans_[key] = std::move(dp);
  return out;
}

int Context::alltoallv(const AlgoSpec& spec, int ts, const CallArgs& ca, const CallOptions& opt,
                       cudaStream_t stream) {
  Prepared pc;
  int rc = prepare(spec, ts, ca, opt, stream, false, &pc);
  if (rc) return rc;
  return launch(pc, stream);
}

int Context::launch(const Prepared& pc, cudaStream_t stream) {
  // cooperative_mode_: 1 always cooperative, 0 never (in-place calls excepted), -1 only for calls that need it
  const bool coop = cooperative_mode_ > 0 || (cooperative_mode_ < 0 && pc.cooperative);
  // The host passes the call number along (one trip to device memory less before the first byte moves).  A launch
  // that is being recorded into a CUDA graph must read the number on the device, and after the first such launch
  // the host's count can no longer be trusted (replays advance the number unseen), so hints stay off from then on.
  if (seq_hints_) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
      (void)cudaGetLastError();
      seq_hints_ = false;
    }
  }
  cudaError_t e;
  if (pc.is_static) {
    StaticArgs sa = pc.sa;
    sa.seq_hint = host_seq_; sa.use_seq_hint = seq_hints_ ? 1u : 0u;
    e = a2av_static_launch(sa, pc.grid, static_occ_, coop, stream);
  } else {
    KernelArgs ka = pc.ka;
    ka.seq_hint = host_seq_; ka.use_seq_hint = seq_hints_ ? 1u : 0u;
    e = pc.eager ? a2av_eager_launch(ka, pc.grid, coop, stream) : a2av_launch(ka, pc.grid, coop, stream);
  }
  if (e == cudaSuccess) host_seq_++;
  if (e != cudaSuccess) {
    last_error_ = std::string("kernel launch failed: ") + cudaGetErrorString(e);
    return RBV_ERR_BAD_ARG;
  }
  return 0;
}

void Context::release(Prepared& pc) {
  if (pc.owned_meta) cudaFree(pc.owned_meta);
  pc.owned_meta = nullptr;
  if (pc.owned_items) cudaFree(pc.owned_items);
  pc.owned_items = nullptr;
}

int Context::prepare(const AlgoSpec& spec_in, int ts, const CallArgs& ca, const CallOptions& opt,
                     cudaStream_t stream, bool persistent, Prepared* out) {
  AlgoSpec spec = spec_in;
  spec.P = P_;
  const DevPlan* dp = plan_for(spec);
  if (dp->plan.err) { last_error_ = dp->plan.errmsg; return dp->plan.err; }
  last_plan_ = dp;
  if (ts < 1) { last_error_ = "type size must be positive"; return RBV_ERR_BAD_ARG; }
  const bool inplace = (opt.flags & CALL_INPLACE) != 0;
  const bool eager = opt.eager_max_bytes > 0;
  const unsigned long long emax = (opt.eager_max_bytes + 7) & ~7ull;
  out->is_static = false;
  out->cooperative = true;
  if (eager) {
    if (inplace) { last_error_ = "the eager protocol does not take in-place calls"; return RBV_ERR_BAD_ARG; }
    if (dp->has_parts) { last_error_ = "a schedule that sends a block in slices needs the rendezvous protocol"; return RBV_ERR_BAD_ARG; }
    if ((unsigned long long)(P_ + dp->plan.ncells) * (16 + 2 * emax) > lay_.arena_bytes) {
      last_error_ = "staging arena too small for the eager cells of this plan";
      return RBV_ERR_CAPACITY;
    }
  }
  if (inplace && ca.counts_on_device) { last_error_ = "in-place calls need host-side counts"; return RBV_ERR_BAD_ARG; }
  if (!ca.sendcounts || !ca.sdispls || !ca.rdispls || !ca.recvbufs || (!inplace && !ca.sendbufs)) {
    last_error_ = "null argument"; return RBV_ERR_BAD_ARG;
  }

  out->owned_meta = nullptr;
  out->owned_items = nullptr;
  for (int q = 0; q < nproc_; q++)
    if (!peer_[q]) { last_error_ = "peer heaps are not connected"; return RBV_ERR_BAD_ARG; }
  // A persistent call whose counts are all on the host (own ranks only when this process hosts every rank, or the
  // gathered tables) is resolved into copy descriptors and runs the static kernel.
  const bool will_be_static = persistent && opt.allow_static && !ca.counts_on_device && !eager && !inplace &&
                              absent_rank_ < 0 && (nproc_ == 1 || (ca.g_counts && ca.g_rdispls && ca.g_recvoff));
  // With host-side counts the receive extents are known: a buffer that ends beyond the heap is refused here
  // instead of letting peers store outside their mapping of it.  A static call of a single process addresses
  // everything absolutely and has no peers: there any device-accessible memory will do (pinned host memory
  // included) when the caller has checked the extents against its own knowledge of the buffers.
  if (!ca.counts_on_device && !eager && !(will_be_static && nproc_ == 1 && opt.recv_anywhere)) {
    for (int lr = 0; lr < L_; lr++) {
      long long ext = 0;
      for (int s2 = 0; s2 < P_; s2++) {
        long long cnt = 0;
        if (ca.recvcounts) cnt = ca.recvcounts[(size_t)lr * P_ + s2];
        else if (ca.g_counts) cnt = ca.g_counts[(size_t)s2 * P_ + (proc_ * L_ + lr)];
        else if (L_ == P_) cnt = ca.sendcounts[(size_t)s2 * P_ + lr];
        ext = std::max(ext, (ca.rdispls[(size_t)lr * P_ + s2] + std::max(cnt, 0ll)) * ts);
      }
      if (!in_heap(ca.recvbufs[lr], (size_t)std::max(ext, 1ll))) {
        last_error_ = "recvbuf must lie inside the symmetric heap with room for every block (displacement + count)";
        return RBV_ERR_BAD_ARG;
      }
    }
  }
  if (will_be_static) return prepare_static(dp, ts, ca, opt, out);
  if (P_ > kMaxRanks) {
    last_error_ = "communicators of more than 64 ranks take persistent calls with host-side counts only "
                  "(rendezvous protocol, not in place): prepare the call, then launch it";
    return RBV_ERR_BAD_ARG;
  }

  KernelArgs& ka = out->ka;
  std::memset(&ka, 0, sizeof ka);
  ka.P = P_; ka.L = L_; ka.nproc = nproc_; ka.proc = proc_;
  ka.type_size = ts;
  ka.flags = (opt.flags & CALL_INPLACE) | (trace_ ? (unsigned)CALL_TRACE : 0u);
  ka.nops = dp->nops;
  ka.absent_rank = absent_rank_;
  ka.ncells = dp->plan.ncells;
  ka.ops = dp->d_ops;
  ka.op_done = dp->d_done;
  ka.timeout_ns = timeout_ns_;
  ka.lay = lay_;
  for (int q = 0; q < nproc_; q++) ka.heap[q] = peer_[q];
  ka.host_status = host_status_dev_;
  ka.host_trace = host_trace_dev_;
  ka.meta_self = nvls_mc_ ? nvls_self_ : heap_ + lay_.meta_off;
  ka.meta_mc = nvls_mc_;
  for (int lr = 0; lr < L_; lr++) {
    if (!eager && !in_heap(ca.recvbufs[lr], 1)) {
      last_error_ = "recvbuf must be allocated from the symmetric heap";
      return RBV_ERR_BAD_ARG;
    }
    ka.recvoff[lr] = static_cast<char*>(ca.recvbufs[lr]) - heap_;
    ka.sendbuf[lr] = inplace ? nullptr : static_cast<const char*>(ca.sendbufs[lr]);
  }

  // --- counts / displacements ---
  const size_t n = (size_t)L_ * P_;
  long long send_bytes = ca.bytes_hint;
  if (!ca.counts_on_device) {
    send_bytes = 0;
    for (size_t i = 0; i < n; i++) {
      if (ca.sendcounts[i] < 0 || ca.sdispls[i] < 0 || ca.rdispls[i] < 0 || (ca.recvcounts && ca.recvcounts[i] < 0)) {
        last_error_ = "negative count or displacement"; return RBV_ERR_BAD_ARG;
      }
      send_bytes += (long long)ca.sendcounts[i] * ts;
      if (eager && (unsigned long long)ca.sendcounts[i] * ts > emax) {
        last_error_ = "a block is larger than the eager cell size"; return RBV_ERR_CAPACITY;
      }
    }
    if (inplace) {
      size_t total = 0;
      for (int lr = 0; lr < L_; lr++) {
        size_t ext = 0;
        for (int d = 0; d < P_; d++)
          ext = std::max(ext, (size_t)(ca.sdispls[(size_t)lr * P_ + d] + ca.sendcounts[(size_t)lr * P_ + d]) * ts);
        ka.sendcopy_bytes[lr] = ext;
        total += align_up(ext, 256);
      }
      if (total > sendcopy_bytes_) {
        if (sendcopy_) symm_free(sendcopy_);
        sendcopy_ = symm_alloc(total);
        sendcopy_bytes_ = sendcopy_ ? total : 0;
        if (!sendcopy_) { last_error_ = "symmetric heap exhausted (in-place copy)"; return RBV_ERR_CAPACITY; }
      }
      size_t off = static_cast<char*>(sendcopy_) - heap_;
      for (int lr = 0; lr < L_; lr++) {
        ka.sendcopy_off[lr] = off;
        off += align_up(ka.sendcopy_bytes[lr], 256);
      }
    }
    if (n <= (size_t)kInlineMeta) {
      ka.flags |= CALL_META_INLINE;
      for (size_t i = 0; i < n; i++) {
        ka.inl.sendcounts[i] = ca.sendcounts[i];
        ka.inl.recvcounts[i] = ca.recvcounts ? ca.recvcounts[i] : -1;
        ka.inl.sdispls[i] = ca.sdispls[i];
        ka.inl.rdispls[i] = ca.rdispls[i];
      }
    } else if (persistent) {
      // a prepared call owns a device copy of its count arrays
      const size_t need = n * (4 + 4 + 8 + 8);
      std::vector<char> h(need);
      long long* h_sd = reinterpret_cast<long long*>(h.data());
      long long* h_rd = h_sd + n;
      int* h_sc = reinterpret_cast<int*>(h_rd + n);
      int* h_rc = h_sc + n;
      for (size_t i = 0; i < n; i++) {
        h_sd[i] = ca.sdispls[i]; h_rd[i] = ca.rdispls[i];
        h_sc[i] = ca.sendcounts[i]; h_rc[i] = ca.recvcounts ? ca.recvcounts[i] : -1;
      }
      RBV_CUDA_THROW(cudaMalloc(&out->owned_meta, need));
      RBV_CUDA_THROW(cudaMemcpy(out->owned_meta, h.data(), need, cudaMemcpyHostToDevice));
      long long* d_sd = reinterpret_cast<long long*>(out->owned_meta);
      int* d_sc = reinterpret_cast<int*>(d_sd + 2 * n);
      ka.sdispls = d_sd; ka.rdispls = d_sd + n;
      ka.sendcounts = d_sc; ka.recvcounts = d_sc + n;
    } else {
      const size_t need = n * (4 + 4 + 8 + 8);
      if (need > ring_bytes_) {
        for (int i = 0; i < kRing; i++) {
          if (ring_ev_[i]) cudaEventSynchronize(ring_ev_[i]);
          if (ring_host_[i]) cudaFreeHost(ring_host_[i]);
          if (ring_dev_[i]) cudaFree(ring_dev_[i]);
          RBV_CUDA_THROW(cudaHostAlloc(&ring_host_[i], need, cudaHostAllocDefault));
          RBV_CUDA_THROW(cudaMalloc(&ring_dev_[i], need));
          if (!ring_ev_[i]) RBV_CUDA_THROW(cudaEventCreateWithFlags(&ring_ev_[i], cudaEventDisableTiming));
        }
        ring_bytes_ = need;
      }
      const int slot = ring_next_;
      ring_next_ = (ring_next_ + 1) % kRing;
      RBV_CUDA_THROW(cudaEventSynchronize(ring_ev_[slot]));
      char* h = ring_host_[slot];
      long long* h_sd = reinterpret_cast<long long*>(h);
      long long* h_rd = h_sd + n;
      int* h_sc = reinterpret_cast<int*>(h_rd + n);
      int* h_rc = h_sc + n;
      for (size_t i = 0; i < n; i++) {
        h_sd[i] = ca.sdispls[i]; h_rd[i] = ca.rdispls[i];
        h_sc[i] = ca.sendcounts[i]; h_rc[i] = ca.recvcounts ? ca.recvcounts[i] : -1;
      }
      RBV_CUDA_THROW(cudaMemcpyAsync(ring_dev_[slot], h, need, cudaMemcpyHostToDevice, stream));
      RBV_CUDA_THROW(cudaEventRecord(ring_ev_[slot], stream));
      long long* d_sd = reinterpret_cast<long long*>(ring_dev_[slot]);
      int* d_sc = reinterpret_cast<int*>(d_sd + 2 * n);
      ka.sdispls = d_sd;
      ka.rdispls = d_sd + n;
      ka.sendcounts = d_sc;
      ka.recvcounts = d_sc + n;
    }
  } else {
    ka.sendcounts = ca.sendcounts; ka.recvcounts = ca.recvcounts;
    ka.sdispls = ca.sdispls; ka.rdispls = ca.rdispls;
  }

  // --- launch shape ---
  // Bytes this process moves, counting forwarded hops (a relay moves other ranks' blocks of
  // about the same size).
  double hop_factor = dp->nops > 0 ? (double)dp->nops / (double)((size_t)L_ * P_) : 1.0;
  double work = send_bytes >= 0 ? (double)send_bytes * std::max(1.0, hop_factor) : -1.0;
  unsigned long long chunk = opt.chunk_bytes;
  int grid = opt.grid;
  const int warps_per_cta = kThreads / 32;
  // Bulk-copy engine: worth its shared memory (one CTA per SM) once every warp has at least 16 KB to move.  Its
  // loads must read this GPU's own memory, so send buffers in host memory keep the vector path.
  bool bulk = false;
  if (!eager && bulk_mode_ != 0 && bulk_ctas_ > 0) {
    const bool want = bulk_mode_ > 0 || (work >= 0 && work / (1.0 * bulk_ctas_ * warps_per_cta) >= 16.0 * 1024);
    if (want) {
      bulk = true;
      for (int lr = 0; lr < L_ && bulk && !inplace; lr++) {
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, ca.sendbufs[lr]) != cudaSuccess || at.type != cudaMemoryTypeDevice ||
            at.device != device_) {
          (void)cudaGetLastError();
          bulk = false;
        }
      }
    }
  }
  const int max_ctas = bulk ? bulk_ctas_ : max_ctas_;
  if (bulk) ka.flags |= CALL_BULK;
  if (!chunk) {
    if (work < 0) chunk = 32 << 10;
    else {
      // a chunk is one warp's unit of work, at most 64 KB and at least 2 KB.  Chunks are dealt to the resident
      // warps in turn, so the byte count is cut into a whole number of rounds: with 64 KB chunks and 1.8 rounds,
      // a tenth of the warps would work alone at the end.  Measured on B200: with fewer, larger chunks most warps
      // idle and a 4 MB exchange takes twice as long.
      const double warps = 1.0 * max_ctas * warps_per_cta;
      const double rounds = std::max(1.0, std::ceil(work / (warps * 64.0 * 1024)));
      const double c = work / (warps * rounds);
      chunk = (unsigned long long)std::min(64.0 * 1024, std::max(bulk ? 4.0 * 1024 : 2.0 * 1024, c));
      chunk = align_up(chunk, bulk ? 4096 : 1024);
    }
  }
  chunk = align_up(chunk, 16);
  if (grid <= 0) {
    if (work < 0) grid = max_ctas;
    else {
      double chunks = work / (double)chunk + dp->nops;
      grid = (int)std::min<double>(max_ctas, std::max<double>(1.0, std::ceil(chunks / warps_per_cta)));
    }
  }
  grid = std::max(1, std::min(grid, max_ctas));
  ka.chunk_bytes = chunk;
  out->grid = grid;
  out->eager = eager;
  // A direct schedule has no CTA that waits for another CTA of the same grid (the final wait of CTA 0 holds no one
  // up), so it does not need the residency guarantee of a cooperative launch.
  out->cooperative = dp->plan.ncells > 0 || inplace;
  if (eager) {
    ka.ops = dp->d_eops;
    ka.nops = dp->n_eops;
    ka.eager_payload = emax;
    // Work items: one warp per chunk of payload; relay and unpack items are sized by the cell (or by the largest
    // block this process knows of).  Small chunks win (measured on 8 x B200: 512-byte chunks beat larger ones
    // from 16 B to 64 KB blocks) as long as all items fit the resident warps at once.
    long long mx = (long long)emax;
    if (!ca.counts_on_device) {
      mx = 0;
      for (size_t i = 0; i < n; i++) {
        mx = std::max<long long>(mx, (long long)ca.sendcounts[i] * ts);
        if (ca.recvcounts) mx = std::max<long long>(mx, (long long)ca.recvcounts[i] * ts);
      }
      mx = std::max<long long>(mx, 1);
    }
    // exact item count for a chunk size: first hops by their own size, unpacks by the receiver's recvcount,
    // relays by the largest block
    auto count_items = [&](unsigned long long ch) {
      double items = 0;
      for (const Op& o : dp->h_eops) {
        const int lr = o.src - proc_ * L_;
        long long bytes = mx;
        if (!ca.counts_on_device) {
          if (o.flags & 2u) { if (ca.recvcounts) bytes = (long long)ca.recvcounts[(size_t)lr * P_ + o.origin] * ts; }
          else if (o.src_cell < 0) bytes = (long long)ca.sendcounts[(size_t)lr * P_ + o.dest] * ts;
        }
        items += std::max(1.0, std::ceil((double)bytes / (double)ch));
      }
      return items;
    };
    unsigned long long ech = opt.chunk_bytes ? align_up(opt.chunk_bytes, 16) : 512;
    double items = count_items(ech);
    if (!opt.chunk_bytes)
      while (items > (double)max_ctas_ * warps_per_cta && ech < 8192) {
        ech *= 2;
        items = count_items(ech);
      }
    ka.chunk_bytes = ech;
    // A persistent call with host-side counts knows every item in advance: the table spares the kernel its sizing
    // pass (two block-wide barriers and a scan before the first byte moves).  Same rule as the kernel's own pass.
    if (persistent && !ca.counts_on_device && items < 1e6) {
      std::vector<EagerItem> tab;
      tab.reserve((size_t)items);
      bool fits = true;
      for (size_t oi = 0; fits && oi < dp->h_eops.size(); oi++) {
        const Op& o = dp->h_eops[oi];
        const int lr = o.src - proc_ * L_;
        unsigned long long b;
        if (o.flags & 2u) {
          const long long cap = ca.recvcounts ? (long long)ca.recvcounts[(size_t)lr * P_ + o.origin] : -1;
          b = cap >= 0 ? std::min<unsigned long long>((unsigned long long)cap * ts, emax) : emax;
        } else if (o.src_cell < 0) {
          b = (unsigned long long)ca.sendcounts[(size_t)lr * P_ + o.dest] * ts;
        } else {
          b = emax;
        }
        const unsigned long long nch = std::max<unsigned long long>(1, (b + ech - 1) / ech);
          for (unsigned long long k = 0; k < nch; k++) tab.push_back(EagerItem{o, (unsigned)k, (unsigned)oi});
      }
      if (fits && !tab.empty()) {
        RBV_CUDA_THROW(cudaMalloc(&out->owned_items, tab.size() * sizeof(EagerItem)));
        RBV_CUDA_THROW(cudaMemcpy(out->owned_items, tab.data(), tab.size() * sizeof(EagerItem), cudaMemcpyHostToDevice));
        ka.items = static_cast<const EagerItem*>(out->owned_items);
        ka.nitems = (unsigned)tab.size();
        std::memcpy(ka.inl_items, tab.data(), std::min(tab.size(), (size_t)kInlineEagerItems) * sizeof(EagerItem));
        items = (double)tab.size();
      }
    }
    const bool spread = eager_spread_ != 0 && ka.items != nullptr && opt.grid <= 0;
    if (spread) ka.flags |= CALL_SPREAD;
    int g = opt.grid > 0 ? opt.grid
                         : (int)std::min<double>(max_ctas_, std::max(1.0, spread ? items : std::ceil(items / warps_per_cta)));
    out->grid = std::max(1, std::min(g, max_ctas_));
    // Items wait for units that other items send.  A sender never waits, and items are listed senders first, so a
    // grid that covers all items in one round cannot block itself as long as CTAs start in index order; with one
    // rank per GPU and no relay hops every wait is for another GPU anyway.  Everything else is launched cooperatively.
    out->cooperative = !((L_ == 1 && dp->plan.ncells == 0) || items <= (double)out->grid * warps_per_cta);
  }
  return 0;
}

namespace {
// Chunk size of the rendezvous copy loops for `work` bytes moved by one process (forwarded hops included): a chunk
// is one warp's unit of work, at most 64 KB and at least 2 KB.  Chunks are dealt to the resident warps in turn, so
// the byte count is cut into a whole number of rounds: with 64 KB chunks and 1.8 rounds a tenth of the warps would
// work alone at the end.  Measured on B200: with fewer, larger chunks most warps idle and a 4 MB exchange takes
// twice as long.
unsigned long long chunk_for(double work, int max_ctas) {
  const double warps = 1.0 * max_ctas * (kThreads / 32);
  const double rounds = std::max(1.0, std::ceil(work / (warps * 64.0 * 1024)));
  const double c = work / (warps * rounds);
  unsigned long long chunk = (unsigned long long)std::min(64.0 * 1024, std::max(2.0 * 1024, c));
  return align_up(chunk, 1024);
}
}  // namespace

int Context::prepare_static(const DevPlan* dp, int ts, const CallArgs& ca, const CallOptions& opt, Prepared* out) {
  const int P = P_, L = L_, first = proc_ * L_;
  // ---- the communicator-wide tables ----
  std::vector<int> own_counts, own_caps;
  std::vector<long long> own_rd;
  std::vector<unsigned long long> own_ro;
  const int* gc = ca.g_counts;
  const int* gcap = ca.g_caps;
  const long long* grd = ca.g_rdispls;
  const unsigned long long* gro = ca.g_recvoff;
  if (!gc) {   // this process hosts every rank
    own_counts.assign(ca.sendcounts, ca.sendcounts + (size_t)P * P);
    own_rd.assign(ca.rdispls, ca.rdispls + (size_t)P * P);
    own_ro.resize(P);
    for (int d = 0; d < P; d++) own_ro[d] = (unsigned long long)(static_cast<char*>(ca.recvbufs[d]) - heap_);
    if (ca.recvcounts) { own_caps.assign(ca.recvcounts, ca.recvcounts + (size_t)P * P); gcap = own_caps.data(); }
    gc = own_counts.data(); grd = own_rd.data(); gro = own_ro.data();
  }
  long long maxcount = 0;
  for (size_t i = 0; i < (size_t)P * P; i++) {
    if (gc[i] < 0 || grd[i] < 0) { last_error_ = "negative count or displacement"; return RBV_ERR_BAD_ARG; }
    maxcount = std::max<long long>(maxcount, gc[i]);
  }
  for (size_t i = 0; i < (size_t)L * P; i++)
    if (ca.sdispls[i] < 0) { last_error_ = "negative count or displacement"; return RBV_ERR_BAD_ARG; }
  if (gcap)
    for (int s = 0; s < P; s++)
      for (int d = 0; d < P; d++)
        if (gcap[(size_t)d * P + s] >= 0 && gc[(size_t)s * P + d] > gcap[(size_t)d * P + s]) {
          last_error_ = "block " + std::to_string(s) + " -> " + std::to_string(d) + " is larger than the receiver's recvcount";
          return RBV_ERR_TRUNCATE;
        }
  const bool anywhere = nproc_ == 1 && opt.recv_anywhere;   // no peers, extents checked by the caller
  for (int d = 0; d < P && !anywhere; d++) {
    unsigned long long ext = 0;
    for (int s = 0; s < P; s++)
      ext = std::max(ext, (unsigned long long)(grd[(size_t)d * P + s] + gc[(size_t)s * P + d]) * ts);
    if (gro[d] < lay_.user_off || gro[d] + ext > lay_.total_bytes) {
      last_error_ = "receive buffer of rank " + std::to_string(d) + " does not fit inside the symmetric heap";
      return RBV_ERR_BAD_ARG;
    }
  }
  const size_t stride = align_up((size_t)maxcount * ts, 16);
  const int ncells = dp->plan.ncells;
  if (ncells > 0 && stride * (size_t)ncells > lay_.arena_bytes) {
    last_error_ = "staging arena too small: " + std::to_string(ncells) + " cells of " + std::to_string(stride) + " bytes";
    return RBV_ERR_CAPACITY;
  }
  auto slice_bytes = [&](const Op& o, long long* first_el) {
    long long f = 0, n = 0;
    op_slice(o, gc[(size_t)o.origin * P + o.dest], &f, &n);
    if (first_el) *first_el = f;
    return (unsigned long long)n * ts;
  };
  // ---- chunk size: the same on every process (receivers count chunks), so it is derived from the busiest process ----
  unsigned long long chunk = opt.chunk_bytes;
  if (!chunk) {
    std::vector<double> work(nproc_, 0.0);
    for (const Op& o : dp->plan.ops) work[o.src / L] += (double)slice_bytes(o, nullptr);
    chunk = chunk_for(*std::max_element(work.begin(), work.end()), static_max_ctas_);
  }
  chunk = align_up(chunk, 16);
  const unsigned long long fpc = ncells > 0 ? lay_.flags_per_rank / (unsigned long long)ncells : 0;
  if (ncells > 0) chunk = std::max<unsigned long long>(chunk, align_up((stride + fpc - 1) / fpc, 16));
  if (chunk > 0xffffffffull) chunk = 0xfffffff0ull;
  auto nchunks = [&](unsigned long long bytes) { return (bytes + chunk - 1) / chunk; };

  // ---- items of this process: plan order.  Across GPUs the chunks of the ops of one key alternate, so that a rank
  // writes to all peers of a round at once (with one block after the other, two senders meet at one receiver while
  // another receiver idles as soon as block sizes differ).  Inside one GPU the copies are bound by HBM, where
  // walking block after block measured 4-8 % faster than alternating (better DRAM page locality). ----
  const bool alternate = nproc_ > 1;
  std::vector<StaticItem> items;
  const std::vector<Op>& ops = dp->h_ops;
  auto stage_addr = [&](int proc, int lr, int cell) {
    return reinterpret_cast<unsigned long long>(peer_[proc]) + lay_.stage_off + (unsigned long long)(lr * 2) * lay_.arena_bytes +
           (unsigned long long)cell * stride;
  };
  for (size_t g0 = 0; g0 < ops.size();) {
    size_t g1 = g0;
    while (g1 < ops.size() && ops[g1].key == ops[g0].key) g1++;
    unsigned long long maxn = 0;
    for (size_t i = g0; i < g1; i++) maxn = std::max(maxn, nchunks(slice_bytes(ops[i], nullptr)));
    // (outer, inner) = (chunk, op) when alternating, (op, chunk) otherwise
    const unsigned long long n_outer = alternate ? maxn : (unsigned long long)(g1 - g0);
    const unsigned long long n_inner = alternate ? (unsigned long long)(g1 - g0) : maxn;
    for (unsigned long long outer = 0; outer < n_outer; outer++)
      for (unsigned long long inner = 0; inner < n_inner; inner++) {
        const unsigned long long k = alternate ? outer : inner;
        const size_t i = g0 + (size_t)(alternate ? inner : outer);
        const Op& o = ops[i];
        long long f = 0;
        const unsigned long long bytes = slice_bytes(o, &f);
        if (k >= nchunks(bytes)) continue;
        const int lsrc = o.src - first, dproc = o.dst / L, ldst = o.dst - dproc * L;
        const unsigned long long off = k * chunk;
        StaticItem it{};
        it.len = (unsigned)std::min<unsigned long long>(chunk, bytes - off);
        it.dst_rank = o.dst;
        unsigned fl = 0;
        if (o.src_cell < 0) {
          it.src = reinterpret_cast<unsigned long long>(ca.sendbufs[lsrc]) +
                   (unsigned long long)(ca.sdispls[(size_t)lsrc * P + o.dest] + f) * ts + off;
          it.wait_flag = kNoFlag;
        } else {
          it.src = stage_addr(proc_, lsrc, o.src_cell) + off;
          it.wait_flag = (unsigned)((unsigned long long)lsrc * lay_.flags_per_rank + (unsigned long long)o.src_cell * fpc + k);
          fl |= ITEM_SRC_STAGE;
        }
        if (o.dst_cell < 0) {
          it.dst = reinterpret_cast<unsigned long long>(peer_[dproc]) + gro[o.dst] +
                   (unsigned long long)(grd[(size_t)o.dst * P + o.origin] + f) * ts + off;
          it.signal_flag = kNoFlag;
        } else {
          it.dst = stage_addr(dproc, ldst, o.dst_cell) + off;
          it.signal_flag = (unsigned)((unsigned long long)ldst * lay_.flags_per_rank + (unsigned long long)o.dst_cell * fpc + k);
          fl |= ITEM_DST_STAGE;
        }
        if (dproc != proc_) fl |= ITEM_REMOTE;
        if (o.flags & kOpSelf) fl |= ITEM_SELF;
        it.flags = (unsigned short)(fl | (std::min<unsigned>(op_key_index(o), 255u) << 8));
        items.push_back(it);
      }
    g0 = g1;
  }
  // chunks that land in the receive buffers of this process's ranks, from every process
  std::vector<unsigned long long> expect(L, 0);
  for (const Op& o : dp->plan.ops)
    if (o.dst_cell < 0 && o.dst / L == proc_) expect[o.dst - first] += nchunks(slice_bytes(o, nullptr));

  // blocks to copy on to the caller's own buffers once everything has arrived (pieces of at most 64 KB, so that
  // the warps of the copying CTA share a large block)
  std::vector<DrainItem> drain;
  if (ca.recv_mirror)
    for (int lr = 0; lr < L; lr++) {
      if (!ca.recv_mirror[lr] || ca.recv_mirror[lr] == ca.recvbufs[lr]) continue;
      const int d = first + lr;
      for (int s2 = 0; s2 < P; s2++) {
        const unsigned long long len = (unsigned long long)std::max(gc[(size_t)s2 * P + d], 0) * ts;
        const unsigned long long off = (unsigned long long)grd[(size_t)d * P + s2] * ts;
        for (unsigned long long o2 = 0; o2 < len; o2 += 64u << 10) {
          DrainItem di{};
          di.src = reinterpret_cast<unsigned long long>(ca.recvbufs[lr]) + off + o2;
          di.dst = reinterpret_cast<unsigned long long>(ca.recv_mirror[lr]) + off + o2;
          di.len = (unsigned)std::min<unsigned long long>(64u << 10, len - o2);
          drain.push_back(di);
        }
      }
    }

  // ---- device copy: [expect[L] | items | drain] ----
  const size_t head = align_up(sizeof(unsigned long long) * L, 32);
  const size_t items_bytes = std::max<size_t>(items.size(), 1) * sizeof(StaticItem);
  const size_t bytes = head + items_bytes + drain.size() * sizeof(DrainItem);
  std::vector<char> blob(bytes, 0);
  std::memcpy(blob.data(), expect.data(), sizeof(unsigned long long) * L);
  if (!items.empty()) std::memcpy(blob.data() + head, items.data(), items.size() * sizeof(StaticItem));
  if (!drain.empty()) std::memcpy(blob.data() + head + items_bytes, drain.data(), drain.size() * sizeof(DrainItem));
  RBV_CUDA_THROW(cudaMalloc(&out->owned_items, bytes));
  RBV_CUDA_THROW(cudaMemcpy(out->owned_items, blob.data(), bytes, cudaMemcpyHostToDevice));

  StaticArgs& sa = out->sa;
  std::memset(&sa, 0, sizeof sa);
  sa.P = P; sa.L = L; sa.nproc = nproc_; sa.proc = proc_;
  sa.flags = trace_ ? (unsigned)CALL_TRACE : 0u;
  sa.nitems = (unsigned)items.size();
  sa.expect = static_cast<const unsigned long long*>(out->owned_items);
  sa.items = reinterpret_cast<const StaticItem*>(static_cast<char*>(out->owned_items) + head);
  sa.drain = reinterpret_cast<const DrainItem*>(static_cast<char*>(out->owned_items) + head + items_bytes);
  sa.ndrain = (unsigned)drain.size();
  sa.timeout_ns = timeout_ns_;
  sa.lay = lay_;
  for (int q = 0; q < nproc_; q++) sa.heap[q] = peer_[q];
  sa.host_status = host_status_dev_;
  sa.host_trace = host_trace_dev_;
  std::memcpy(sa.inl, items.data(), std::min(items.size(), (size_t)kInlineItems) * sizeof(StaticItem));
  const int warps_per_cta = kThreads / 32;
  // One process: item c goes to warp c / grid of CTA c % grid (a2av_static.cu), so with one CTA per item (up to the
  // CTAs that are resident at once) a small call spreads over as many SMs as it has items instead of filling the 16
  // warps of a few.  Several processes: 16 items per CTA (see the kernel).
  const bool spread = static_spread_ && nproc_ == 1;
  int grid = opt.grid > 0 ? opt.grid
                          : (int)(spread ? items.size() : (items.size() + warps_per_cta - 1) / warps_per_cta);
  out->grid = std::max(1, std::min(grid, static_max_ctas_));
  out->is_static = true;
  out->eager = false;
  // Only items that forward a staged chunk wait for other items; those come later in the list than what they wait
  // for, on every process.  With one round of items per warp that order cannot block as long as CTAs start in index
  // order; several rounds per warp need all CTAs resident.
  out->cooperative = ncells > 0 && items.size() > (size_t)out->grid * warps_per_cta;
  return 0;
}

int Context::set_nvls_meta(void* self_ptr, void* mc_ptr, size_t bytes) {
  if (!self_ptr || !mc_ptr) { nvls_self_ = nvls_mc_ = nullptr; nvls_bytes_ = 0; return 0; }
  if (bytes < nvls_bytes_needed() || (reinterpret_cast<uintptr_t>(self_ptr) & 15) || (reinterpret_cast<uintptr_t>(mc_ptr) & 15)) {
    last_error_ = "NVLS metadata buffer too small or misaligned";
    return RBV_ERR_BAD_ARG;
  }
  nvls_self_ = static_cast<char*>(self_ptr); nvls_mc_ = static_cast<char*>(mc_ptr); nvls_bytes_ = bytes;
  return cudaMemset(nvls_self_, 0, nvls_bytes_needed()) == cudaSuccess ? 0 : RBV_ERR_BAD_ARG;
}

// ---- NVLS: the library's own multicast object (CUDA driver API) ---------------------------------------------
// The driver entry points are looked up at run time (cudaGetDriverEntryPoint), so the library loads on a machine
// without a driver (a build host) and needs libcudart only.
namespace {
struct DriverApi {
#define RBV_DRV(name) decltype(&::name) name = nullptr;
  RBV_DRV(cuGetErrorName) RBV_DRV(cuDeviceGetAttribute) RBV_DRV(cuMulticastGetGranularity) RBV_DRV(cuMulticastCreate)
  RBV_DRV(cuMemExportToShareableHandle) RBV_DRV(cuMemImportFromShareableHandle) RBV_DRV(cuMulticastAddDevice)
  RBV_DRV(cuMemGetAllocationGranularity) RBV_DRV(cuMemCreate) RBV_DRV(cuMulticastBindMem)
  RBV_DRV(cuMemAddressReserve) RBV_DRV(cuMemMap) RBV_DRV(cuMemSetAccess) RBV_DRV(cuMemUnmap)
  RBV_DRV(cuMemAddressFree) RBV_DRV(cuMulticastUnbind) RBV_DRV(cuMemRelease)
#undef RBV_DRV
  bool ok = false;
  std::string missing;
};

template <typename F>
bool drv_lookup(const char* name, F* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    cudaGetLastError();
    return false;
  }
  *out = reinterpret_cast<F>(p);
  return true;
}

const DriverApi& drv() {
  static DriverApi d = [] {
    DriverApi a;
    bool ok = true;
#define RBV_DRV(name) if (!drv_lookup(#name, &a.name)) { ok = false; a.missing += std::string(a.missing.empty() ? "" : ", ") + #name; }
    RBV_DRV(cuGetErrorName) RBV_DRV(cuDeviceGetAttribute) RBV_DRV(cuMulticastGetGranularity) RBV_DRV(cuMulticastCreate)
    RBV_DRV(cuMemExportToShareableHandle) RBV_DRV(cuMemImportFromShareableHandle) RBV_DRV(cuMulticastAddDevice)
    RBV_DRV(cuMemGetAllocationGranularity) RBV_DRV(cuMemCreate) RBV_DRV(cuMulticastBindMem)
    RBV_DRV(cuMemAddressReserve) RBV_DRV(cuMemMap) RBV_DRV(cuMemSetAccess) RBV_DRV(cuMemUnmap)
    RBV_DRV(cuMemAddressFree) RBV_DRV(cuMulticastUnbind) RBV_DRV(cuMemRelease)
#undef RBV_DRV
    a.ok = ok;
    return a;
  }();
  return d;
}

const char* cu_name(CUresult r) {
  const char* s = nullptr;
  if (drv().cuGetErrorName) drv().cuGetErrorName(r, &s);
  return s ? s : "unknown CUDA driver error";
}
}  // namespace
#define RBV_CU(expr)                                                              \
  do {                                                                            \
    if (!drv().ok) {                                                              \
      last_error_ = "CUDA driver entry points not found: " + drv().missing;       \
      return -1;                                                                  \
    }                                                                             \
    CUresult r__ = (drv().expr);                                                  \
    if (r__ != CUDA_SUCCESS) {                                                    \
      last_error_ = std::string(#expr) + " failed: " + cu_name(r__);              \
      return (int)r__;                                                            \
    }                                                                             \
  } while (0)

int Context::nvls_create(size_t bytes, int* fd_out) {
  int supported = 0;
  RBV_CU(cuDeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device_));
  if (!supported) { last_error_ = "this device does not support NVLink multicast"; return -1; }
  CUmulticastObjectProp prop{};
  prop.numDevices = (unsigned)nproc_;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  prop.size = bytes;
  size_t gran = 0;
  RBV_CU(cuMulticastGetGranularity(&gran, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED));
  prop.size = align_up(std::max<size_t>(bytes, 1), gran);
  CUmemGenericAllocationHandle mc = 0;
  RBV_CU(cuMulticastCreate(&mc, &prop));
  own_mc_handle_ = mc;
  own_mc_bytes_ = prop.size;
  int fd = -1;
  RBV_CU(cuMemExportToShareableHandle(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *fd_out = fd;
  return 0;
}

int Context::nvls_import(int fd, size_t bytes) {
  int supported = 0;
  RBV_CU(cuDeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device_));
  if (!supported) { last_error_ = "this device does not support NVLink multicast"; return -1; }
  CUmemGenericAllocationHandle mc = 0;
  RBV_CU(cuMemImportFromShareableHandle(&mc, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  own_mc_handle_ = mc;
  own_mc_bytes_ = bytes;   // the size process 0 rounded up
  return 0;
}

int Context::nvls_add_device() {
  if (!own_mc_handle_) { last_error_ = "no multicast object"; return -1; }
  RBV_CU(cuMulticastAddDevice(own_mc_handle_, device_));
  return 0;
}

int Context::nvls_bind_and_map(void** self_ptr, void** mc_ptr, size_t* bytes_out) {
  if (!own_mc_handle_) { last_error_ = "no multicast object"; return -1; }
  CUmemAllocationProp ap{};
  ap.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  ap.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  ap.location.id = device_;
  ap.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;   // the same kind as the multicast object's
  size_t gran = 0;
  RBV_CU(cuMemGetAllocationGranularity(&gran, &ap, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  const size_t size = own_mc_bytes_;
  if (size % gran) { last_error_ = "multicast size is not a multiple of the allocation granularity"; return -1; }
  CUmemGenericAllocationHandle mem = 0;
  RBV_CU(cuMemCreate(&mem, size, &ap, 0));
  own_mem_handle_ = mem;
  RBV_CU(cuMulticastBindMem(own_mc_handle_, 0, mem, 0, size, 0));
  own_mc_bound_ = true;
  CUmemAccessDesc acc{};
  acc.location = ap.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CUdeviceptr va = 0, mva = 0;
  RBV_CU(cuMemAddressReserve(&va, size, gran, 0, 0));
  own_va_ = va;
  RBV_CU(cuMemMap(va, size, 0, mem, 0));
  RBV_CU(cuMemSetAccess(va, size, &acc, 1));
  RBV_CU(cuMemAddressReserve(&mva, size, gran, 0, 0));
  own_mc_va_ = mva;
  RBV_CU(cuMemMap(mva, size, 0, own_mc_handle_, 0));
  RBV_CU(cuMemSetAccess(mva, size, &acc, 1));
  *self_ptr = reinterpret_cast<void*>(va);
  *mc_ptr = reinterpret_cast<void*>(mva);
  *bytes_out = size;
  return 0;
}

void Context::nvls_teardown() {
  if (!own_mc_handle_) return;
  cudaDeviceSynchronize();
  nvls_self_ = nvls_mc_ = nullptr;
  nvls_bytes_ = 0;
  const DriverApi& d = drv();   // complete, or no object could have been made
  if (own_mc_va_) { d.cuMemUnmap(own_mc_va_, own_mc_bytes_); d.cuMemAddressFree(own_mc_va_, own_mc_bytes_); }
  if (own_va_) { d.cuMemUnmap(own_va_, own_mc_bytes_); d.cuMemAddressFree(own_va_, own_mc_bytes_); }
  if (own_mc_bound_) d.cuMulticastUnbind(own_mc_handle_, device_, 0, own_mc_bytes_);
  if (own_mem_handle_) d.cuMemRelease(own_mem_handle_);
  d.cuMemRelease(own_mc_handle_);
  own_mc_handle_ = own_mem_handle_ = own_va_ = own_mc_va_ = 0;
  own_mc_bound_ = false;
}
#undef RBV_CU

StatusBlock Context::status(cudaStream_t stream) {
  cudaStreamSynchronize(stream);
  StatusBlock s = *host_status_;
  host_status_->code = 0;   // errors are sticky until they have been read once
  return s;
}

cudaError_t Context::reset() {
  cudaError_t e = cudaSetDevice(device_);
  if (e != cudaSuccess) return e;
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return e;
  e = clear_library_regions();
  if (e != cudaSuccess) return e;
  if (nvls_self_) cudaMemset(nvls_self_, 0, nvls_bytes_needed());
  for (auto& kv : plans_)
    if (kv.second->d_done) cudaMemset(kv.second->d_done, 0, kv.second->nops * sizeof(unsigned));
  std::memset(host_status_, 0, sizeof(StatusBlock));
  std::memset(host_trace_, 0, sizeof(TraceBlock));
  host_seq_ = 0;
  return cudaDeviceSynchronize();
}

}  // namespace rbv
