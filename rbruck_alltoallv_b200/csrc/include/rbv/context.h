// Host runtime: one Context per process (one GPU).  It owns the symmetric heap, the peer mappings
// obtained through CUDA IPC, the device copies of compiled plans and the call sequence number.
// It stands in for what the MPI runtime and MPI_Comm_split provide in the reference
// (groups are index arithmetic on ranks; no sub-communicator is ever created).
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <string>
#include <tuple>
#include <vector>

#include "rbv/device_types.h"
#include "rbv/plan.h"

namespace rbv {

struct DevPlan {
  Plan plan;               // host copy (all ranks)
  Op* d_ops = nullptr;     // ops of this process's ranks
  std::vector<Op> h_ops;   // host copy of the same list
  bool has_parts = false;  // some block travels in slices (split_alltoallv)
  unsigned* d_done = nullptr;
  int nops = 0;
  // eager protocol: the same ops retargeted at arrival / staging cells, followed by one unpack op per
  // (local rank, source); cell indices: 0..P-1 arrival cell of source s, P + c staging cell c
  Op* d_eops = nullptr;
  int n_eops = 0;
  std::vector<Op> h_eops;  // host copy (sizing of work items per call)
};

struct CallOptions {
  int grid = 0;                       // CTAs; 0 = choose
  unsigned long long chunk_bytes = 0; // 0 = choose
  unsigned flags = 0;                 // CALL_INPLACE
  unsigned long long eager_max_bytes = 0;  // > 0: eager protocol with cells of this payload size (same on all ranks)
  bool allow_static = true;           // persistent calls with host-side counts may resolve everything on the host
  bool recv_anywhere = false;         // the caller has checked the receive extents itself: a static call of a
                                      // single process may then receive into any device-accessible memory
};

// Arguments of one collective call for all L local ranks.  Count arrays are [L][P].
struct CallArgs {
  const void* const* sendbufs = nullptr;   // [L] device pointers (ignored for in-place calls)
  void* const* recvbufs = nullptr;         // [L] device pointers inside the symmetric heap
  void* const* recv_mirror = nullptr;      // [L] or null: where the caller wants each rank's received blocks in the end
                                           // (any device-accessible memory; static calls copy them there in the kernel)
  const int* sendcounts = nullptr;
  const int* recvcounts = nullptr;         // may be null
  const long long* sdispls = nullptr;
  const long long* rdispls = nullptr;
  bool counts_on_device = false;           // the four arrays are device memory
  long long bytes_hint = -1;               // total bytes sent by this process, if known (device counts)
  // The whole communicator's arguments, when the caller has gathered them on the host (all null otherwise):
  // g_counts[s * P + d] = sendcounts of rank s, g_caps[d * P + s] = recvcounts of rank d (-1: unchecked; the array
  // may be null), g_rdispls[d * P + s], g_recvoff[d] = offset of rank d's receive buffer in its process's heap.
  // A process that hosts every rank needs none of them: its own arguments are the whole picture.
  const int* g_counts = nullptr;
  const int* g_caps = nullptr;
  const long long* g_rdispls = nullptr;
  const unsigned long long* g_recvoff = nullptr;
};

// A fully resolved call: launching it again repeats the collective with the same buffers and counts
// (the call number lives in device memory, so nothing in here changes between launches).
struct Prepared {
  KernelArgs ka;
  int grid = 1;
  bool eager = false;
  bool is_static = false;       // runs the static kernel with `sa`; `ka` is unused then
  bool cooperative = true;      // launch mode this call needs (false: a plain launch is safe)
  StaticArgs sa;
  void* owned_meta = nullptr;   // device copy of host count arrays that did not fit the kernel parameters
  void* owned_items = nullptr;  // device copy of the precomputed work-item table (eager protocol)
};

class Context {
 public:
  Context(int P, int nproc, int proc, int device, size_t user_bytes, size_t arena_bytes);
  ~Context();
  Context(const Context&) = delete;

  int P() const { return P_; }
  int L() const { return L_; }
  int nproc() const { return nproc_; }
  int proc() const { return proc_; }
  int device() const { return device_; }
  const HeapLayout& layout() const { return lay_; }
  char* heap() const { return heap_; }
  char* peer_heap(int q) const { return peer_[q]; }
  int max_ctas() const { return max_ctas_; }
  int sm_count() const { return sm_count_; }

  cudaError_t ipc_handle(void* out64);
  cudaError_t connect(const void* handles);  // nproc x 64 bytes, in process order

  void* symm_alloc(size_t bytes);
  int symm_free(void* p);
  bool in_heap(const void* p, size_t bytes) const;

  // Launches the collective on `stream`.  Returns 0, the plan's error code (< 0), or a positive
  // Status for argument errors detected on the host.  Device-side errors are reported by status().
  int alltoallv(const AlgoSpec& spec, int type_size, const CallArgs& args, const CallOptions& opt,
                cudaStream_t stream);

  // The two halves of alltoallv(): resolve everything once, launch many times (the analogue of MPI's
  // persistent collectives).  `persistent` makes the call own a device copy of large host count arrays.
  int prepare(const AlgoSpec& spec, int type_size, const CallArgs& args, const CallOptions& opt,
              cudaStream_t stream, bool persistent, Prepared* out);
  int launch(const Prepared& pc, cudaStream_t stream);
  void release(Prepared& pc);
  // Cooperative launches guarantee that all CTAs are resident; a plain launch is a little cheaper.  Default (-1):
  // cooperative only for calls in which a CTA may wait for work of a later CTA of the same grid (store-and-forward
  // schedules with more items than resident warps); 1: always; 0: never, except for in-place calls, whose grid-wide
  // barrier needs it.  RBV_COOPERATIVE=0/1 sets the same.
  void set_cooperative(int mode) { cooperative_mode_ = mode; }
  // Copy the phase time stamps to the host after every call (off: only failing calls report).
  void set_trace(bool on) { trace_ = on; }
  // Bulk-copy engine for large chunks: 0 = never (default), 1 = whenever the buffers allow it, -1 = by size
  // (16 KB or more per warp).  Measured on B200 it moves data as fast as the vector path (same HBM copy rate
  // on one GPU, 0.97x over NVLink at 128 MB blocks), so it is an option rather than the default.
  void set_bulk(int mode) { bulk_mode_ = mode; }

  // First error since the last status() call (0 if none); synchronises `stream` first.
  StatusBlock status(cudaStream_t stream);
  // Per-key time stamps of the most recent traced call (valid after status() has synchronised), and the plan
  // that call ran (null before the first call).
  const TraceBlock& last_trace() const { return *host_trace_; }
  const DevPlan* last_plan() const { return last_plan_; }
  double last_plan_build_s() const { return last_plan_build_s_; }
  // Clears all synchronisation state.  Every process must call it between the same two calls,
  // with a host barrier before and after.
  cudaError_t reset();
  void set_timeout_ns(unsigned long long ns) { timeout_ns_ = ns; }
  unsigned long long timeout_ns() const { return timeout_ns_; }
  // Fault injection for tests: the given local rank skips its metadata row in the next calls (-1: off).
  void set_absent_rank(int lr) { absent_rank_ = lr; }
  // NVLS: metadata tables in an externally provided multicast-capable buffer (local address, multicast address,
  // size).  Every process must set it, or none.  Null pointers switch back to the tables inside the heap.
  int set_nvls_meta(void* self_ptr, void* mc_ptr, size_t bytes);
  // Bytes an NVLS buffer must have: two metadata tables and the arrival counters of the auxiliary barriers.
  size_t nvls_bytes_needed() const { return nvls_aux_off() + 256; }
  size_t nvls_aux_off() const { return (2 * (size_t)lay_.meta_bytes + 255) & ~(size_t)255; }
  // Arrival counters of the auxiliary barriers (MoE dispatch / combine, transpose) inside the NVLS buffer: this
  // GPU's copy and the multicast address that reaches every GPU's copy; null when NVLS is off.
  unsigned long long* nvls_aux_self() const {
    return nvls_mc_ ? reinterpret_cast<unsigned long long*>(nvls_self_ + nvls_aux_off()) : nullptr;
  }
  unsigned long long* nvls_aux_mc() const {
    return nvls_mc_ ? reinterpret_cast<unsigned long long*>(nvls_mc_ + nvls_aux_off()) : nullptr;
  }
  // NVLS set-up done by the library itself (CUDA driver API): an NVLink multicast object over one buffer per GPU.
  // Collective, in four steps with a host barrier after each: (1) process 0 creates the object and exports it as a
  // file descriptor, which the caller hands to the other processes (SCM_RIGHTS over a Unix socket); (2) every
  // process imports it (process 0 skips this) and adds its device; (3) every process allocates its physical buffer,
  // binds it to the object and maps both the buffer and the multicast view; (4) set_nvls_meta() with the two
  // addresses.  Each returns 0 or a CUDA driver error code (last_error() has the text).
  int nvls_create(size_t bytes, int* fd_out);
  int nvls_import(int fd, size_t bytes);
  int nvls_add_device();
  int nvls_bind_and_map(void** self_ptr, void** mc_ptr, size_t* bytes_out);
  void nvls_teardown();
  size_t nvls_object_bytes() const { return own_mc_bytes_; }
  const std::string& last_error() const { return last_error_; }
  const DevPlan* plan_for(const AlgoSpec& spec);

 private:
  int P_, L_, nproc_, proc_, device_;
  HeapLayout lay_{};
  char* heap_ = nullptr;
  char* peer_[kMaxProcs] = {};
  bool opened_[kMaxProcs] = {};
  int cooperative_mode_ = -1;
  cudaError_t clear_library_regions();
  bool trace_ = false;
  int bulk_mode_ = 0;
  int bulk_ctas_ = 0;
  int absent_rank_ = -1;
  char* nvls_self_ = nullptr;
  char* nvls_mc_ = nullptr;
  size_t nvls_bytes_ = 0;
  // own multicast object (0: none, or the buffer came from the caller)
  unsigned long long own_mc_handle_ = 0, own_mem_handle_ = 0, own_va_ = 0, own_mc_va_ = 0;
  size_t own_mc_bytes_ = 0;
  bool own_mc_bound_ = false;
  unsigned long long timeout_ns_ = 2000000000ull;
  int max_ctas_ = 1, sm_count_ = 1;
  StatusBlock* host_status_ = nullptr;
  StatusBlock* host_status_dev_ = nullptr;
  TraceBlock* host_trace_ = nullptr;
  TraceBlock* host_trace_dev_ = nullptr;
  const DevPlan* last_plan_ = nullptr;
  double last_plan_build_s_ = 0;   // host time spent compiling the plan of the last prepare() (0: cached)
  unsigned host_seq_ = 0;          // the call number as the host counts it (every launch advances it once)
  bool seq_hints_ = true;          // off for good once a launch was recorded into a CUDA graph (or RBV_SEQ_HINT=0)
  int static_max_ctas_ = 1;
  int static_occ_ = 1;             // CTAs per SM the static kernel is built for (RBV_STATIC_OCC=2: the 64-register build)
  int eager_spread_ = 0;           // eager calls with a prepared item table: one CTA per item (RBV_EAGER_SPREAD=1);
                                   // off: measured on 2 GPUs it cost 1-2 us per call (16.8 against 15.0 us)
  bool static_spread_ = true;      // few items: one per CTA over many SMs instead of 16 per CTA on few (RBV_STATIC_SPREAD=0)
  int prepare_static(const DevPlan* dp, int type_size, const CallArgs& args, const CallOptions& opt, Prepared* out);
  std::string last_error_;
  std::map<std::tuple<int, int, int, int, int, int, int>, std::unique_ptr<DevPlan>> plans_;
  // free list of the user region: offset -> size
  std::map<size_t, size_t> free_;
  std::map<size_t, size_t> used_;
  // staging ring for host-side count arrays that do not fit in the kernel parameters
  static constexpr int kRing = 4;
  char* ring_host_[kRing] = {};
  char* ring_dev_[kRing] = {};
  cudaEvent_t ring_ev_[kRing] = {};
  size_t ring_bytes_ = 0;
  int ring_next_ = 0;
  // private copies for in-place calls
  void* sendcopy_ = nullptr;
  size_t sendcopy_bytes_ = 0;
};

// implemented in kernels/a2av_kernel.cu
size_t a2av_smem_bytes(int P);
size_t a2av_smem_bytes_bulk(int P);
int a2av_bulk_ctas_per_sm(int P);
cudaError_t a2av_configure(int P, int* max_ctas_per_sm);
cudaError_t a2av_launch(const KernelArgs& args, int grid, bool cooperative, cudaStream_t stream);
// implemented in kernels/a2av_static.cu
cudaError_t a2av_static_configure(int occupancy, int* max_ctas_per_sm);
cudaError_t a2av_static_launch(const StaticArgs& args, int grid, int occupancy, bool cooperative, cudaStream_t stream);
// implemented in kernels/a2av_eager.cu
cudaError_t a2av_eager_launch(const KernelArgs& args, int grid, bool cooperative, cudaStream_t stream);

}  // namespace rbv
