// Allocation-free alltoallv entry point (see rbv/noalloc.h for the contract and the reasons).
//
// All device scratch is the file-scope array `g_scratch`.  In host code that name is only a handle for
// the runtime: the device address is obtained once per device with cudaGetSymbolAddress and it is that
// address which is handed to the kernel.  Nothing here calls cudaMalloc / cudaFree or any routine that
// allocates (host containers included): the schedule is generated into fixed-size host arrays.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "rbv/context.h"
#include "rbv/device_types.h"
#include "rbv/noalloc.h"

namespace {

using namespace rbv;

constexpr int kNR = RBV_NOALLOC_MAX_RANKS;
constexpr int kMaxCellsNA = 5;                       // radix 2, 8 ranks: sum_j (popcount(j) - 1)
constexpr size_t kArena = (size_t)kMaxCellsNA * RBV_NOALLOC_MAX_BLOCK_BYTES;
constexpr int kMaxOpsNA = kNR * 13;                  // 12 hops + 1 self copy per rank

constexpr size_t align_up_c(size_t v, size_t a) { return (v + a - 1) / a * a; }
constexpr size_t kCtrlOff = 0;
constexpr size_t kTraceOff = align_up_c(sizeof(CtrlBlock), 256);
constexpr size_t kFlagsOff = kTraceOff + align_up_c(sizeof(TraceBlock), 256);
constexpr size_t kFlagsPerRank = 256;                // 5 staging cells x up to 51 chunk flags each
constexpr size_t kFlagsBytes = sizeof(unsigned) * 2ull * kNR * kFlagsPerRank;
constexpr size_t kMetaOff = kFlagsOff + kFlagsBytes;
constexpr size_t kMetaBytes = 3584;                  // >= meta_table_bytes(8)
constexpr size_t kClearBytes = align_up_c(kMetaOff + 2 * kMetaBytes, 256);   // starts at zero in every call
// schedules for every rank count 1..8, uploaded once per device; slot P - 1 holds kMaxOpsNA ops
constexpr size_t kOpsOff = kClearBytes;
constexpr size_t kOpsSlot = align_up_c(sizeof(Op) * kMaxOpsNA, 256);
constexpr size_t kStageOff = align_up_c(kOpsOff + kOpsSlot * kNR, 4096);
constexpr size_t kTotal = kStageOff + 2ull * kNR * kArena;
static_assert(kMetaBytes >= 48 * kNR * kNR + 16 * kNR, "metadata tables do not fit");
static_assert(kTotal <= RBV_NOALLOC_SCRATCH_BYTES, "scratch array too small for the stated limits");

// The one scratch array.  Device code may name it directly; host code must not use this name as an address.
static __device__ __align__(256) unsigned char g_scratch[RBV_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
struct DeviceState {
  bool ready;
  unsigned char* base;     // device address of g_scratch on that device
  int nops[kNR + 1], ncells[kNR + 1];   // per rank count
  int sm_count;
};
DeviceState g_dev[kMaxDevices];
std::mutex g_dev_mutex;    // guards the first-call set-up of a device against concurrent host threads
thread_local char g_msg[256];

int fail(int code, const char* what, cudaError_t e = cudaSuccess) {
  if (e != cudaSuccess) std::snprintf(g_msg, sizeof g_msg, "%s: %s", what, cudaGetErrorString(e));
  else std::snprintf(g_msg, sizeof g_msg, "%s", what);
  return code;
}

// Radix-2 low-digit-first Bruck schedule for P ranks into a fixed array (same ops as the plan compiler's
// "rbruck_om" with r = 2; the test compares the two paths).
int build_schedule(int P, Op* ops, int* ncells_out) {
  int cellid[kNR][3];
  int ncells = 0;
  for (int j = 1; j < P; j++) {
    int top = 0;
    for (int x = 0; x < 3; x++) if (j >> x & 1) top = x;
    for (int x = 0; x < 3; x++) cellid[j][x] = ((j >> x & 1) && x != top) ? ncells++ : -1;
  }
  int n = 0;
  auto put = [&](int src, int dst, int S, int D, int sc, int dc, unsigned key, unsigned flags) {
    Op& o = ops[n++];
    o.src = (uint16_t)src; o.dst = (uint16_t)dst; o.origin = (uint16_t)S; o.dest = (uint16_t)D;
    o.src_cell = sc; o.dst_cell = dc; o.key = key; o.flags = flags;
  };
  for (int R = 0; R < P; R++) put(R, R, R, R, -1, -1, 0u, 1u);
  for (int x = 0; (1 << x) < P; x++) {
    const int sp = 1 << x;
    for (int q = 0; q < P; q++) {
      const int t = ((q - sp) % P + P) % P;
      for (int j = 1; j < P; j++) {
        if (!(j >> x & 1)) continue;
        const int L = j & (sp - 1);
        const int S = (q + L) % P, D = ((S - j) % P + P) % P;
        int prev = 0;
        for (int b = 0; b < x; b++) if (L >> b & 1) prev = b;
        const bool first = (L == 0), final_ = (j >> (x + 1)) == 0;
        put(q, t, S, D, first ? -1 : cellid[j][prev], final_ ? -1 : cellid[j][x], (1u << 24) | (unsigned)x, 0u);
      }
    }
  }
  *ncells_out = ncells;
  return n;
}

}  // namespace

extern "C" const char* rbv_noalloc_last_error(void) { return g_msg; }

extern "C" int rbv_alltoallv_noalloc(int nranks, int type_size, const void* const* sendbufs, void* const* recvbufs,
                                     const int* sendcounts, const long long* sdispls, const int* recvcounts,
                                     const long long* rdispls, void* cuda_stream) {
  g_msg[0] = 0;
  if (nranks < 1 || type_size < 1 || !sendbufs || !recvbufs || !sendcounts || !sdispls || !rdispls)
    return fail(RBV_NOALLOC_ERR_BAD_ARG, "bad argument (rank count, type size or null pointer)");
  if (nranks > RBV_NOALLOC_MAX_RANKS) {
    std::snprintf(g_msg, sizeof g_msg, "nranks = %d exceeds the built-in limit of %d", nranks, RBV_NOALLOC_MAX_RANKS);
    return RBV_NOALLOC_ERR_TOO_LARGE;
  }
  const int P = nranks;
  for (int i = 0; i < P * P; i++) {
    if (sendcounts[i] < 0 || sdispls[i] < 0 || rdispls[i] < 0 || (recvcounts && recvcounts[i] < 0))
      return fail(RBV_NOALLOC_ERR_BAD_ARG, "negative count or displacement");
    if ((long long)sendcounts[i] * type_size > RBV_NOALLOC_MAX_BLOCK_BYTES) {
      std::snprintf(g_msg, sizeof g_msg, "block %d -> %d has %lld bytes; the built-in scratch allows %d per block",
                    i / P, i % P, (long long)sendcounts[i] * type_size, RBV_NOALLOC_MAX_BLOCK_BYTES);
      return RBV_NOALLOC_ERR_TOO_LARGE;
    }
  }
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(RBV_NOALLOC_ERR_CUDA, "cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return fail(RBV_NOALLOC_ERR_BAD_ARG, "device index out of range");
  DeviceState& ds = g_dev[dev];

  // ---- first call on this device: resolve the scratch array's device address (with this device current) and
  //      upload the schedules of all rank counts; later calls never synchronise ----
  {
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!ds.ready) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_scratch);
    if (e != cudaSuccess || !p) return fail(RBV_NOALLOC_ERR_CUDA, "cudaGetSymbolAddress(scratch)", e);
    ds.base = static_cast<unsigned char*>(p);
    e = cudaDeviceGetAttribute(&ds.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return fail(RBV_NOALLOC_ERR_CUDA, "cudaDeviceGetAttribute", e);
    int per_sm = 0;
    e = a2av_configure(kNR, &per_sm);
    if (e != cudaSuccess || per_sm < 1) return fail(RBV_NOALLOC_ERR_CUDA, "kernel configuration", e);
    for (int np = 1; np <= kNR; np++) {
      Op host_ops[kMaxOpsNA];
      ds.nops[np] = build_schedule(np, host_ops, &ds.ncells[np]);
      e = cudaMemcpy(ds.base + kOpsOff + kOpsSlot * (np - 1), host_ops, sizeof(Op) * ds.nops[np], cudaMemcpyHostToDevice);
      if (e != cudaSuccess) return fail(RBV_NOALLOC_ERR_CUDA, "schedule upload", e);
    }
    // the per-key stamps of a traced call start at "never"; this path does not trace, but the block is part of the layout
    e = cudaMemset(ds.base + kTraceOff, 0xff, sizeof(TraceBlock::kstart));
    if (e != cudaSuccess) return fail(RBV_NOALLOC_ERR_CUDA, "cudaMemset(trace block)", e);
    ds.ready = true;
  }
  }

  // ---- per call: control words start at zero ----
  e = cudaMemsetAsync(ds.base, 0, kClearBytes, st);
  if (e != cudaSuccess) return fail(RBV_NOALLOC_ERR_CUDA, "cudaMemsetAsync(control words)", e);

  KernelArgs ka;
  std::memset(&ka, 0, sizeof ka);
  ka.P = P; ka.L = P; ka.nproc = 1; ka.proc = 0;
  ka.type_size = type_size;
  ka.flags = CALL_META_INLINE;
  ka.nops = ds.nops[P];
  ka.absent_rank = -1;
  ka.ncells = ds.ncells[P];
  ka.ops = reinterpret_cast<const Op*>(ds.base + kOpsOff + kOpsSlot * (P - 1));
  ka.op_done = nullptr;
  ka.chunk_bytes = 8 << 10;
  ka.timeout_ns = 2000000000ull;
  ka.lay.ctrl_off = kCtrlOff; ka.lay.trace_off = kTraceOff; ka.lay.flags_off = kFlagsOff;
  ka.lay.flags_per_rank = kFlagsPerRank; ka.lay.meta_off = kMetaOff;
  ka.lay.meta_bytes = kMetaBytes; ka.lay.stage_off = kStageOff; ka.lay.arena_bytes = kArena;
  ka.lay.eager_off = kTotal; ka.lay.user_off = kTotal; ka.lay.total_bytes = kTotal;
  ka.heap[0] = reinterpret_cast<char*>(ds.base);
  ka.host_status = nullptr;
  ka.host_trace = nullptr;
  ka.meta_self = reinterpret_cast<char*>(ds.base) + kMetaOff;
  ka.meta_mc = nullptr;
  for (int r = 0; r < P; r++) {
    ka.sendbuf[r] = static_cast<const char*>(sendbufs[r]);
    // receive buffers are addressed relative to the scratch base; the difference wraps modulo 2^64 and the
    // kernel's pointer addition undoes it
    ka.recvoff[r] = (unsigned long long)(reinterpret_cast<uintptr_t>(recvbufs[r]) - reinterpret_cast<uintptr_t>(ds.base));
    for (int d = 0; d < P; d++) {
      ka.inl.sendcounts[r * P + d] = sendcounts[r * P + d];
      ka.inl.recvcounts[r * P + d] = recvcounts ? recvcounts[r * P + d] : -1;
      ka.inl.sdispls[r * P + d] = sdispls[r * P + d];
      ka.inl.rdispls[r * P + d] = rdispls[r * P + d];
    }
  }
  int grid = ds.sm_count < 32 ? ds.sm_count : 32;
  e = a2av_launch(ka, grid, true, st);
  if (e != cudaSuccess) return fail(RBV_NOALLOC_ERR_CUDA, "kernel launch", e);
  return RBV_NOALLOC_OK;
}

// Synchronises the stream and returns the device-side status code of the last call on the current device:
// 0 ok; otherwise the rbv::Status value that the kernel recorded first (1 a bounded wait ran out, 3 staging
// capacity, 4 a block larger than the receiver's recvcount, 5 stopped after an error elsewhere).
extern "C" int rbv_noalloc_status(void* cuda_stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices || !g_dev[dev].ready) return -1;
  if (cudaStreamSynchronize(static_cast<cudaStream_t>(cuda_stream)) != cudaSuccess) return -1;
  // the kernel keeps the code of the call it has just finished in the control block
  CtrlBlock c;
  if (cudaMemcpy(&c, g_dev[dev].base, sizeof c, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (c.last_code) return c.last_code;
  return c.abort_flag ? (int)RBV_ERR_ABORTED : 0;
}
