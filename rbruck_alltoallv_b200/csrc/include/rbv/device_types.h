// Structures shared by the host runtime and the device kernels.
//
// Execution model.  A *context* is one process driving one GPU.  It hosts L consecutive logical
// ranks of a P-rank communicator (L = P / nproc).  L = 1 is the production layout (one rank per
// GPU); L = P runs a whole communicator inside one kernel on one GPU, which is how the multi-rank
// logic is exercised where only one GPU is available and how a fixed P-rank problem is spread
// over fewer GPUs.  The kernels never distinguish the two: a rank's memory is reached through
// `heap[proc_of(rank)]`, which is either this GPU's heap or a peer mapping over NVLink.
//
// Every context owns one "symmetric heap" with the same internal layout on all processes:
//
//   [ CtrlBlock | cell flags | metadata tables x2 | staging arenas (L ranks x 2 parities) |
//     eager cell arenas (L ranks x 2 parities) | user ]
//
// Everything in front of the user region is zero when a context is created and after reset().  The eager
// protocol's cells have a region of their own: its units are valid by the call number in their flag words, so
// the region must never hold bytes that did not come from an eager call (user payload staged by the rendezvous
// protocol could carry any value), and the call number never goes back without the region being cleared.
//
// Cross-rank synchronisation uses monotonic counters and sequence-stamped flags only, so nothing
// has to be reset between calls:
//   * metadata table units and eager cell units carry the call number in their flag words
//   * recv_arrivals[local rank]  += 1 per chunk landed in recvbuf; the owner keeps the running target
//   * chunk_flag[parity][lr][f]   = seq + 1 when chunk f % flags_per_cell of staging cell f / flags_per_cell holds
//     this call's data (a relay hop forwards chunk k as soon as chunk k has landed, so the hops of a
//     store-and-forward schedule overlap chunk by chunk)
// Staging arenas, cell flags and metadata tables alternate by call parity: a peer can run at most
// one call ahead (it cannot finish call c+1 without data this rank sends in call c+1), so two
// copies suffice.
#pragma once
#include <cstdint>

#include "rbv/plan.h"

namespace rbv {

constexpr int kMaxRanks = 64;         // logical ranks per communicator for calls whose arguments travel as kernel
                                      // parameters and whose tables sit in shared memory (dynamic and eager kernels)
constexpr int kMaxRanksStatic = 1024; // logical ranks per communicator for persistent calls with host-side counts
                                      // (static kernel: no per-rank state in the kernel beyond its arrival tallies);
                                      // the reference's recorded traces go up to 1024 ranks
constexpr int kMaxProcs = 16;         // processes (GPUs) per communicator
constexpr int kMaxCellsPerRank = 2048;
constexpr int kMaxFlagsPerRank = 16384;   // chunk flags per rank and parity (cells x chunks per cell of one call)
constexpr int kMaxTraceKeys = 256;        // plan keys (rounds / batches) that can carry their own time stamps
constexpr int kInlineMeta = 64;       // L * P up to this many count/displacement entries travel as kernel parameters
constexpr int kThreads = 512;

enum Status : int {
  RBV_OK = 0,
  RBV_ERR_TIMEOUT = 1,    // a bounded wait ran out (peer absent or late)
  RBV_ERR_BAD_ARG = 2,
  RBV_ERR_CAPACITY = 3,   // staging arena too small for ncells * max block
  RBV_ERR_TRUNCATE = 4,   // a block is larger than the receiver's recvcount
  RBV_ERR_ABORTED = 5,    // another rank reported an error and asked everyone to stop
};

enum WaitSite : int { WAIT_META = 1, WAIT_CELL = 2, WAIT_RECV = 3, WAIT_BULK = 4 };

struct StatusBlock {
  int code;        // Status of the first error of the most recent call, 0 if none
  int site;        // WaitSite for time-outs
  int detail0;     // op index / local rank / cell, depending on site
  int detail1;     // peer rank or expected count
  unsigned long long trace[8];  // %globaltimer stamps of CTA 0: 0 start, 1 metadata published,
                                // 2 metadata complete, 3 own ops issued, 4 all blocks received,
                                // 5 / 6 before and after the fence that precedes the arrival report, 7 arrivals reported.
                                // Eager protocol: 1 work items sized, 2 first warp done, 3 first CTA done, 4 last CTA out,
                                // and with CALL_TRACE 5 latest CTA start, 6 latest CTA done
};

// Time stamps per plan key of the most recent traced call (CALL_TRACE): earliest start and latest end over all
// warps of the process that executed an item of that key.  Keys are numbered in issue order (Op::flags >> 16).
struct TraceBlock {
  unsigned long long kstart[kMaxTraceKeys];   // ~0ull: no item of this key ran
  unsigned long long kend[kMaxTraceKeys];
};

// Lives at offset 0 of every heap.  Peers write the counters with system-scope atomics.
struct CtrlBlock {
  unsigned long long recv_arrivals[kMaxRanksStatic];   // += 1 per chunk landed in a local rank's recvbuf
  unsigned long long recv_target[kMaxRanksStatic];     // running total of chunks expected so far (kept by the owner)
  unsigned int abort_flag;       // set locally on error, and by peers that want everyone to stop
  unsigned int pad0;
  unsigned int exit_count;       // traced calls only: CTAs that finished (the last one copies the stamps to the host)
  unsigned int call_seq;         // 0-based number of the next call; advanced by whoever completes start_count, so
                                 // that kernel arguments do not change from call to call
  StatusBlock status;
  // Auxiliary barriers of the fused kernels built on the same heap (0 MoE dispatch, 1 MoE combine,
  // 2 FFT transpose, 3 spare): arrivals are monotonic, seq counts finished calls, exit counts CTAs.
  unsigned long long aux_arrivals[4];
  unsigned int aux_seq[4];
  unsigned int aux_exit[4];
  // entered[q] = call number + 1 of the latest static call that process q has started; written by q.  A sender of
  // the static kernel stores into process q's memory only once q has entered the same call: without it a fast rank
  // could overwrite a receive buffer (or a staging cell of the same parity) that q still uses for the call before.
  // The dynamic kernel gets the same guarantee from its metadata exchange, the eager protocol from its headers.
  unsigned int entered[kMaxProcs];
  int last_code;                 // code of the first failure since the block was last cleared
  unsigned int start_count;      // CTAs (eager protocol with an item table: warps) that have read call_seq in this call
};

// Byte offsets of the regions of a heap; identical on every process of a communicator.
struct HeapLayout {
  unsigned long long ctrl_off;      // CtrlBlock
  unsigned long long trace_off;     // TraceBlock
  unsigned long long flags_off;     // uint32 chunk_flag[2][L][flags_per_rank]
  unsigned long long flags_per_rank;
  unsigned long long meta_off;      // 2 x MetaTable(P)
  unsigned long long meta_bytes;    // size of one parity copy
  unsigned long long stage_off;     // staging arenas: [L][2] x arena_bytes
  unsigned long long arena_bytes;   // per rank per parity
  unsigned long long eager_off;     // eager cell arenas: [L][2] x arena_bytes (only eager units are ever stored here)
  unsigned long long user_off;      // user allocations
  unsigned long long total_bytes;
};

// One parity copy of the metadata tables (sizes depend on P):
//   int32  counts[P][P]   row s written by rank s: what s sends to each d
//   int32  caps  [P][P]   row d written by rank d: recvcounts of d per source, -1 = unchecked
//   int64  rdispl[P][P]   row d written by rank d, in elements
//   uint64 recvoff[P]     offset of rank d's recvbuf inside its process's heap
// Stored as self-validating 16-byte units { word0, flag, word1, flag } with flag = call number + 1, so that a
// reader needs no separate arrival signal (one NVLink trip instead of store + acknowledged release):
//   CT[s][d]  { count, chunk bytes of sender s }        row s written by rank s
//   RT[d][s]  { cap, 0 } { rdispl lo, rdispl hi }       row d written by rank d (two units per entry)
//   RO[d]     { recvoff lo, recvoff hi }                written by rank d
__host__ __device__ inline unsigned long long meta_ct_off(int P) { (void)P; return 0; }
__host__ __device__ inline unsigned long long meta_rt_off(int P) { return 16ull * P * P; }
__host__ __device__ inline unsigned long long meta_ro_off(int P) { return 48ull * P * P; }
__host__ __device__ inline unsigned long long meta_table_bytes(int P) {
  return (48ull * P * P + 16ull * P + 255) & ~255ull;
}

enum CallFlags : unsigned {
  CALL_INPLACE = 1u,      // send data is taken from recvbuf (copied to a private region first)
  CALL_META_INLINE = 2u,  // counts/displacements are in KernelArgs::inl, not behind the pointers
  CALL_TRACE = 4u,        // copy the status block (with the phase time stamps) to the host after every call,
                          // not only after a failing one
  CALL_BULK = 8u,         // large aligned chunks go through the bulk-copy engine (shared-memory ring per warp)
  CALL_STATIC = 16u,      // every count of the call was known on the host: the kernel walks a table of resolved
                          // copy descriptors (StaticItem) and has no metadata phase
  CALL_SPREAD = 32u,      // eager kernel: work items are dealt CTA by CTA (item c to warp c / grid of CTA c % grid)
                          // over a grid of up to one CTA per item, instead of 16 consecutive items per CTA
};

// One resolved copy of the static rendezvous kernel: chunk k of one op with its addresses worked out on the host.
// Addresses that point into a staging arena are those of call parity 0; the kernel adds the parity stride.
struct alignas(16) StaticItem {
  unsigned long long src;   // address in this process (send buffer, staging cell, or own heap)
  unsigned long long dst;   // address as mapped in this process (own heap or a peer mapping)
  unsigned len;             // bytes (0: the item only signals)
  unsigned short dst_rank;  // logical rank written to
  unsigned short flags;     // ITEM_* bits | key index << 8
  unsigned wait_flag;       // chunk flag of this process to wait for (index at parity 0), kNoFlag: none
  unsigned signal_flag;     // chunk flag on the destination's process to raise, kNoFlag: the chunk counts as an
                            // arrival in dst_rank's receive buffer instead
};
static_assert(sizeof(StaticItem) == 32, "two 16-byte loads per item");
constexpr unsigned kNoFlag = 0xffffffffu;
enum ItemFlags : unsigned short {
  ITEM_SRC_STAGE = 1, ITEM_DST_STAGE = 2, ITEM_REMOTE = 4, ITEM_SELF = 8,
};

struct InlineMeta {
  int sendcounts[kInlineMeta];
  int recvcounts[kInlineMeta];
  long long sdispls[kInlineMeta];
  long long rdispls[kInlineMeta];
};

// One precomputed work item of the eager protocol: chunk `k` of op number `index`, with the op itself.
struct alignas(16) EagerItem {
  Op op;
  unsigned k;
  unsigned index;
};
static_assert(sizeof(EagerItem) == 32, "two 16-byte loads per item");

constexpr int kInlineEagerItems = 128;  // the first work items of an eager call with an item table travel in the
                                        // kernel parameters (all of them for a small call)

struct KernelArgs {
  int P, L, nproc, proc;
  int type_size;
  unsigned flags;
  // The call number as the host counts it (use_seq_hint != 0), which spares the kernel a trip to device memory
  // before its first byte moves.  The host counts exactly: every launch advances the number once, whatever becomes
  // of the call.  Launches recorded into a CUDA graph read the number from CtrlBlock::call_seq instead (their
  // arguments are frozen), and a context that has seen such a launch stops passing hints for good, because replays
  // advance the number behind the host's back.  The CTA that advances the number checks the hint against memory.
  unsigned seq_hint, use_seq_hint;
  int nops;                // ops executed by this process
  int absent_rank;         // fault injection for tests: this local rank never publishes its metadata (-1: none)
  int ncells;
  const Op* ops;           // device copy of the process's op list
  unsigned* op_done;       // [nops] completion counters of multi-chunk ops (zero between calls)
  unsigned long long chunk_bytes;
  unsigned long long eager_payload;  // eager protocol: payload bytes a cell can hold (0: rendezvous protocol)
  const EagerItem* items;            // eager protocol, persistent calls with host-side counts: the work items,
  unsigned nitems;                   // each with a copy of its op (one load instead of two); null: sized in the kernel
  unsigned long long timeout_ns;
  HeapLayout lay;
  char* heap[kMaxProcs];   // heap base of every process as mapped in this process
  char* meta_self;         // this process's metadata tables (both parities); normally heap[proc] + lay.meta_off
  char* meta_mc;           // NVLS: multicast address of the same tables on ALL processes (null: peer stores)
  const char* sendbuf[kMaxRanks];         // per local rank (any device memory of this GPU)
  unsigned long long recvoff[kMaxRanks];  // per local rank: recvbuf offset in this process's heap
  unsigned long long sendcopy_off[kMaxRanks];  // CALL_INPLACE: private copy location (heap offset)
  unsigned long long sendcopy_bytes[kMaxRanks];
  // device arrays [L][P]; recvcounts may be null (no truncation check)
  const int* sendcounts;
  const int* recvcounts;
  const long long* sdispls;
  const long long* rdispls;
  StatusBlock* host_status;  // pinned, mapped: a copy of the final status
  TraceBlock* host_trace;    // pinned, mapped: per-key stamps of a traced call
  InlineMeta inl;
  EagerItem inl_items[kInlineEagerItems];   // the first items of the table behind `items` (when there is one)
};

constexpr int kInlineItems = 128;  // the first items of a static call travel in the kernel parameters

// One received block (or a piece of it) that the static kernel copies on, once everything has arrived, from the
// receive buffer in the symmetric heap to the caller's own buffer (any device-accessible memory, e.g. pinned host
// memory).
struct alignas(16) DrainItem {
  unsigned long long src, dst;
  unsigned len, pad0, pad1, pad2;
};

// Arguments of the static rendezvous kernel (a2av_static.cu): a persistent call whose counts were all known on
// the host.  Everything that depends on counts sits in the table behind `items`.
struct StaticArgs {
  int P, L, nproc, proc;
  unsigned flags;                       // CALL_TRACE
  unsigned nitems;
  unsigned seq_hint, use_seq_hint;      // as in KernelArgs
  const StaticItem* items;              // issue order; item c is handled by warp c mod (warps in the grid)
  const unsigned long long* expect;     // [L] chunks that land in each local rank's receive buffer per call
  const DrainItem* drain;               // copies made after the last arrival (receive buffers mirrored elsewhere)
  unsigned ndrain, pad;
  unsigned long long timeout_ns;
  HeapLayout lay;
  char* heap[kMaxProcs];
  StatusBlock* host_status;
  TraceBlock* host_trace;               // pinned copy of the per-key stamps (written when CALL_TRACE is set)
  // The first kInlineItems items of the table: a warp whose first item is among them starts without a trip to
  // device memory (after an L2 flush that trip is a DRAM access on the critical path of a small call).
  StaticItem inl[kInlineItems];
};

}  // namespace rbv
