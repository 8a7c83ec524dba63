// Host-side schedule compiler ("plan compiler") for every alltoallv algorithm of the library.
//
// An alltoallv over P ranks is described as an ordered list of transfer operations ("ops").
// One op moves one (origin S -> destination D) block one hop: the executing rank `src` reads the
// block either from its own send buffer (first hop) or from one of its staging cells (relay hop)
// and stores it either into the final location in the receive buffer of `dst` (last hop) or into
// a staging cell of `dst`.  The size of the block is always C[S][D] * type_size, where C is the
// global P x P count matrix, so no per-round metadata has to travel with the data.
//
// Staging cells are single-assignment within one call: a cell is written by exactly one op and
// read by exactly one later op.  That removes the write-after-read hazard that MPI's copy-in /
// copy-out semantic hides in the reference (it packs a staging slot into a temporary buffer
// before the same round's incoming data is unpacked into it, e.g. src/tuna2.cpp:167-223).
//
// All algorithm families of the reference differ only in (a) which intermediate ranks a block
// visits, (b) the order / batching in which ops are issued.  The kernels are generic interpreters
// of this op list.  Reference files covered: src/twophase_tunable_rbruckv.cpp, -om.cpp, tuna.cpp,
// tuna2.cpp, twophase_twolayer_rbruck.cpp, twolayer_rbruck.cpp, twolayer_communicator_linear.cpp,
// MPICH_scattered.cpp, OpenMPI_basic_linear.cpp, OpenMPI_pairwise.cpp, exclusive_or_alltoallv.cpp,
// benchmarks/common.cpp.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace rbv {

enum Algo : int {
  ALG_LINEAR = 0,             // ompi_alltoallv_intra_basic_linear
  ALG_SPREADOUT = 1,          // spreadout_alltoallv
  ALG_SCATTERED = 2,          // MPICH_intra_scattered(bblock)
  ALG_PAIRWISE = 3,           // ompi_alltoallv_intra_pairwise
  ALG_XOR = 4,                // exclisive_or_alltoallv
  ALG_TWOLAYER_LINEAR = 5,    // twolayer_communicator_linear(n)
  ALG_TWOLAYER_LINEAR_S2 = 6, // ..._s2(n, bblock1, bblock2)
  ALG_TWOLAYER_LINEAR_S3 = 7, // ..._s3(n, bblock1, bblock2)
  ALG_TWOLAYER_LINEAR_S4 = 8, // ..._s4 (declared only in the reference)
  ALG_RBRUCK = 9,             // twophase_rbruck_alltoallv(r)        digits high -> low
  ALG_RBRUCK_OM = 10,         // twophase_rbruck_alltoallv_om(r)     digits low -> high
  ALG_TUNA = 11,              // tuna_algorithm(r, b)
  ALG_TUNA2 = 12,             // tuna2_algorithm(r, b)
  ALG_TTPL = 13,              // TTPL_rbruck_alltoallv(n, r)         Bruck at both layers
  ALG_TTPL_BT = 14,           // TTPL_BT_alltoallv(n, r, bblock)     coalesced inter phase
  ALG_TTPL_BT_S1 = 15,        // TTPL_BT_alltoallv_s1                staggered inter phase
  ALG_TTPL_BT_S2 = 16,        // TTPL_BT_alltoallv_s2                staggered + in-place option
  ALG_UNIFORM_SPREADOUT_TWOLAYER = 17,  // uniform_spreadout_twolayer(n, r)
  ALG_UNIFORM_ISPLIT_RBRUCK = 18,       // uniform_inverse_isplit_r_bruck(n, r1, r2)
  ALG_MERGE = 19,             // merge_alltoallv(n): benchmarks/merge_benchmark.cpp:155-332 (completed)
  ALG_SIMPLE_MERGE = 20,      // simply_merge_alltoallv(n): benchmarks/simple_merge_benchmark.cpp:138-210
  ALG_SPLIT = 21,             // split_alltoallv: benchmarks/split_benchmark.cpp:147-205
  ALG_COUNT = 22
};

const char* algo_name(int algo);
int algo_from_name(const char* name);  // -1 if unknown

struct AlgoSpec {
  int algo = ALG_SPREADOUT;
  int P = 1;    // number of logical ranks
  int n = 0;    // ranks per group (hierarchical algorithms)
  int r = 2;    // radix (r1 for the uniform two-layer Bruck)
  int r2 = 0;   // inter-group radix (uniform_inverse_isplit_r_bruck)
  int b = 0;    // batch: b (TuNA), bblock (scattered / TTPL), bblock1 (two-layer linear)
  int b2 = 0;   // bblock2 (two-layer linear)
};

// One hop of one block.  24 bytes; the device kernels read this layout directly.
struct Op {
  uint16_t src;      // logical rank that executes the op (reads its own memory)
  uint16_t dst;      // logical rank whose memory is written
  uint16_t origin;   // S: rank whose send buffer the block came from
  uint16_t dest;     // D: rank whose receive buffer the block ends in
  int32_t src_cell;  // -1: read sendbuf[sdispls[D]] of src (then src == S); else staging cell of src
  int32_t dst_cell;  // -1: write recvbuf[rdispls[S]] of dst (then dst == D); else staging cell of dst
  uint32_t key;      // issue order: ops are executed in non-decreasing key order per process
  uint32_t flags;    // bit 0: self copy; bit 1: eager unpack (added by the runtime); bits 2-8: part index and
                     // bits 9-15: part count of an op that moves one slice of its block (0: the whole block);
                     // bits 16-31: number of the op's key among the plan's distinct keys, in issue order
};
static_assert(sizeof(Op) == 24, "device code depends on this layout");

#if defined(__CUDACC__)
#define RBV_HD __host__ __device__
#else
#define RBV_HD
#endif
constexpr uint32_t kOpSelf = 1u, kOpUnpack = 2u;
RBV_HD inline uint32_t op_part(const Op& o) { return (o.flags >> 2) & 127u; }
RBV_HD inline uint32_t op_nparts(const Op& o) { return (o.flags >> 9) & 127u; }
RBV_HD inline uint32_t op_key_index(const Op& o) { return o.flags >> 16; }
// Elements [first, first + n) of a block of `count` elements that the op moves: the whole block, or slice
// `part` of `nparts` equal slices (the last one also takes the remainder).
RBV_HD inline void op_slice(const Op& o, long long count, long long* first, long long* n) {
  const long long np = op_nparts(o);
  if (np == 0) { *first = 0; *n = count; return; }
  const long long div = count / np, p = op_part(o);
  *first = p * div;
  *n = (p == np - 1) ? count - p * div : div;
}

struct PlanStats {
  int w = 0;            // digits of the (intra) Bruck
  int K = 0;            // communication rounds of the (intra) Bruck
  int w2 = 0, K2 = 0;   // inter-group Bruck, if any
  int max_blocks_per_round = 0;
  long long hops = 0;   // total ops excluding self copies (forwarded volume in blocks)
  int phases = 0;       // number of distinct keys
};
constexpr int kMaxOpParts = 127;

struct Plan {
  AlgoSpec spec;        // normalised (clamped) parameters
  int err = 0;          // 0 ok; -1 invalid argument in the reference's sense (its return code)
  std::string errmsg;
  int ncells = 0;       // staging cells needed on every rank
  std::vector<Op> ops;  // all ranks, stable-sorted by key
  std::vector<uint32_t> keys;  // the distinct keys in issue order (Op::flags >> 16 indexes this list)
  PlanStats stats;
  bool uniform = false;       // algorithm takes one count for all pairs
  bool inplace_ok = false;    // algorithm accepts sendbuf == NULL (data taken from recvbuf)
};

// Builds the plan.  Never throws; check plan.err.
Plan build_plan(const AlgoSpec& spec);

// The subset of plan.ops executed by the given logical ranks (order preserved).
std::vector<Op> ops_for_ranks(const Plan& plan, const std::vector<int>& ranks);

// Integer helpers shared with the C API (reference: src/utils.cpp:9-29).
int ipow(int x, unsigned p);
int ndigits(int max_value, int r);  // number of base-r digits of max_value (0 for 0)
std::vector<int> to_base(int w, int N, int b);

// CPU executor: runs the plan on host buffers, processing ops strictly in list order.  It is the
// executable specification of what the kernels must do and doubles as the host fallback.
// sendbufs/recvbufs: P pointers.  counts: sendcounts[s*P+d], sdispls[s*P+d] (elements, per sender s),
// rdispls[d*P+s] (elements, per receiver d).  Returns 0, or a negative code when the plan violates a
// hazard rule (read of an unfilled cell: -10, second write to a cell: -11, bad op: -12).
// build_plan itself refuses (err -13) a schedule in which some (origin, destination) pair has no first hop or
// more than one: the eager protocol's cell reuse relies on every pair exchanging a header in every call.
int host_execute(const Plan& plan, int type_size, const char* const* sendbufs, char* const* recvbufs,
                 const int* sendcounts, const long long* sdispls, const long long* rdispls);

}  // namespace rbv
