// C API: context management and the reference-shaped collective entry points (rbv/rbruckv.h).
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "rbv/context.h"
#include "rbv/rbruckv.h"
#include "api/ctx_internal.h"

using namespace rbv;

static thread_local std::string g_err;

double init_time = 0, findMax_time = 0, rotateIndex_time = 0, alcCopy_time = 0, getBlock_time = 0, prepData_time = 0,
       excgMeta_time = 0, excgData_time = 0, replace_time = 0, orgData_time = 0, prepSP_time = 0, SP_time = 0;
double intra_time = 0;
double* iteration_time = nullptr;

static_assert(sizeof(rbv_status) == sizeof(StatusBlock), "status layouts must agree");

extern "C" {

const char* rbv_last_error(void) { return g_err.c_str(); }

rbv_ctx_t rbv_ctx_create(int nranks, int nproc, int proc, int device, size_t user_bytes, size_t arena_bytes) {
  try {
    auto ctx = std::make_unique<rbv_ctx_s>();
    ctx->c = std::make_unique<Context>(nranks, nproc, proc, device, user_bytes, arena_bytes);
    const int L = ctx->c->L();
    ctx->comms.resize(L);
    for (int i = 0; i < L; i++) ctx->comms[i] = rbv_comm_s{ctx.get(), i};
    ctx->seen.assign(L, 0);
    ctx->sendbufs.assign(L, nullptr);
    ctx->recvbufs.assign(L, nullptr);
    const size_t n = (size_t)L * nranks;
    ctx->sc.assign(n, 0); ctx->rc.assign(n, 0); ctx->sd.assign(n, 0); ctx->rd.assign(n, 0);
    return ctx.release();
  } catch (const std::exception& e) {
    g_err = e.what();
    return nullptr;
  }
}

void rbv_ctx_destroy(rbv_ctx_t ctx) {
  if (!ctx) return;
  if (ctx->cached) rbv_prepared_free(ctx, ctx->cached);
  delete ctx;
}

int rbv_ctx_ipc_handle(rbv_ctx_t ctx, void* out64) {
  cudaError_t e = ctx->c->ipc_handle(out64);
  if (e != cudaSuccess) { g_err = cudaGetErrorString(e); return (int)e; }
  return 0;
}
int rbv_ctx_connect(rbv_ctx_t ctx, const void* handles) {
  cudaError_t e = ctx->c->connect(handles);
  if (e != cudaSuccess) { g_err = cudaGetErrorString(e); return (int)e; }
  return 0;
}
void rbv_ctx_set_stream(rbv_ctx_t ctx, void* s) { ctx->stream = static_cast<cudaStream_t>(s); }
void rbv_ctx_set_timeout_ms(rbv_ctx_t ctx, double ms) { ctx->c->set_timeout_ns((unsigned long long)(ms * 1e6)); }
void rbv_ctx_set_launch(rbv_ctx_t ctx, int grid, size_t chunk) { ctx->grid = grid; ctx->chunk = chunk; }
void rbv_ctx_set_absent_rank(rbv_ctx_t ctx, int lr) { ctx->c->set_absent_rank(lr); }
int rbv_ctx_sync(rbv_ctx_t ctx) { return (int)cudaStreamSynchronize(ctx->stream); }
int rbv_ctx_status(rbv_ctx_t ctx, rbv_status* out) {
  StatusBlock s = ctx->c->status(ctx->stream);
  std::memcpy(out, &s, sizeof s);
  return s.code;
}
int rbv_ctx_reset(rbv_ctx_t ctx) {
  ctx->pend = 0;
  std::fill(ctx->seen.begin(), ctx->seen.end(), 0);
  return (int)ctx->c->reset();
}
int rbv_ctx_info(rbv_ctx_t ctx, long long* o) {
  o[0] = ctx->c->P(); o[1] = ctx->c->L(); o[2] = ctx->c->nproc(); o[3] = ctx->c->proc();
  o[4] = ctx->c->device(); o[5] = 0; o[6] = ctx->c->max_ctas(); o[7] = ctx->c->sm_count();
  return 0;
}
void* rbv_ctx_heap(rbv_ctx_t ctx, int proc) { return ctx->c->peer_heap(proc); }
int rbv_ctx_in_heap(rbv_ctx_t ctx, const void* p, size_t bytes) { return ctx->c->in_heap(p, bytes ? bytes : 1) ? 1 : 0; }
void* rbv_symm_alloc(rbv_ctx_t ctx, size_t bytes) { return ctx->c->symm_alloc(bytes); }
int rbv_symm_free(rbv_ctx_t ctx, void* p) { return ctx->c->symm_free(p); }
rbv_comm_t rbv_comm(rbv_ctx_t ctx, int local_rank) {
  if (local_rank < 0 || local_rank >= (int)ctx->comms.size()) return nullptr;
  return &ctx->comms[local_rank];
}
int rbv_comm_rank(rbv_comm_t comm) { return comm->ctx->c->proc() * comm->ctx->c->L() + comm->local; }
int rbv_comm_size(rbv_comm_t comm) { return comm->ctx->c->P(); }

int rbv_alltoallv(rbv_ctx_t ctx, int algo, int n, int r, int r2, int b, int b2, int type_size,
                  const void* const* sendbufs, void* const* recvbufs, const int* sendcounts,
                  const int* recvcounts, const long long* sdispls, const long long* rdispls,
                  int counts_on_device, long long bytes_hint, unsigned flags, int grid, size_t chunk_bytes,
                  void* cuda_stream) {
  try {
    AlgoSpec s;
    s.algo = algo; s.P = ctx->c->P(); s.n = n; s.r = r; s.r2 = r2; s.b = b; s.b2 = b2;
    CallArgs ca;
    ca.sendbufs = sendbufs; ca.recvbufs = recvbufs;
    ca.sendcounts = sendcounts; ca.recvcounts = recvcounts; ca.sdispls = sdispls; ca.rdispls = rdispls;
    ca.counts_on_device = counts_on_device != 0;
    ca.bytes_hint = bytes_hint;
    CallOptions opt;
    opt.grid = grid; opt.chunk_bytes = chunk_bytes; opt.flags = flags;
    opt.eager_max_bytes = ctx->eager;
    int rc = ctx->c->alltoallv(s, type_size, ca, opt, static_cast<cudaStream_t>(cuda_stream));
    if (rc) g_err = ctx->c->last_error();
    return rc;
  } catch (const std::exception& e) {
    g_err = e.what();
    return RBV_ERR_BAD_ARG;
  }
}

void* rbv_prepare_global(rbv_ctx_t ctx, int algo, int n, int r, int r2, int b, int b2, int type_size,
                         const void* const* sendbufs, void* const* recvbufs, const int* sendcounts,
                         const int* recvcounts, const long long* sdispls, const long long* rdispls,
                         int counts_on_device, long long bytes_hint, unsigned flags, int grid, size_t chunk_bytes,
                         const int* g_counts, const int* g_caps, const long long* g_rdispls,
                         const unsigned long long* g_recvoff) {
  try {
    AlgoSpec s;
    s.algo = algo; s.P = ctx->c->P(); s.n = n; s.r = r; s.r2 = r2; s.b = b; s.b2 = b2;
    CallArgs ca;
    ca.sendbufs = sendbufs; ca.recvbufs = recvbufs;
    ca.sendcounts = sendcounts; ca.recvcounts = recvcounts; ca.sdispls = sdispls; ca.rdispls = rdispls;
    ca.counts_on_device = counts_on_device != 0;
    ca.bytes_hint = bytes_hint;
    ca.g_counts = g_counts; ca.g_caps = g_caps; ca.g_rdispls = g_rdispls; ca.g_recvoff = g_recvoff;
    std::vector<void*> mirror;
    mirror.swap(ctx->recv_mirror);   // holds for this call only
    if ((int)mirror.size() == ctx->c->L()) ca.recv_mirror = mirror.data();
    CallOptions opt;
    opt.grid = grid; opt.chunk_bytes = chunk_bytes; opt.flags = flags & CALL_INPLACE;
    opt.allow_static = ctx->allow_static && !(flags & 0x100u);
    opt.recv_anywhere = (flags & 0x200u) != 0;
    opt.eager_max_bytes = ctx->eager;
    auto pc = std::make_unique<Prepared>();
    int rc = ctx->c->prepare(s, type_size, ca, opt, nullptr, true, pc.get());
    ctx->last_rc = rc;
    if (rc) { g_err = ctx->c->last_error(); return nullptr; }
    return pc.release();
  } catch (const std::exception& e) {
    g_err = e.what();
    ctx->last_rc = RBV_ERR_BAD_ARG;
    return nullptr;
  }
}
void* rbv_prepare(rbv_ctx_t ctx, int algo, int n, int r, int r2, int b, int b2, int type_size,
                  const void* const* sendbufs, void* const* recvbufs, const int* sendcounts,
                  const int* recvcounts, const long long* sdispls, const long long* rdispls,
                  int counts_on_device, long long bytes_hint, unsigned flags, int grid, size_t chunk_bytes) {
  return rbv_prepare_global(ctx, algo, n, r, r2, b, b2, type_size, sendbufs, recvbufs, sendcounts, recvcounts, sdispls,
                            rdispls, counts_on_device, bytes_hint, flags, grid, chunk_bytes, nullptr, nullptr, nullptr,
                            nullptr);
}
// 0 dynamic rendezvous kernel, 1 eager kernel, 2 static rendezvous kernel; out3 = grid, cooperative launch needed, items
int rbv_prepared_info(void* prepared, long long* out3) {
  const Prepared* pc = static_cast<Prepared*>(prepared);
  if (out3) { out3[0] = pc->grid; out3[1] = pc->cooperative ? 1 : 0; out3[2] = pc->is_static ? pc->sa.nitems : pc->ka.nitems; }
  return pc->is_static ? 2 : (pc->eager ? 1 : 0);
}
int rbv_launch(rbv_ctx_t ctx, void* prepared, void* cuda_stream) {
  int rc = ctx->c->launch(*static_cast<Prepared*>(prepared), static_cast<cudaStream_t>(cuda_stream));
  if (rc) g_err = ctx->c->last_error();
  return rc;
}
void rbv_prepared_free(rbv_ctx_t ctx, void* prepared) {
  Prepared* pc = static_cast<Prepared*>(prepared);
  if (!pc) return;
  ctx->c->release(*pc);
  delete pc;
}
int rbv_ctx_set_nvls_meta(rbv_ctx_t ctx, void* self_ptr, void* mc_ptr, size_t bytes) {
  int rc = ctx->c->set_nvls_meta(self_ptr, mc_ptr, bytes);
  if (rc) g_err = ctx->c->last_error();
  return rc;
}
size_t rbv_ctx_meta_bytes(rbv_ctx_t ctx) { return ctx->c->nvls_bytes_needed(); }
// The library's own NVLS set-up (see Context::nvls_*): each step returns 0 or an error code.
int rbv_ctx_nvls_create(rbv_ctx_t ctx, size_t bytes, int* fd_out, size_t* size_out) {
  int rc = ctx->c->nvls_create(bytes, fd_out);
  if (rc) g_err = ctx->c->last_error();
  else if (size_out) *size_out = ctx->c->nvls_object_bytes();
  return rc;
}
int rbv_ctx_nvls_import(rbv_ctx_t ctx, int fd, size_t bytes) {
  int rc = ctx->c->nvls_import(fd, bytes);
  if (rc) g_err = ctx->c->last_error();
  return rc;
}
int rbv_ctx_nvls_add_device(rbv_ctx_t ctx) {
  int rc = ctx->c->nvls_add_device();
  if (rc) g_err = ctx->c->last_error();
  return rc;
}
int rbv_ctx_nvls_bind(rbv_ctx_t ctx) {
  void *self = nullptr, *mc = nullptr;
  size_t bytes = 0;
  int rc = ctx->c->nvls_bind_and_map(&self, &mc, &bytes);
  if (!rc) rc = ctx->c->set_nvls_meta(self, mc, bytes);
  if (rc) g_err = ctx->c->last_error();
  return rc;
}
void rbv_ctx_nvls_teardown(rbv_ctx_t ctx) { ctx->c->nvls_teardown(); }
void rbv_ctx_set_eager(rbv_ctx_t ctx, unsigned long long max_block_bytes) { ctx->eager = max_block_bytes; }
void rbv_ctx_set_trace(rbv_ctx_t ctx, int on) { ctx->c->set_trace(on != 0); }
void rbv_ctx_set_bulk(rbv_ctx_t ctx, int mode) { ctx->c->set_bulk(mode); }
void rbv_ctx_set_cooperative(rbv_ctx_t ctx, int mode) { ctx->c->set_cooperative(mode < 0 ? -1 : (mode ? 1 : 0)); }
void rbv_ctx_set_static(rbv_ctx_t ctx, int on) { ctx->allow_static = on != 0; }
void rbv_ctx_set_recv_mirror(rbv_ctx_t ctx, void* const* mirrors) {
  ctx->recv_mirror.clear();
  if (mirrors) ctx->recv_mirror.assign(mirrors, mirrors + ctx->c->L());
}
void rbv_ctx_set_auto_hint(rbv_ctx_t ctx, double mean_block_bytes, double cv) { ctx->hint_mean = mean_block_bytes; ctx->hint_cv = cv; }

// Per-key time stamps of the most recent traced call: fills keys[i] (plan key: phase << 24 | step), start_ns[i],
// end_ns[i] for up to `max` keys and returns the number of keys of the plan (the eager protocol adds one more entry
// for unpacking, with key 0xffffffff).  Synchronises the context's stream.
int rbv_ctx_last_trace(rbv_ctx_t ctx, unsigned* keys, unsigned long long* start_ns, unsigned long long* end_ns, int max) {
  cudaStreamSynchronize(ctx->stream);
  const DevPlan* dp = ctx->c->last_plan();
  if (!dp) return 0;
  const TraceBlock& tb = ctx->c->last_trace();
  const int nk = (int)dp->plan.keys.size();
  int n = 0;
  for (int i = 0; i <= nk && i < kMaxTraceKeys && n < max; i++) {
    if (i == nk && (tb.kstart[i] == ~0ull || tb.kend[i] == 0)) break;
    keys[n] = i < nk ? dp->plan.keys[i] : 0xffffffffu;
    start_ns[n] = tb.kstart[i];
    end_ns[n] = tb.kend[i];
    n++;
  }
  return n;
}

// Fills the reference's timer globals (src/twophase_twolayer_rbruck.cpp:10-12, src/twolayer_communicator_linear.cpp:
// 10-11) from the device stamps of the most recent traced call.  What each name means here:
//   init_time        kernel start until the first item of the call starts (launch ramp, call number, tables)
//   findMax_time     metadata publish (the reference's max-count MPI_Allreduce happens in the same exchange)
//   rotateIndex_time host time spent compiling the schedule (the reference's index-rotation arrays; 0 when cached)
//   alcCopy_time     self copies (the reference times its allocations and the self memcpy under this name)
//   getBlock_time    0: block lists are part of the compiled schedule
//   prepData_time    0: nothing is packed, blocks are read in place
//   excgMeta_time    waiting for the peers' metadata (or, in the static kernel, for the peers to enter the call)
//   excgData_time    first to last item of the intra-group / flat Bruck rounds (phase 1 keys)
//   replace_time     eager protocol: unpacking arrival cells into the receive buffer; otherwise 0
//   orgData_time     hand-out stage of the leader-routed exchanges (phase 3 keys); otherwise 0
//   prepSP_time      0: the inter-group displacement tables are part of the compiled schedule
//   SP_time          first to last item of the inter-group phase (phase 2 keys)
//   intra_time       same span as excgData_time
//   iteration_time   one entry per inter-group batch (phase 2 key), malloc'ed here; like in the reference the
//                    caller frees it (the previous array is not freed by the library)
// Returns the status code of that call.
int rbv_update_timers(rbv_ctx_t ctx) {
  StatusBlock s = ctx->c->status(ctx->stream);
  auto sec = [&](int a, int b) { return s.trace[b] > s.trace[a] ? (double)(s.trace[b] - s.trace[a]) * 1e-9 : 0.0; };
  init_time = findMax_time = rotateIndex_time = alcCopy_time = getBlock_time = prepData_time = excgMeta_time =
      excgData_time = replace_time = orgData_time = prepSP_time = SP_time = intra_time = 0;
  iteration_time = nullptr;
  const DevPlan* dp = ctx->c->last_plan();
  if (!dp) return s.code;
  rotateIndex_time = ctx->plan_build_s;
  const TraceBlock& tb = ctx->c->last_trace();
  const int nk = std::min<int>((int)dp->plan.keys.size(), kMaxTraceKeys - 1);
  unsigned long long lo[4] = {~0ull, ~0ull, ~0ull, ~0ull}, hi[4] = {0, 0, 0, 0}, first = ~0ull;
  std::vector<double> batches;
  for (int i = 0; i < nk; i++) {
    if (tb.kstart[i] == ~0ull || tb.kend[i] < tb.kstart[i]) continue;
    const unsigned ph = std::min(3u, dp->plan.keys[i] >> 24);
    lo[ph] = std::min(lo[ph], tb.kstart[i]);
    hi[ph] = std::max(hi[ph], tb.kend[i]);
    first = std::min(first, tb.kstart[i]);
    if (ph == 2) batches.push_back((double)(tb.kend[i] - tb.kstart[i]) * 1e-9);
  }
  auto span = [&](int ph) { return hi[ph] > lo[ph] && lo[ph] != ~0ull ? (double)(hi[ph] - lo[ph]) * 1e-9 : 0.0; };
  if (first != ~0ull && first > s.trace[0]) init_time = (double)(first - s.trace[0]) * 1e-9;
  alcCopy_time = span(0);
  excgData_time = intra_time = span(1);
  SP_time = span(2);
  orgData_time = span(3);
  if (s.trace[2] > s.trace[1] && s.trace[1] > s.trace[0] && s.trace[2] - s.trace[0] < 1000000000ull) {
    findMax_time = sec(0, 1);      // dynamic kernel: publish, then wait for the peers' rows
    excgMeta_time = sec(1, 2);
  }
  if (nk < kMaxTraceKeys - 1 && tb.kstart[nk] != ~0ull && tb.kend[nk] > tb.kstart[nk])
    replace_time = (double)(tb.kend[nk] - tb.kstart[nk]) * 1e-9;
  if (!batches.empty()) {
    iteration_time = static_cast<double*>(std::malloc(batches.size() * sizeof(double)));
    if (iteration_time) std::memcpy(iteration_time, batches.data(), batches.size() * sizeof(double));
  }
  return s.code;
}
int rbv_iteration_count(rbv_ctx_t ctx) {
  const DevPlan* dp = ctx->c->last_plan();
  int n = 0;
  if (dp) for (unsigned k : dp->plan.keys) if ((k >> 24) == 2) n++;
  return n;
}

int myPow(int x, unsigned int p) { return ipow(x, p); }

int check_errors(int* recvcounts, long long* recv_buffer, int rank, int nprocs) {
  int error = 0;
  long long index = 0;
  for (int p = 0; p < nprocs; p++)
    for (int s = 0; s < recvcounts[p]; s++, index++) {
      if ((p != 0 || rank != 0) && recv_buffer[index] == 0) error++;
      if ((recv_buffer[index] % 10) != (rank % 10)) error++;
    }
  return error;
}

}  // extern "C"

std::vector<int> convert10tob(int w, int N, int b) { return to_base(w, N, b); }

// ---- per-rank entry points -------------------------------------------------------------------
namespace {

AlgoSpec mk(int algo, int n = 0, int r = 2, int r2 = 0, int b = 0, int b2 = 0) {
  AlgoSpec s;
  s.algo = algo; s.n = n; s.r = r; s.r2 = r2; s.b = b; s.b2 = b2;
  return s;
}
AlgoSpec mk_spreadout() { return mk(ALG_SPREADOUT); }

int enqueue(rbv_comm_t comm, const AlgoSpec& spec_in, int ts, const char* sendbuf, const int* sendcounts,
            const int* sdispls, char* recvbuf, const int* recvcounts, const int* rdispls, unsigned flags) {
  if (!comm) { g_err = "null communicator"; return RBV_ERR_BAD_ARG; }
  rbv_ctx_s* ctx = comm->ctx;
  Context& c = *ctx->c;
  const int P = c.P(), L = c.L(), lr = comm->local;
  AlgoSpec spec = spec_in;
  spec.P = P;
  const bool automatic = spec.algo < 0;
  if (automatic) spec = mk_spreadout();   // placeholder until all local ranks have arrived
  spec.P = P;
  // argument validation happens in the plan compiler; evaluate it now so that every rank gets the code
  try {
    const DevPlan* dp = c.plan_for(spec);
    if (c.last_plan_build_s() > 0) ctx->plan_build_s = c.last_plan_build_s();
    if (dp->plan.err) { g_err = dp->plan.errmsg; return dp->plan.err; }
  } catch (const std::exception& e) { g_err = e.what(); return RBV_ERR_BAD_ARG; }
  if (ctx->pend == 0) {
    ctx->spec = spec; ctx->ts = ts; ctx->flags = flags; ctx->automatic = automatic;
  } else if (std::memcmp(&ctx->spec, &spec, sizeof spec) != 0 || ctx->ts != ts || ctx->flags != flags ||
             ctx->automatic != automatic) {
    g_err = "local ranks called different collectives";
    return RBV_ERR_BAD_ARG;
  }
  if (ctx->seen[lr]) { g_err = "rank called twice before the others arrived"; return RBV_ERR_BAD_ARG; }
  ctx->seen[lr] = 1;
  ctx->sendbufs[lr] = sendbuf;
  ctx->recvbufs[lr] = recvbuf;
  for (int i = 0; i < P; i++) {
    ctx->sc[(size_t)lr * P + i] = sendcounts[i];
    ctx->rc[(size_t)lr * P + i] = recvcounts ? recvcounts[i] : -1;
    ctx->sd[(size_t)lr * P + i] = sdispls[i];
    ctx->rd[(size_t)lr * P + i] = rdispls[i];
  }
  if (++ctx->pend < L) return 0;
  ctx->pend = 0;
  std::fill(ctx->seen.begin(), ctx->seen.end(), 0);
  bool have_rc = true;
  for (int v : ctx->rc) if (v < 0) have_rc = false;
  unsigned long long saved_eager = ctx->eager;
  if (automatic) {
    // The choice must be the same on every process.  A process that hosts all ranks sees the whole count matrix;
    // otherwise the caller's hint decides, and without one the spread-out order with the rendezvous protocol,
    // which every process can pick on its own.
    double mean = ctx->hint_mean, cv = ctx->hint_cv;
    long long mx = 0;
    if (L == P) {
      double s1 = 0, s2 = 0;
      for (int v : ctx->sc) { const double b2 = (double)v * ts; s1 += b2; s2 += b2 * b2; mx = std::max<long long>(mx, (long long)v * ts); }
      const double nn = (double)ctx->sc.size();
      mean = s1 / nn;
      cv = mean > 0 ? std::sqrt(std::max(0.0, s2 / nn - mean * mean)) / mean : 0.0;
    }
    rbv_choice ch;
    std::memset(&ch, 0, sizeof ch);
    ch.algo = ALG_SPREADOUT; ch.r = 2;
    if (mean >= 0) rbv_tuner_choose(P, c.nproc(), mean, cv, &ch);
    spec = mk(ch.algo, ch.n, ch.r, ch.r2, ch.b, ch.b2);
    spec.P = P;
    const DevPlan* dp = nullptr;
    try { dp = c.plan_for(spec); } catch (const std::exception&) { dp = nullptr; }
    if (!dp || dp->plan.err) { spec = mk_spreadout(); spec.P = P; ch.eager = 0; }   // a table entry that does not fit this communicator
    // eager needs one cell size on all processes: known only where the whole matrix is
    ctx->eager = (ch.eager && L == P && mx > 0 && mx <= (256 << 10) &&
                  (unsigned long long)(P + 64) * (2ull * mx + 16) <= c.layout().arena_bytes) ? (unsigned long long)mx : 0ull;
    ctx->last_choice = ch;
  }
  struct Restore { rbv_ctx_s* c; unsigned long long e; bool on; ~Restore() { if (on) c->eager = e; } } restore{ctx, saved_eager, automatic};
  // The call is resolved once and kept: a loop that repeats the same collective (same buffers, counts and
  // parameters) pays for the resolution once and then for one kernel launch per iteration.
  std::vector<char> key;
  auto put = [&](const void* p, size_t n) { key.insert(key.end(), static_cast<const char*>(p), static_cast<const char*>(p) + n); };
  put(&spec, sizeof spec); put(&ts, sizeof ts); put(&flags, sizeof flags); put(&ctx->eager, sizeof ctx->eager);
  put(&ctx->grid, sizeof ctx->grid); put(&ctx->chunk, sizeof ctx->chunk); put(&have_rc, sizeof have_rc);
  put(ctx->sendbufs.data(), ctx->sendbufs.size() * sizeof(void*));
  put(ctx->recvbufs.data(), ctx->recvbufs.size() * sizeof(void*));
  put(ctx->sc.data(), ctx->sc.size() * sizeof(int)); put(ctx->rc.data(), ctx->rc.size() * sizeof(int));
  put(ctx->sd.data(), ctx->sd.size() * sizeof(long long)); put(ctx->rd.data(), ctx->rd.size() * sizeof(long long));
  if (!ctx->cached || key != ctx->cached_key) {
    if (ctx->cached) { cudaStreamSynchronize(ctx->stream); rbv_prepared_free(ctx, ctx->cached); ctx->cached = nullptr; }
    ctx->cached = rbv_prepare(ctx, spec.algo, spec.n, spec.r, spec.r2, spec.b, spec.b2, ts, ctx->sendbufs.data(),
                              ctx->recvbufs.data(), ctx->sc.data(), have_rc ? ctx->rc.data() : nullptr, ctx->sd.data(),
                              ctx->rd.data(), 0, -1, flags, ctx->grid, ctx->chunk);
    if (!ctx->cached) {
      ctx->cached_key.clear();
      return ctx->last_rc ? ctx->last_rc : (int)RBV_ERR_BAD_ARG;
    }
    ctx->cached_key.swap(key);
  }
  return rbv_launch(ctx, ctx->cached, ctx->stream);
}



int uniform_call(const AlgoSpec& s, char* sendbuf, int sendcount, int ts, char* recvbuf, int recvcount,
                 rbv_comm_t comm) {
  if (!comm) return RBV_ERR_BAD_ARG;
  const int P = comm->ctx->c->P();
  std::vector<int> sc(P, sendcount), rc(P, recvcount), sd(P), rd(P);
  for (int i = 0; i < P; i++) { sd[i] = i * sendcount; rd[i] = i * recvcount; }
  return enqueue(comm, s, ts, sendbuf, sc.data(), sd.data(), recvbuf, rc.data(), rd.data(), 0);
}

}  // namespace

extern "C" {

#define RBV_V_ARGS                                                                                      \
  char *sendbuf, int *sendcounts, int *sdispls, rbv_datatype sendtype, char *recvbuf, int *recvcounts, \
      int *rdispls, rbv_datatype recvtype, rbv_comm_t comm
#define RBV_V_PASS(spec, flags) \
  ((void)recvtype, enqueue(comm, spec, sendtype, sendbuf, sendcounts, sdispls, recvbuf, recvcounts, rdispls, flags))

int twophase_rbruck_alltoallv(int r, RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_RBRUCK, 0, r), 0); }
int twophase_rbruck_alltoallv_om(int r, RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_RBRUCK_OM, 0, r), 0); }
int tuna_algorithm(int r, int b, RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_TUNA, 0, r, 0, b), 0); }
int tuna2_algorithm(int r, int b, RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_TUNA2, 0, r, 0, b), 0); }
int TTPL_rbruck_alltoallv(int n, int r, RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_TTPL, n, r), 0); }
int TTPL_BT_alltoallv(int n, int r, int bblock, RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_TTPL_BT, n, r, 0, bblock), 0); }
int TTPL_BT_alltoallv_s1(int n, int r, int bblock, RBV_V_ARGS) {
  return RBV_V_PASS(mk(ALG_TTPL_BT_S1, n, r, 0, bblock), 0);
}
// sendbuf == NULL: the data to send is taken from recvbuf (src/twophase_twolayer_rbruck.cpp:702-709).
int TTPL_BT_alltoallv_s2(int n, int r, int bblock, RBV_V_ARGS) {
  return RBV_V_PASS(mk(ALG_TTPL_BT_S2, n, r, 0, bblock), sendbuf ? 0u : (unsigned)CALL_INPLACE);
}
int MPICH_intra_scattered(int bblock, RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_SCATTERED, 0, 2, 0, bblock), 0); }
int ompi_alltoallv_intra_basic_linear(RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_LINEAR), 0); }
int ompi_alltoallv_intra_pairwise(RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_PAIRWISE), 0); }
int exclisive_or_alltoallv(RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_XOR), 0); }
int exclusive_or_alltoallv(RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_XOR), 0); }
int twolayer_communicator_linear(int n, RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_TWOLAYER_LINEAR, n), 0); }
int twolayer_communicator_linear_s2(int n, int bblock1, int bblock2, RBV_V_ARGS) {
  return RBV_V_PASS(mk(ALG_TWOLAYER_LINEAR_S2, n, 2, 0, bblock1, bblock2), 0);
}
int twolayer_communicator_linear_s3(int n, int bblock1, int bblock2, RBV_V_ARGS) {
  return RBV_V_PASS(mk(ALG_TWOLAYER_LINEAR_S3, n, 2, 0, bblock1, bblock2), 0);
}
int twolayer_communicator_linear_s4(int n, int bblock1, int bblock2, RBV_V_ARGS) {
  return RBV_V_PASS(mk(ALG_TWOLAYER_LINEAR_S4, n, 2, 0, bblock1, bblock2), 0);
}
// benchmarks/merge_benchmark.cpp:155-332, benchmarks/simple_merge_benchmark.cpp:138-210,
// benchmarks/split_benchmark.cpp:147-205 (functions of the reference's benchmark programs, same argument order)
int merge_alltoallv(int ncores, RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_MERGE, ncores), 0); }
int simply_merge_alltoallv(int ncores, RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_SIMPLE_MERGE, ncores), 0); }
int split_alltoallv(RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_SPLIT), 0); }
// algo -1: resolved by the tuner once all local ranks have made their call
int rbv_alltoallv_auto(RBV_V_ARGS) { return RBV_V_PASS(mk(-1), 0); }
int ML_benchmark(RBV_V_ARGS) { return RBV_V_PASS(mk(-1), 0); }
// the configuration the latest automatic call resolved to
void rbv_ctx_last_choice(rbv_ctx_t ctx, rbv_choice* out) { *out = ctx->last_choice; }
void spreadout_alltoallv(RBV_V_ARGS) { (void)RBV_V_PASS(mk(ALG_SPREADOUT), 0); }

int uniform_spreadout_twolayer(int n, int r, char* sendbuf, int sendcount, rbv_datatype sendtype, char* recvbuf,
                               int recvcount, rbv_datatype recvtype, rbv_comm_t comm) {
  (void)recvtype;
  return uniform_call(mk(ALG_UNIFORM_SPREADOUT_TWOLAYER, n, r), sendbuf, sendcount, sendtype, recvbuf, recvcount, comm);
}
void uniform_inverse_isplit_r_bruck(int n, int r1, int r2, char* sendbuf, int sendcount, rbv_datatype sendtype,
                                    char* recvbuf, int recvcount, rbv_datatype recvtype, rbv_comm_t comm) {
  (void)recvtype;
  (void)uniform_call(mk(ALG_UNIFORM_ISPLIT_RBRUCK, n, r1, r2), sendbuf, sendcount, sendtype, recvbuf, recvcount, comm);
}

}  // extern "C"
