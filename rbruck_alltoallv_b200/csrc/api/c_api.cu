// C API: context management and the reference-shaped collective entry points (rbv/rbruckv.h).
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

void rbv_ctx_destroy(rbv_ctx_t ctx) { delete ctx; }

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

void* rbv_prepare(rbv_ctx_t ctx, int algo, int n, int r, int r2, int b, int b2, int type_size,
                  const void* const* sendbufs, void* const* recvbufs, const int* sendcounts,
                  const int* recvcounts, const long long* sdispls, const long long* rdispls,
                  int counts_on_device, long long bytes_hint, unsigned flags, int grid, size_t chunk_bytes) {
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
    auto pc = std::make_unique<Prepared>();
    int rc = ctx->c->prepare(s, type_size, ca, opt, nullptr, true, pc.get());
    if (rc) { g_err = ctx->c->last_error(); return nullptr; }
    return pc.release();
  } catch (const std::exception& e) {
    g_err = e.what();
    return nullptr;
  }
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
void rbv_ctx_set_eager(rbv_ctx_t ctx, unsigned long long max_block_bytes) { ctx->eager = max_block_bytes; }
void rbv_ctx_set_trace(rbv_ctx_t ctx, int on) { ctx->c->set_trace(on != 0); }
void rbv_ctx_set_bulk(rbv_ctx_t ctx, int mode) { ctx->c->set_bulk(mode); }
void rbv_ctx_set_cooperative(rbv_ctx_t ctx, int on) { ctx->c->set_cooperative(on != 0); }

int rbv_update_timers(rbv_ctx_t ctx) {
  StatusBlock s = ctx->c->status(ctx->stream);
  auto sec = [&](int a, int b) { return s.trace[b] > s.trace[a] ? (double)(s.trace[b] - s.trace[a]) * 1e-9 : 0.0; };
  init_time = 0;
  // metadata phase = what the reference spends in its max-count allreduce and per-round count exchanges
  findMax_time = sec(0, 1);
  excgMeta_time = sec(1, 2);
  rotateIndex_time = alcCopy_time = getBlock_time = prepData_time = replace_time = orgData_time = prepSP_time = 0;
  excgData_time = sec(2, 3);
  SP_time = sec(3, 4);
  intra_time = sec(2, 3);
  return s.code;
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

int enqueue(rbv_comm_t comm, const AlgoSpec& spec_in, int ts, const char* sendbuf, const int* sendcounts,
            const int* sdispls, char* recvbuf, const int* recvcounts, const int* rdispls, unsigned flags) {
  if (!comm) { g_err = "null communicator"; return RBV_ERR_BAD_ARG; }
  rbv_ctx_s* ctx = comm->ctx;
  Context& c = *ctx->c;
  const int P = c.P(), L = c.L(), lr = comm->local;
  AlgoSpec spec = spec_in;
  spec.P = P;
  // argument validation happens in the plan compiler; evaluate it now so that every rank gets the code
  try {
    const DevPlan* dp = c.plan_for(spec);
    if (dp->plan.err) { g_err = dp->plan.errmsg; return dp->plan.err; }
  } catch (const std::exception& e) { g_err = e.what(); return RBV_ERR_BAD_ARG; }
  if (ctx->pend == 0) {
    ctx->spec = spec; ctx->ts = ts; ctx->flags = flags;
  } else if (std::memcmp(&ctx->spec, &spec, sizeof spec) != 0 || ctx->ts != ts || ctx->flags != flags) {
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
  int rc = rbv_alltoallv(ctx, spec.algo, spec.n, spec.r, spec.r2, spec.b, spec.b2, ts, ctx->sendbufs.data(),
                         ctx->recvbufs.data(), ctx->sc.data(), have_rc ? ctx->rc.data() : nullptr, ctx->sd.data(),
                         ctx->rd.data(), 0, -1, flags, ctx->grid, ctx->chunk, ctx->stream);
  return rc;
}

AlgoSpec mk(int algo, int n = 0, int r = 2, int r2 = 0, int b = 0, int b2 = 0) {
  AlgoSpec s;
  s.algo = algo; s.n = n; s.r = r; s.r2 = r2; s.b = b; s.b2 = b2;
  return s;
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
int ML_benchmark(RBV_V_ARGS) { return RBV_V_PASS(mk(ALG_SPREADOUT), 0); }
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
