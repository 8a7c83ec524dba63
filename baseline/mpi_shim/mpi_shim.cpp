// Threads-as-ranks implementation of the MPI subset declared in mpi.h.
//
// Point-to-point: eager protocol.  A send looks for a matching posted receive in the destination's
// mailbox and copies straight into the user buffer; otherwise it leaves a heap copy in the mailbox
// ("unexpected message").  Matching follows MPI's rules: (communicator, source, tag), first posted /
// first sent wins.  Sends therefore complete immediately and the shim cannot deadlock on
// send-before-receive orderings.  Collectives publish buffer pointers in the communicator record and
// copy between address spaces directly (all ranks share one address space).
#include "mpi.h"

#include <sched.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
static inline void cpu_relax() { _mm_pause(); }
#else
static inline void cpu_relax() {}
#endif

namespace {

struct Backoff {
  unsigned n = 0;
  void pause() {
    if (++n < 2000) cpu_relax();
    else sched_yield();
  }
};

struct CommRec {
  std::vector<int> members;  // world ranks, in communicator rank order
  std::atomic<int> count{0};
  std::atomic<int> gen{0};
  // scratch for collectives, one slot per member
  std::vector<const void*> pa, pb, pc;
  std::vector<int> ia, ib;
  std::vector<int> handle_slot;
  explicit CommRec(std::vector<int> m) : members(std::move(m)) {
    size_t n = members.size();
    pa.assign(n, nullptr); pb.assign(n, nullptr); pc.assign(n, nullptr);
    ia.assign(n, 0); ib.assign(n, 0); handle_slot.assign(n, -1);
  }
};

struct Msg {
  int src, tag, comm;
  size_t bytes;
  char* data;
};

struct Mailbox {
  std::mutex mu;
  std::deque<Msg> unexpected;
  std::deque<shim_request*> posted;
};

// Communicator table: slots are written once under the mutex and then only read.
constexpr int kMaxComms = 1 << 16;
std::mutex g_comm_mu;
std::atomic<CommRec*> g_comms[kMaxComms];
int g_ncomms = 0;
int add_comm(std::vector<int> members) {  // caller holds g_comm_mu
  if (g_ncomms >= kMaxComms) { std::fprintf(stderr, "[mpi shim] too many communicators\n"); std::_Exit(1); }
  g_comms[g_ncomms].store(new CommRec(std::move(members)), std::memory_order_release);
  return g_ncomms++;
}
std::vector<std::unique_ptr<Mailbox>> g_boxes;
int g_world = 0;
thread_local int tl_rank = 0;
const auto g_t0 = std::chrono::steady_clock::now();

CommRec& comm_rec(MPI_Comm c) { return *g_comms[(size_t)c].load(std::memory_order_acquire); }
int comm_rank_of(const CommRec& c, int world) {
  for (size_t i = 0; i < c.members.size(); i++)
    if (c.members[i] == world) return (int)i;
  return -1;
}
void barrier(CommRec& c) {
  const int n = (int)c.members.size();
  if (n <= 1) return;
  const int gen = c.gen.load(std::memory_order_acquire);
  if (c.count.fetch_add(1, std::memory_order_acq_rel) == n - 1) {
    c.count.store(0, std::memory_order_relaxed);
    c.gen.fetch_add(1, std::memory_order_release);
  } else {
    Backoff b;
    while (c.gen.load(std::memory_order_acquire) == gen) b.pause();
  }
}

size_t type_size(MPI_Datatype t) {
  switch (t) {
    case MPI_CHAR: case MPI_BYTE: case MPI_UNSIGNED_CHAR: return 1;
    case MPI_INT: case MPI_FLOAT: case MPI_UNSIGNED: return 4;
    case MPI_DOUBLE: case MPI_LONG_LONG: case MPI_UNSIGNED_LONG_LONG: case MPI_LONG: return 8;
    case MPI_DOUBLE_INT: return 16;
    default: return 1;
  }
}

}  // namespace

struct shim_request {
  std::atomic<int> done{0};
  void* buf = nullptr;
  size_t cap = 0;
  int src = 0, tag = 0, comm = 0;  // src is a world rank or MPI_ANY_SOURCE
  MPI_Status st{};
};

namespace {
bool matches(const shim_request* r, int src, int tag, int comm) {
  return r->comm == comm && (r->src == MPI_ANY_SOURCE || r->src == src) && (r->tag == MPI_ANY_TAG || r->tag == tag);
}
void complete_recv(shim_request* r, const void* data, size_t bytes, int src_world, int tag) {
  size_t n = bytes < r->cap ? bytes : r->cap;
  if (n) std::memcpy(r->buf, data, n);
  r->st.MPI_SOURCE = comm_rank_of(comm_rec(r->comm), src_world);
  r->st.MPI_TAG = tag;
  r->st.MPI_ERROR = bytes > r->cap ? MPI_ERR_OTHER : MPI_SUCCESS;
  r->st.count_bytes = (int)n;
  r->done.store(1, std::memory_order_release);
}

void do_send(const void* buf, size_t bytes, int dest_world, int tag, int comm) {
  Mailbox& mb = *g_boxes[(size_t)dest_world];
  auto try_match = [&]() -> shim_request* {
    for (auto it = mb.posted.begin(); it != mb.posted.end(); ++it)
      if (matches(*it, tl_rank, tag, comm)) {
        shim_request* r = *it;
        mb.posted.erase(it);
        return r;
      }
    return nullptr;
  };
  shim_request* r;
  {
    std::lock_guard<std::mutex> lk(mb.mu);
    r = try_match();
  }
  if (r) { complete_recv(r, buf, bytes, tl_rank, tag); return; }
  char* copy = bytes ? (char*)std::malloc(bytes) : nullptr;
  if (bytes) std::memcpy(copy, buf, bytes);
  {
    std::lock_guard<std::mutex> lk(mb.mu);
    r = try_match();
    if (!r) mb.unexpected.push_back(Msg{tl_rank, tag, comm, bytes, copy});
  }
  if (r) { complete_recv(r, buf, bytes, tl_rank, tag); std::free(copy); }
}

void post_recv(shim_request* r) {
  Mailbox& mb = *g_boxes[(size_t)tl_rank];
  Msg m{};
  bool found = false;
  {
    std::lock_guard<std::mutex> lk(mb.mu);
    for (auto it = mb.unexpected.begin(); it != mb.unexpected.end(); ++it)
      if (matches(r, it->src, it->tag, it->comm)) {
        m = *it;
        mb.unexpected.erase(it);
        found = true;
        break;
      }
    if (!found) mb.posted.push_back(r);
  }
  if (found) {
    complete_recv(r, m.data, m.bytes, m.src, m.tag);
    std::free(m.data);
  }
}

void wait_req(shim_request* r) {
  Backoff b;
  while (!r->done.load(std::memory_order_acquire)) b.pause();
}

template <typename T>
void reduce_typed(const CommRec& c, void* out, int count, MPI_Op op) {
  T* o = static_cast<T*>(out);
  for (int i = 0; i < count; i++) {
    T acc = static_cast<const T*>(c.pa[0])[i];
    for (size_t m = 1; m < c.members.size(); m++) {
      T v = static_cast<const T*>(c.pa[m])[i];
      if (op == MPI_MAX) acc = v > acc ? v : acc;
      else if (op == MPI_MIN) acc = v < acc ? v : acc;
      else acc = acc + v;
    }
    o[i] = acc;
  }
}
struct DoubleInt { double v; int i; };
}  // namespace

extern "C" {

int MPI_Init(int*, char***) { return MPI_SUCCESS; }
int MPI_Finalize(void) { return MPI_SUCCESS; }
int MPI_Abort(MPI_Comm, int code) {
  std::fprintf(stderr, "[mpi shim] MPI_Abort(%d) on rank %d\n", code, tl_rank);
  std::fflush(nullptr);
  std::_Exit(code ? (code & 0xff) | 1 : 1);
}
double MPI_Wtime(void) {
  return std::chrono::duration<double>(std::chrono::steady_clock::now() - g_t0).count();
}
int MPI_Comm_rank(MPI_Comm comm, int* rank) { *rank = comm_rank_of(comm_rec(comm), tl_rank); return MPI_SUCCESS; }
int MPI_Comm_size(MPI_Comm comm, int* size) { *size = (int)comm_rec(comm).members.size(); return MPI_SUCCESS; }

int MPI_Comm_split(MPI_Comm comm, int color, int key, MPI_Comm* newcomm) {
  CommRec& c = comm_rec(comm);
  const int me = comm_rank_of(c, tl_rank), n = (int)c.members.size();
  c.ia[me] = color; c.ib[me] = key;
  barrier(c);
  std::vector<std::pair<std::pair<int, int>, int>> grp;  // ((key, parent rank), world)
  for (int i = 0; i < n; i++)
    if (c.ia[i] == color) grp.push_back({{c.ib[i], i}, c.members[i]});
  std::sort(grp.begin(), grp.end());
  const int leader = grp.front().first.second;
  if (color == MPI_UNDEFINED) {
    barrier(c); barrier(c);
    *newcomm = MPI_COMM_NULL;
    return MPI_SUCCESS;
  }
  if (leader == me) {
    std::vector<int> members;
    for (auto& g : grp) members.push_back(g.second);
    std::lock_guard<std::mutex> lk(g_comm_mu);
    c.handle_slot[me] = add_comm(members);
  }
  barrier(c);
  *newcomm = c.handle_slot[leader];
  barrier(c);
  return MPI_SUCCESS;
}
int MPI_Comm_free(MPI_Comm* comm) { *comm = MPI_COMM_NULL; return MPI_SUCCESS; }
int MPI_Intercomm_create(MPI_Comm, int, MPI_Comm, int, int, MPI_Comm* out) {
  std::fprintf(stderr, "[mpi shim] MPI_Intercomm_create is not supported\n");
  *out = MPI_COMM_NULL;
  return MPI_ERR_OTHER;
}
int MPI_Type_size(MPI_Datatype t, int* size) { *size = (int)type_size(t); return MPI_SUCCESS; }
int MPI_Type_extent(MPI_Datatype t, MPI_Aint* extent) { *extent = (MPI_Aint)type_size(t); return MPI_SUCCESS; }
int MPI_Barrier(MPI_Comm comm) { barrier(comm_rec(comm)); return MPI_SUCCESS; }

int MPI_Allreduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype t, MPI_Op op, MPI_Comm comm) {
  CommRec& c = comm_rec(comm);
  const int me = comm_rank_of(c, tl_rank);
  c.pa[me] = sendbuf;
  barrier(c);
  if (t == MPI_DOUBLE_INT && op == MPI_MAXLOC) {
    DoubleInt* o = static_cast<DoubleInt*>(recvbuf);
    for (int i = 0; i < count; i++) {
      DoubleInt acc = static_cast<const DoubleInt*>(c.pa[0])[i];
      for (size_t m = 1; m < c.members.size(); m++) {
        DoubleInt v = static_cast<const DoubleInt*>(c.pa[m])[i];
        if (v.v > acc.v || (v.v == acc.v && v.i < acc.i)) acc = v;
      }
      o[i] = acc;
    }
  } else if (t == MPI_INT) reduce_typed<int>(c, recvbuf, count, op);
  else if (t == MPI_DOUBLE) reduce_typed<double>(c, recvbuf, count, op);
  else if (t == MPI_FLOAT) reduce_typed<float>(c, recvbuf, count, op);
  else if (t == MPI_LONG_LONG || t == MPI_LONG) reduce_typed<long long>(c, recvbuf, count, op);
  else if (t == MPI_UNSIGNED_LONG_LONG) reduce_typed<unsigned long long>(c, recvbuf, count, op);
  else { barrier(c); return MPI_ERR_OTHER; }
  barrier(c);
  return MPI_SUCCESS;
}

int MPI_Alltoall(const void* sendbuf, int sendcount, MPI_Datatype st, void* recvbuf, int recvcount, MPI_Datatype rt,
                 MPI_Comm comm) {
  CommRec& c = comm_rec(comm);
  const int me = comm_rank_of(c, tl_rank), n = (int)c.members.size();
  const size_t sb = (size_t)sendcount * type_size(st), rb = (size_t)recvcount * type_size(rt);
  c.pa[me] = sendbuf;
  barrier(c);
  for (int k = 0; k < n; k++) {
    int s = (me + k) % n;
    std::memcpy(static_cast<char*>(recvbuf) + (size_t)s * rb, static_cast<const char*>(c.pa[s]) + (size_t)me * sb,
                sb < rb ? sb : rb);
  }
  barrier(c);
  return MPI_SUCCESS;
}

int MPI_Alltoallv(const void* sendbuf, const int* sendcounts, const int* sdispls, MPI_Datatype st, void* recvbuf,
                  const int* recvcounts, const int* rdispls, MPI_Datatype rt, MPI_Comm comm) {
  CommRec& c = comm_rec(comm);
  const int me = comm_rank_of(c, tl_rank), n = (int)c.members.size();
  const size_t ss = type_size(st), rs = type_size(rt);
  c.pa[me] = sendbuf; c.pb[me] = sendcounts; c.pc[me] = sdispls;
  barrier(c);
  for (int k = 0; k < n; k++) {
    int s = (me + k) % n;
    const int* scnt = static_cast<const int*>(c.pb[s]);
    const int* sdsp = static_cast<const int*>(c.pc[s]);
    size_t bytes = (size_t)scnt[me] * ss, cap = (size_t)recvcounts[s] * rs;
    if (bytes > cap) bytes = cap;
    if (bytes)
      std::memcpy(static_cast<char*>(recvbuf) + (size_t)rdispls[s] * rs,
                  static_cast<const char*>(c.pa[s]) + (size_t)sdsp[me] * ss, bytes);
  }
  barrier(c);
  return MPI_SUCCESS;
}

int MPI_Gather(const void* sendbuf, int sendcount, MPI_Datatype st, void* recvbuf, int recvcount, MPI_Datatype rt,
               int root, MPI_Comm comm) {
  CommRec& c = comm_rec(comm);
  const int me = comm_rank_of(c, tl_rank), n = (int)c.members.size();
  c.pa[me] = sendbuf;
  barrier(c);
  if (me == root)
    for (int s = 0; s < n; s++)
      std::memcpy(static_cast<char*>(recvbuf) + (size_t)s * recvcount * type_size(rt), c.pa[s],
                  (size_t)sendcount * type_size(st));
  barrier(c);
  return MPI_SUCCESS;
}

int MPI_Scatter(const void* sendbuf, int sendcount, MPI_Datatype st, void* recvbuf, int recvcount, MPI_Datatype rt,
                int root, MPI_Comm comm) {
  CommRec& c = comm_rec(comm);
  const int me = comm_rank_of(c, tl_rank);
  if (me == root) c.pa[root] = sendbuf;
  barrier(c);
  std::memcpy(recvbuf, static_cast<const char*>(c.pa[root]) + (size_t)me * sendcount * type_size(st),
              (size_t)recvcount * type_size(rt));
  barrier(c);
  return MPI_SUCCESS;
}

int MPI_Isend(const void* buf, int count, MPI_Datatype t, int dest, int tag, MPI_Comm comm, MPI_Request* req) {
  CommRec& c = comm_rec(comm);
  if (dest < 0 || dest >= (int)c.members.size()) return MPI_ERR_OTHER;
  do_send(buf, (size_t)count * type_size(t), c.members[dest], tag, comm);
  shim_request* r = new shim_request;
  r->done.store(1, std::memory_order_relaxed);
  *req = r;
  return MPI_SUCCESS;
}
int MPI_Irecv(void* buf, int count, MPI_Datatype t, int source, int tag, MPI_Comm comm, MPI_Request* req) {
  CommRec& c = comm_rec(comm);
  if (source != MPI_ANY_SOURCE && (source < 0 || source >= (int)c.members.size())) return MPI_ERR_OTHER;
  shim_request* r = new shim_request;
  r->buf = buf; r->cap = (size_t)count * type_size(t);
  r->src = source == MPI_ANY_SOURCE ? MPI_ANY_SOURCE : c.members[source];
  r->tag = tag; r->comm = comm;
  *req = r;
  post_recv(r);
  return MPI_SUCCESS;
}
int MPI_Wait(MPI_Request* req, MPI_Status* status) {
  if (!req || !*req) return MPI_SUCCESS;
  wait_req(*req);
  if (status) *status = (*req)->st;
  int err = (*req)->st.MPI_ERROR;
  delete *req;
  *req = MPI_REQUEST_NULL;
  return err;
}
int MPI_Waitall(int count, MPI_Request* reqs, MPI_Status* statuses) {
  int err = MPI_SUCCESS;
  for (int i = 0; i < count; i++) {
    int e = MPI_Wait(&reqs[i], statuses ? &statuses[i] : MPI_STATUS_IGNORE);
    if (e != MPI_SUCCESS) err = e;
  }
  return err;
}
int MPI_Send(const void* buf, int count, MPI_Datatype t, int dest, int tag, MPI_Comm comm) {
  MPI_Request r;
  int e = MPI_Isend(buf, count, t, dest, tag, comm, &r);
  if (e != MPI_SUCCESS) return e;
  return MPI_Wait(&r, MPI_STATUS_IGNORE);
}
int MPI_Recv(void* buf, int count, MPI_Datatype t, int source, int tag, MPI_Comm comm, MPI_Status* status) {
  MPI_Request r;
  int e = MPI_Irecv(buf, count, t, source, tag, comm, &r);
  if (e != MPI_SUCCESS) return e;
  return MPI_Wait(&r, status);
}
int MPI_Sendrecv(const void* sendbuf, int sendcount, MPI_Datatype st, int dest, int sendtag, void* recvbuf,
                 int recvcount, MPI_Datatype rt, int source, int recvtag, MPI_Comm comm, MPI_Status* status) {
  MPI_Request rr, rs;
  int e = MPI_Irecv(recvbuf, recvcount, rt, source, recvtag, comm, &rr);
  if (e != MPI_SUCCESS) return e;
  e = MPI_Isend(sendbuf, sendcount, st, dest, sendtag, comm, &rs);
  if (e != MPI_SUCCESS) return e;
  MPI_Wait(&rs, MPI_STATUS_IGNORE);
  return MPI_Wait(&rr, status);
}

int shim_run(int nranks, shim_rank_fn fn, void* arg) {
  if (nranks < 1) return 1;
  {
    std::lock_guard<std::mutex> lk(g_comm_mu);
    for (int i = 0; i < g_ncomms; i++) delete g_comms[i].exchange(nullptr);
    g_ncomms = 0;
    std::vector<int> world(nranks);
    for (int i = 0; i < nranks; i++) world[i] = i;
    add_comm(world);
  }
  g_boxes.clear();
  for (int i = 0; i < nranks; i++) g_boxes.push_back(std::make_unique<Mailbox>());
  g_world = nranks;
  std::vector<std::thread> th;
  for (int i = 0; i < nranks; i++)
    th.emplace_back([=]() { tl_rank = i; fn(i, nranks, arg); });
  for (auto& t : th) t.join();
  return 0;
}

}  // extern "C"
