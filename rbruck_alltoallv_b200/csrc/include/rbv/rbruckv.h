/* Public C API.
 *
 * The collective entry points keep the names, argument order and return conventions of the
 * reference's src/rbruckv.h:20-96 (including the `exclisive_or_alltoallv` spelling).  Two types
 * change: MPI_Datatype becomes rbv_datatype (the element size in bytes, which is all the reference
 * ever reads from a datatype) and MPI_Comm becomes rbv_comm_t.  Buffers are device pointers;
 * receive buffers come from rbv_symm_alloc(), count / displacement arrays are host arrays in
 * elements, exactly as with MPI_Alltoallv.
 *
 * Process model: one process per GPU creates one rbv_ctx_t; the context hosts L = nranks / nproc
 * logical ranks and hands out one rbv_comm_t per local rank.  A collective is called once per
 * local rank, like an SPMD program would; the kernel is launched when the last local rank of the
 * process has made its call (L = 1: immediately).  Calls are asynchronous on the context's stream.
 *
 * Return codes: 0 success; -1 invalid radix / rank count (as the reference); -2 invalid group size
 * (the reference calls MPI_Abort there); > 0 an rbv_status detected on the host.  Errors detected
 * on the device (time-out, truncation, staging capacity) are read with rbv_ctx_status().
 */
#ifndef RBV_RBRUCKV_H_
#define RBV_RBRUCKV_H_

#include <stddef.h>

#ifdef __cplusplus
#include <vector>
extern "C" {
#endif

typedef struct rbv_ctx_s* rbv_ctx_t;
typedef struct rbv_comm_s* rbv_comm_t;
typedef int rbv_datatype; /* element size in bytes */

#define RBV_CHAR 1
#define RBV_BF16 2
#define RBV_INT 4
#define RBV_FLOAT 4
#define RBV_LONG_LONG 8
#define RBV_UNSIGNED_LONG_LONG 8
#define RBV_DOUBLE 8
#define RBV_COMPLEX64 8

typedef struct rbv_status_s {
  int code;    /* 0 ok, 1 time-out, 2 bad argument, 3 staging capacity, 4 truncation, 5 aborted by a peer */
  int site;    /* for time-outs: 1 metadata, 2 staging cell, 3 final arrival */
  int detail0;
  int detail1;
  unsigned long long trace[8]; /* device clock (ns): start, metadata published, metadata complete,
                                  own transfers issued, all blocks received */
} rbv_status;

/* ---- context / communicator ---- */
rbv_ctx_t rbv_ctx_create(int nranks, int nproc, int proc, int device, size_t user_bytes, size_t arena_bytes);
void rbv_ctx_destroy(rbv_ctx_t ctx);
const char* rbv_last_error(void);
int rbv_ctx_ipc_handle(rbv_ctx_t ctx, void* out64);
int rbv_ctx_connect(rbv_ctx_t ctx, const void* handles);
void rbv_ctx_set_stream(rbv_ctx_t ctx, void* cuda_stream);
void rbv_ctx_set_timeout_ms(rbv_ctx_t ctx, double ms);
void rbv_ctx_set_launch(rbv_ctx_t ctx, int grid, size_t chunk_bytes); /* 0 = automatic */
void rbv_ctx_set_absent_rank(rbv_ctx_t ctx, int local_rank); /* test hook: rank skips the metadata phase; -1 off */
int rbv_ctx_sync(rbv_ctx_t ctx);
int rbv_ctx_status(rbv_ctx_t ctx, rbv_status* out); /* synchronises the stream */
int rbv_ctx_reset(rbv_ctx_t ctx);
int rbv_ctx_info(rbv_ctx_t ctx, long long* out8); /* P, L, nproc, proc, device, seq, max_ctas, sm_count */
void* rbv_ctx_heap(rbv_ctx_t ctx, int proc);
int rbv_ctx_in_heap(rbv_ctx_t ctx, const void* ptr, size_t bytes); /* 1 if [ptr, ptr+bytes) lies in the symmetric heap */
void* rbv_symm_alloc(rbv_ctx_t ctx, size_t bytes);
int rbv_symm_free(rbv_ctx_t ctx, void* ptr);
rbv_comm_t rbv_comm(rbv_ctx_t ctx, int local_rank);
int rbv_comm_rank(rbv_comm_t comm);
int rbv_comm_size(rbv_comm_t comm);

/* Generic entry: all local ranks at once.  Arrays are [L] pointers and [L][P] counts
 * (64-bit displacements); `counts_on_device` != 0 means the four count arrays are device memory.
 * algo is an rbv::Algo value. */
int rbv_alltoallv(rbv_ctx_t ctx, int algo, int n, int r, int r2, int b, int b2, int type_size,
                  const void* const* sendbufs, void* const* recvbufs, const int* sendcounts,
                  const int* recvcounts, const long long* sdispls, const long long* rdispls,
                  int counts_on_device, long long bytes_hint, unsigned flags, int grid, size_t chunk_bytes,
                  void* cuda_stream);

/* Persistent form (the analogue of MPI_Alltoallv_init / MPI_Start): resolve a call once, launch it many
 * times with one cheap call each.  Buffers and counts are fixed at preparation. */
void* rbv_prepare(rbv_ctx_t ctx, int algo, int n, int r, int r2, int b, int b2, int type_size,
                  const void* const* sendbufs, void* const* recvbufs, const int* sendcounts,
                  const int* recvcounts, const long long* sdispls, const long long* rdispls,
                  int counts_on_device, long long bytes_hint, unsigned flags, int grid, size_t chunk_bytes);
/* The same with the arguments of the whole communicator, gathered by the caller on the host: g_counts[s * P + d]
 * (what rank s sends to rank d), g_caps[d * P + s] (recvcounts of rank d, -1 unchecked; may be null),
 * g_rdispls[d * P + s], g_recvoff[d] (byte offset of rank d's receive buffer in its process's heap).  With them a
 * call with host-side counts is resolved completely on the host and runs without a metadata phase; every
 * process must then pass them.  A process that hosts all ranks gets this from rbv_prepare already.
 * flags: bit 0 in-place, bit 8 keep the dynamic kernel even where the static one is possible, bit 9 the receive
 * buffers of a single-process static call may lie outside the symmetric heap (any device-accessible memory, pinned
 * host memory included); the caller then answers for displacement + count staying inside them. */
void* rbv_prepare_global(rbv_ctx_t ctx, int algo, int n, int r, int r2, int b, int b2, int type_size,
                         const void* const* sendbufs, void* const* recvbufs, const int* sendcounts,
                         const int* recvcounts, const long long* sdispls, const long long* rdispls,
                         int counts_on_device, long long bytes_hint, unsigned flags, int grid, size_t chunk_bytes,
                         const int* g_counts, const int* g_caps, const long long* g_rdispls,
                         const unsigned long long* g_recvoff);
/* Which kernel a prepared call runs: 0 dynamic rendezvous, 1 eager, 2 static rendezvous;
 * out3 = grid, cooperative launch needed (0 / 1), work items. */
int rbv_prepared_info(void* prepared, long long* out3);
int rbv_launch(rbv_ctx_t ctx, void* prepared, void* cuda_stream);
void rbv_prepared_free(rbv_ctx_t ctx, void* prepared);
/* NVLS: keep the metadata tables in a caller-provided buffer that is bound to an NVLink multicast object (local
 * address, multicast address, at least rbv_ctx_meta_bytes() bytes, zero-filled); the metadata phase then publishes
 * with one multimem.st per unit instead of one store per peer.  Collective: all processes or none. */
int rbv_ctx_set_nvls_meta(rbv_ctx_t ctx, void* self_ptr, void* mc_ptr, size_t bytes);
size_t rbv_ctx_meta_bytes(rbv_ctx_t ctx);
/* The same with a multicast object that the library creates and binds itself (CUDA driver API), in collective steps
 * with a host barrier after each: process 0 calls rbv_ctx_nvls_create (bytes = rbv_ctx_meta_bytes) and passes the
 * file descriptor to the other processes (SCM_RIGHTS over a Unix socket) together with *size_out; they call
 * rbv_ctx_nvls_import; everybody calls rbv_ctx_nvls_add_device, then rbv_ctx_nvls_bind (allocates this GPU's buffer,
 * binds it, maps buffer and multicast view and switches the metadata tables over).  rbv_ctx_nvls_teardown undoes it
 * (also done when the context is destroyed).  Keep NVLS off in anything that tests failures: a process that dies
 * while bound to a multicast object disturbs the other GPUs. */
int rbv_ctx_nvls_create(rbv_ctx_t ctx, size_t bytes, int* fd_out, size_t* size_out);
int rbv_ctx_nvls_import(rbv_ctx_t ctx, int fd, size_t bytes);
int rbv_ctx_nvls_add_device(rbv_ctx_t ctx);
int rbv_ctx_nvls_bind(rbv_ctx_t ctx);
void rbv_ctx_nvls_teardown(rbv_ctx_t ctx);

/* Protocol of the following calls: 0 = rendezvous (any size); > 0 = eager, for blocks of at most this many bytes
 * (every rank must pass the same value; needs (P + cells) * (16 + 2 * bytes) of staging arena per rank). */
void rbv_ctx_set_eager(rbv_ctx_t ctx, unsigned long long max_block_bytes);
void rbv_ctx_set_trace(rbv_ctx_t ctx, int on);       /* report phase time stamps after every call */
void rbv_ctx_set_bulk(rbv_ctx_t ctx, int mode);      /* bulk-copy engine for large chunks: 0 off (default), 1 on, -1 by size */
void rbv_ctx_set_cooperative(rbv_ctx_t ctx, int mode); /* -1 where a call needs it (default), 0 never, 1 always */
void rbv_ctx_set_static(rbv_ctx_t ctx, int on);      /* 0: persistent calls keep the dynamic kernel */
/* For the next rbv_prepare* only: mirrors[L] (null entries: none) name where each local rank wants its received
 * blocks in the end, e.g. pinned host memory.  A call that runs the static kernel copies them there from the receive
 * buffers itself once everything has arrived, so the end of the launch is the end of the whole transfer; other calls
 * ignore it.  The caller answers for displacement + count staying inside the mirrors. */
void rbv_ctx_set_recv_mirror(rbv_ctx_t ctx, void* const* mirrors);
/* Time stamps (device clock, ns) per key of the schedule (a round, a batch; key = phase << 24 | step) of the most
 * recent traced call: earliest start and latest end over all warps of this process.  Returns the number filled. */
int rbv_ctx_last_trace(rbv_ctx_t ctx, unsigned* keys, unsigned long long* start_ns, unsigned long long* end_ns, int max);

/* ---- automatic choice ----
 * A configuration as the tuner's table of measured winners stores it. */
typedef struct rbv_choice_s {
  int algo;          /* rbv::Algo value */
  int n, r, r2, b, b2;
  int eager;         /* 1: eager protocol (blocks up to 256 KB), 0: rendezvous */
} rbv_choice;
/* Table file to read (default: $RBV_TUNER_CACHE; the Python package points this at its own copy). */
void rbv_tuner_set_table(const char* path);
int rbv_tuner_entries(void);
/* Winner for a communicator of P ranks on nproc processes, mean block size and coefficient of variation of the
 * block sizes.  Returns 1 when it comes from the table, 0 for the built-in rule. */
int rbv_tuner_choose(int P, int nproc, double mean_block_bytes, double cv, rbv_choice* out);
/* What the automatic entry points know about the whole exchange when a process hosts only some of the ranks:
 * mean block bytes and coefficient of variation, the same values on every process (mean < 0 forgets the hint;
 * without one, several processes use the spread-out order with the rendezvous protocol, which needs no agreement). */
void rbv_ctx_set_auto_hint(rbv_ctx_t ctx, double mean_block_bytes, double cv);
void rbv_ctx_last_choice(rbv_ctx_t ctx, rbv_choice* out); /* what the latest automatic call resolved to */

/* Phase timers of the most recent call, filled by rbv_update_timers() (which synchronises;
 * call rbv_ctx_set_trace(ctx, 1) first).
 * Names as in the reference (src/rbruckv.h:13-18); phases that no longer exist as separate steps
 * (pack, unpack, organise) stay 0. */
extern double init_time, findMax_time, rotateIndex_time, alcCopy_time, getBlock_time, prepData_time,
    excgMeta_time, excgData_time, replace_time, orgData_time, prepSP_time, SP_time;
extern double intra_time;
extern double* iteration_time;   /* one entry per inter-group batch, malloc'ed by rbv_update_timers, freed by the caller */
int rbv_update_timers(rbv_ctx_t ctx);
int rbv_iteration_count(rbv_ctx_t ctx); /* entries of iteration_time for the most recent call */

/* ---- helpers (src/utils.cpp) ---- */
int myPow(int x, unsigned int p);
int check_errors(int* recvcounts, long long* recv_buffer, int rank, int nprocs); /* host buffer */

/* ---- collectives, one call per local rank ---- */
int twophase_rbruck_alltoallv(int r, char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype,
                              char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int twophase_rbruck_alltoallv_om(int r, char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype,
                                 char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int tuna_algorithm(int r, int b, char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype,
                   char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int tuna2_algorithm(int r, int b, char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype,
                    char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int uniform_spreadout_twolayer(int n, int r, char* sendbuf, int sendcount, rbv_datatype sendtype, char* recvbuf,
                               int recvcount, rbv_datatype recvtype, rbv_comm_t comm);
void uniform_inverse_isplit_r_bruck(int n, int r1, int r2, char* sendbuf, int sendcount, rbv_datatype sendtype,
                                    char* recvbuf, int recvcount, rbv_datatype recvtype, rbv_comm_t comm);
int TTPL_rbruck_alltoallv(int n, int r, char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype,
                          char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int TTPL_BT_alltoallv(int n, int r, int bblock, char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype,
                      char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int TTPL_BT_alltoallv_s1(int n, int r, int bblock, char* sendbuf, int* sendcounts, int* sdispls,
                         rbv_datatype sendtype, char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype,
                         rbv_comm_t comm);
int TTPL_BT_alltoallv_s2(int n, int r, int bblock, char* sendbuf, int* sendcounts, int* sdispls,
                         rbv_datatype sendtype, char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype,
                         rbv_comm_t comm);
int MPICH_intra_scattered(int bblock, char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype,
                          char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int ompi_alltoallv_intra_basic_linear(char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype,
                                      char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype,
                                      rbv_comm_t comm);
int ompi_alltoallv_intra_pairwise(char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype, char* recvbuf,
                                  int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int exclisive_or_alltoallv(char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype, char* recvbuf,
                           int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int exclusive_or_alltoallv(char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype, char* recvbuf,
                           int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int twolayer_communicator_linear(int n, char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype,
                                 char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int twolayer_communicator_linear_s2(int n, int bblock1, int bblock2, char* sendbuf, int* sendcounts, int* sdispls,
                                    rbv_datatype sendtype, char* recvbuf, int* recvcounts, int* rdispls,
                                    rbv_datatype recvtype, rbv_comm_t comm);
int twolayer_communicator_linear_s3(int n, int bblock1, int bblock2, char* sendbuf, int* sendcounts, int* sdispls,
                                    rbv_datatype sendtype, char* recvbuf, int* recvcounts, int* rdispls,
                                    rbv_datatype recvtype, rbv_comm_t comm);
int twolayer_communicator_linear_s4(int n, int bblock1, int bblock2, char* sendbuf, int* sendcounts, int* sdispls,
                                    rbv_datatype sendtype, char* recvbuf, int* recvcounts, int* rdispls,
                                    rbv_datatype recvtype, rbv_comm_t comm);
/* Exchange schemes of the reference's benchmark programs (benchmarks/merge_benchmark.cpp,
 * simple_merge_benchmark.cpp, split_benchmark.cpp), with the hand-out to the destinations that the reference's
 * merge leaves commented out. */
int merge_alltoallv(int ncores, char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype, char* recvbuf,
                    int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int simply_merge_alltoallv(int ncores, char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype,
                           char* recvbuf, int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int split_alltoallv(char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype, char* recvbuf,
                    int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
/* Declared but never defined in the reference (src/rbruckv.h:80-81); here: the automatic choice, that is
 * rbv_alltoallv_auto under the reference's name. */
int rbv_alltoallv_auto(char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype, char* recvbuf,
                       int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
int ML_benchmark(char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype, char* recvbuf, int* recvcounts,
                 int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);
void spreadout_alltoallv(char* sendbuf, int* sendcounts, int* sdispls, rbv_datatype sendtype, char* recvbuf,
                         int* recvcounts, int* rdispls, rbv_datatype recvtype, rbv_comm_t comm);

#ifdef __cplusplus
} /* extern "C" */
std::vector<int> convert10tob(int w, int N, int b);
#endif

#endif /* RBV_RBRUCKV_H_ */
