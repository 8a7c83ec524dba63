/* A small MPI stand-in: ranks are threads of one process, messages are copies through per-rank
 * mailboxes.  It exists so that the reference library (which needs <mpi.h>) can be built and timed,
 * unchanged, on machines that have no MPI installation.  Only the calls the reference uses are
 * provided.  Timings taken with it are a shared-memory CPU baseline.
 */
#ifndef RBV_MPI_SHIM_H_
#define RBV_MPI_SHIM_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
typedef long MPI_Aint;
typedef struct shim_request* MPI_Request;
typedef struct MPI_Status {
  int MPI_SOURCE;
  int MPI_TAG;
  int MPI_ERROR;
  int count_bytes;
} MPI_Status;

#define MPI_COMM_WORLD 0
#define MPI_COMM_NULL (-1)
#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15
#define MPI_UNDEFINED (-32766)
#define MPI_ANY_SOURCE (-1)
#define MPI_ANY_TAG (-1)
#define MPI_REQUEST_NULL ((MPI_Request)0)
#define MPI_STATUS_IGNORE ((MPI_Status*)0)
#define MPI_STATUSES_IGNORE ((MPI_Status*)0)

#define MPI_CHAR 1
#define MPI_BYTE 2
#define MPI_UNSIGNED_CHAR 3
#define MPI_INT 4
#define MPI_FLOAT 5
#define MPI_DOUBLE 6
#define MPI_LONG_LONG 7
#define MPI_UNSIGNED_LONG_LONG 8
#define MPI_LONG 9
#define MPI_DOUBLE_INT 10
#define MPI_UNSIGNED 11

#define MPI_MAX 1
#define MPI_MIN 2
#define MPI_SUM 3
#define MPI_MAXLOC 4

int MPI_Init(int* argc, char*** argv);
int MPI_Finalize(void);
int MPI_Abort(MPI_Comm comm, int code);
double MPI_Wtime(void);
int MPI_Comm_rank(MPI_Comm comm, int* rank);
int MPI_Comm_size(MPI_Comm comm, int* size);
int MPI_Comm_split(MPI_Comm comm, int color, int key, MPI_Comm* newcomm);
int MPI_Comm_free(MPI_Comm* comm);
int MPI_Intercomm_create(MPI_Comm local_comm, int local_leader, MPI_Comm peer_comm, int remote_leader, int tag,
                         MPI_Comm* newintercomm);
int MPI_Type_size(MPI_Datatype t, int* size);
int MPI_Type_extent(MPI_Datatype t, MPI_Aint* extent);
int MPI_Barrier(MPI_Comm comm);
int MPI_Allreduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype t, MPI_Op op, MPI_Comm comm);
int MPI_Alltoall(const void* sendbuf, int sendcount, MPI_Datatype st, void* recvbuf, int recvcount, MPI_Datatype rt,
                 MPI_Comm comm);
int MPI_Alltoallv(const void* sendbuf, const int* sendcounts, const int* sdispls, MPI_Datatype st, void* recvbuf,
                  const int* recvcounts, const int* rdispls, MPI_Datatype rt, MPI_Comm comm);
int MPI_Gather(const void* sendbuf, int sendcount, MPI_Datatype st, void* recvbuf, int recvcount, MPI_Datatype rt,
               int root, MPI_Comm comm);
int MPI_Scatter(const void* sendbuf, int sendcount, MPI_Datatype st, void* recvbuf, int recvcount, MPI_Datatype rt,
                int root, MPI_Comm comm);
int MPI_Isend(const void* buf, int count, MPI_Datatype t, int dest, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Irecv(void* buf, int count, MPI_Datatype t, int source, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Send(const void* buf, int count, MPI_Datatype t, int dest, int tag, MPI_Comm comm);
int MPI_Recv(void* buf, int count, MPI_Datatype t, int source, int tag, MPI_Comm comm, MPI_Status* status);
int MPI_Sendrecv(const void* sendbuf, int sendcount, MPI_Datatype st, int dest, int sendtag, void* recvbuf,
                 int recvcount, MPI_Datatype rt, int source, int recvtag, MPI_Comm comm, MPI_Status* status);
int MPI_Wait(MPI_Request* req, MPI_Status* status);
int MPI_Waitall(int count, MPI_Request* reqs, MPI_Status* statuses);

/* Shim control (not MPI): run `fn(arg)` on `nranks` threads, each being one rank of MPI_COMM_WORLD.
 * Returns 0, or 1 when a rank called MPI_Abort. */
typedef void (*shim_rank_fn)(int rank, int nranks, void* arg);
int shim_run(int nranks, shim_rank_fn fn, void* arg);

#ifdef __cplusplus
}
#endif
#endif
