/* An alltoallv entry point for callers that must not allocate device memory.
 *
 * This has no counterpart in the reference library.  It exists for hosts that embed the library where
 * cudaMalloc / cudaFree are off limits at call time: inside a region that is being captured or replayed as
 * a CUDA graph, inside a memory-pool owner that forbids foreign allocations, or in a process whose device
 * memory is fully budgeted by another framework.  The regular entry points create a context that owns a
 * heap obtained from cudaMalloc; this one keeps all of its scratch (flags, metadata tables, staging cells,
 * the schedule) in one array that is part of the library image.
 *
 * What it does: the radix-2, low-digit-first two-phase Bruck alltoallv (the schedule of
 * twophase_rbruck_alltoallv_om with r = 2) among `nranks` logical ranks that all live on the current device;
 * the same kernel as the regular path runs it.  The caller passes every rank's buffers and counts.
 *
 * Limits (fixed by the size of the built-in scratch array, RBV_NOALLOC_SCRATCH_BYTES, which every GPU that
 * loads the library holds until the process exits):
 *   1 <= nranks <= RBV_NOALLOC_MAX_RANKS, every block (count * type_size) <= RBV_NOALLOC_MAX_BLOCK_BYTES.
 * Larger requests are refused with RBV_NOALLOC_ERR_TOO_LARGE before anything is launched.
 *
 * The first call on a device looks up the device address of the scratch array and uploads the schedules of all
 * rank counts from 1 to RBV_NOALLOC_MAX_RANKS (synchronous copies of about 20 KB in total).  Make that first call
 * outside any stream capture.  Later calls on that device, with any rank count, only enqueue a memset and a
 * kernel.  The first-call set-up is guarded by a mutex, so host threads may race to make it.
 *
 * All calls on a device share the one scratch array.  Each call clears the control words it needs at zero
 * (stream-ordered) and otherwise overwrites what the previous call left.  Two calls that overlap on the GPU
 * (different streams without ordering between them) race on it: serialise them.
 *
 * The call is asynchronous on `cuda_stream`.  Arguments: sendbufs / recvbufs [nranks] device pointers;
 * sendcounts[s * nranks + d], sdispls[s * nranks + d] describe rank s's send side, recvcounts[d * nranks + s],
 * rdispls[d * nranks + s] rank d's receive side, all host arrays in elements of type_size bytes.
 */
#ifndef RBV_NOALLOC_H_
#define RBV_NOALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define RBV_NOALLOC_MAX_RANKS 8
#define RBV_NOALLOC_MAX_BLOCK_BYTES (64 * 1024)
#define RBV_NOALLOC_SCRATCH_BYTES (6 * 1024 * 1024)

#define RBV_NOALLOC_OK 0
#define RBV_NOALLOC_ERR_BAD_ARG (-1)
#define RBV_NOALLOC_ERR_TOO_LARGE (-2)
#define RBV_NOALLOC_ERR_CUDA (-3)

int rbv_alltoallv_noalloc(int nranks, int type_size, const void* const* sendbufs, void* const* recvbufs,
                          const int* sendcounts, const long long* sdispls, const int* recvcounts,
                          const long long* rdispls, void* cuda_stream);

/* Waits for `cuda_stream`, then returns 0 if the last call on the current device completed, or the code of the
 * first failure its kernel recorded: 1 a bounded wait ran out, 3 the blocks do not fit the built-in staging cells,
 * 4 a block was larger than the receiver's recvcount, 5 stopped because of an error elsewhere; -1 if the query
 * itself failed.  Allocates nothing. */
int rbv_noalloc_status(void* cuda_stream);

/* Text of the last error returned to this thread by rbv_alltoallv_noalloc. */
const char* rbv_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
