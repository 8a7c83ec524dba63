/* Fused pencil transpose (strided gather -> all-to-all -> transposed scatter) for distributed 3-D FFTs.
 * The reference ships only the count patterns of this exchange (examples/FFT_distribution.cpp). */
#ifndef RBV_FFT_H_
#define RBV_FFT_H_

#include "rbv/rbruckv.h"

#ifdef __cplusplus
extern "C" {
#endif

/* What this rank sends to one destination rank: a box of n0 x n1 x n2 elements of the local array (dimension 2
 * is contiguous in the source: element (i, j, k) sits at src_off + i*s0 + j*s1 + k) that lands in the
 * destination rank's array at dst_off + i*t0 + j*t1 + k*t2.  Exactly one of t0, t1, t2 is 1 (the destination's
 * contiguous dimension).  All offsets and strides are in elements. */
typedef struct rbv_box_s {
  int n0, n1, n2;
  long long src_off, s0, s1;
  long long dst_off, t0, t1, t2;
} rbv_box;

/* boxes: host array with one entry per rank (n0 = 0 for "nothing").  `dst_off_bytes` is the byte offset of the
 * destination array inside every process's symmetric heap.  Returns when all ranks' boxes have landed here.
 * One logical rank per process; elem_size 4, 8 or 16. */
int rbv_transpose_exchange(rbv_ctx_t ctx, const void* src, unsigned long long dst_off_bytes, int elem_size,
                           const rbv_box* boxes, int* error_flag, int max_ctas, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif
