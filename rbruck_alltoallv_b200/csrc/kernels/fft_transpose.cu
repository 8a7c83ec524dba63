// Pencil transpose for distributed 3-D FFTs: strided gather -> all-to-all -> transposed scatter in ONE kernel.
// For every destination rank the caller describes a 3-D box of the local array and where (and with which
// strides) it lands in the destination rank's array; the kernel moves 64 x 64 element tiles through shared
// memory so that both the local reads and the peer writes over NVLink are contiguous runs, then signals all
// ranks and waits (bounded) until every rank's boxes have landed here.  The reference only generates the
// count patterns of such an exchange (examples/FFT_distribution.cpp:66-87) and leaves packing to the caller.
#include <cuda_runtime.h>

#include <cstdint>

#include "api/ctx_internal.h"
#include "kernels/primitives.cuh"
#include "rbv/device_types.h"
#include "rbv/fft.h"

namespace rbv {
namespace {

constexpr int TS = 32;          // tile edge (elements)
constexpr int kThreadsT = 256;  // 32 x 8

struct TransposeArgs {
  int nproc, proc;
  unsigned long long ctrl_off, timeout_ns;
  int* error;
  unsigned long long* aux_self;   // arrival counter copies in the NVLS buffer and their multicast address
  unsigned long long* aux_mc;     // (null: the counters of the control blocks are used)
  char* heap[kMaxProcs];
  const char* src;
  unsigned long long dst_off;   // byte offset of the destination array inside every heap
  int elem_size;                // 4, 8 or 16
  rbv_box box[kMaxProcs];
};

// TF x TK tile: TF elements along the destination's contiguous dimension, TK along the source's (dimension 2).
template <typename T, int TF, int TK>
__device__ void move_boxes(const TransposeArgs& a, T* tile_raw) {
  T (*tile)[TK + 1] = reinterpret_cast<T(*)[TK + 1]>(tile_raw);
  // tiles are enumerated over all destinations; a CTA takes tile ids blockIdx.x, blockIdx.x + gridDim.x, ...
  // Destinations are visited starting with this rank and going upwards (the spread-out order): at any moment the
  // ranks of a group write to different peers, so no GPU's NVLink ingress is shared by the whole group.
  long long tile_base = 0;
  for (int dd = 0; dd < a.nproc; dd++) {
    const int d = (a.proc + dd) % a.nproc;
    const rbv_box& b = a.box[d];
    if (b.n0 <= 0 || b.n1 <= 0 || b.n2 <= 0) continue;
    const T* src = reinterpret_cast<const T*>(a.src) + b.src_off;
    T* dst = reinterpret_cast<T*>(a.heap[d] + a.dst_off) + b.dst_off;
    // the source's fastest dimension is 2; the destination's fastest is whichever has stride 1
    const int fast = b.t2 == 1 ? 2 : (b.t1 == 1 ? 1 : 0);
    const int nf = fast == 1 ? b.n1 : b.n0;                  // extent of the destination-fastest dim (if != 2)
    const int no = fast == 1 ? b.n0 : b.n1;                  // the remaining ("outer") dim
    const long long sf = fast == 1 ? b.s1 : b.s0, so = fast == 1 ? b.s0 : b.s1;
    const long long to = fast == 1 ? b.t0 : b.t1;
    const int W2 = fast == 2 ? kThreadsT : TK;               // elements of dim 2 per tile
    const int t2n = (b.n2 + W2 - 1) / W2;
    // Tiles start `lead` elements before the box along the destination-fastest dimension, so that every run a
    // tile writes begins on a 128-byte line of the destination (whole lines over NVLink instead of a ragged head
    // and tail per run).  Possible when all rows of the box share their alignment.
    constexpr int kLine = 128 / (int)sizeof(T);
    int lead = 0;
    if (fast != 2 && to % kLine == 0 && b.t2 % kLine == 0)
      lead = (int)((reinterpret_cast<uintptr_t>(dst) / sizeof(T)) % kLine);
    const int tfn = fast == 2 ? 1 : (nf + lead + TF - 1) / TF;
    const long long ntiles = fast == 2 ? (long long)b.n0 * b.n1 * t2n : (long long)no * tfn * t2n;
    const long long first = ((long long)blockIdx.x - (tile_base % (long long)gridDim.x) + gridDim.x) % gridDim.x;
    for (long long t = first; t < ntiles; t += gridDim.x) {
      if (fast == 2) {
        // no transposition: contiguous rows along dim 2
        const int k = (int)(t % t2n) * kThreadsT + (int)threadIdx.x;
        const long long ij = t / t2n;
        const int j = (int)(ij % b.n1), i = (int)(ij / b.n1);
        if (k < b.n2) dst[i * b.t0 + j * b.t1 + k] = src[i * b.s0 + j * b.s1 + k];
      } else {
        const int k0 = (int)(t % t2n) * TK;
        const long long r1 = t / t2n;
        const int f0 = (int)(r1 % tfn) * TF - lead;
        const int o = (int)(r1 / tfn);
        // read: rows along dim 2 (contiguous in the source); all loads of a thread are issued back to back
        {
          const int tx = threadIdx.x % TK, ty = threadIdx.x / TK;
          constexpr int RS = kThreadsT / TK;
          T v[TF / RS];
          const int k = k0 + tx;
          const T* p = src + o * so + (long long)(f0 + ty) * sf + k;
          const long long step = (long long)RS * sf;
          #pragma unroll
          for (int i = 0; i < TF / RS; i++, p += step) {
            const int f = f0 + i * RS + ty;
            if (f >= 0 && f < nf && k < b.n2) v[i] = *p;
          }
          #pragma unroll
          for (int i = 0; i < TF / RS; i++) tile[i * RS + ty][tx] = v[i];
        }
        __syncthreads();
        // write: rows along the destination-fastest dim (contiguous in the destination)
        {
          const int tx = threadIdx.x % TF, ty = threadIdx.x / TF;
          constexpr int RS = kThreadsT / TF;
          #pragma unroll
          for (int r = 0; r < TK; r += RS) {
            const int k = k0 + r + ty, f = f0 + tx;
            if (f >= 0 && f < nf && k < b.n2) dst[o * to + (long long)k * b.t2 + f] = tile[tx][r + ty];
          }
        }
        __syncthreads();
      }
    }
    tile_base += ntiles;
  }
}

__global__ void __launch_bounds__(kThreadsT) transpose_exchange_kernel(const __grid_constant__ TransposeArgs a) {
  // 64 x 64 tiles (512-byte runs on both sides) for elements up to 8 bytes, 32 x 32 for 16-byte elements
  __shared__ __align__(16) unsigned char tile_raw[64 * 65 * 8];
  static_assert(64 * 65 * 8 >= TS * (TS + 1) * 16, "tile buffer");
  if (a.elem_size == 8) move_boxes<unsigned long long, 64, 64>(a, reinterpret_cast<unsigned long long*>(tile_raw));
  else if (a.elem_size == 4) move_boxes<unsigned, 64, 64>(a, reinterpret_cast<unsigned*>(tile_raw));
  else move_boxes<uint4, TS, TS>(a, reinterpret_cast<uint4*>(tile_raw));
  // completion: last CTA signals every process, then waits for all of them (bounded)
  __syncthreads();
  if (threadIdx.x == 0) {
    CtrlBlock* my = reinterpret_cast<CtrlBlock*>(a.heap[a.proc] + a.ctrl_off);
    dev::fence_acq_rel(a.nproc > 1);
    if (atomicAdd(&my->aux_exit[2], 1u) == gridDim.x - 1) {
      my->aux_exit[2] = 0;
      const unsigned seq = my->aux_seq[2];
      dev::fence_acq_rel(a.nproc > 1);   // one fence publishes every CTA's tiles (each fenced before its exit count)
      if (a.aux_mc) {
        dev::multimem_red_add(a.aux_mc + 2, 1ull);   // NVSwitch bumps the counter on every GPU
      } else {
        for (int q = 0; q < a.nproc; q++)
          dev::red_relaxed_add(&reinterpret_cast<CtrlBlock*>(a.heap[q] + a.ctrl_off)->aux_arrivals[2], 1ull, q != a.proc);
      }
      dev::WaitCfg wc{&my->abort_flag, a.timeout_ns};
      const unsigned long long target = ((unsigned long long)seq + 1ull) * (unsigned long long)a.nproc;
      const unsigned long long* arrivals = a.aux_mc ? a.aux_self + 2 : &my->aux_arrivals[2];
      if (dev::wait_ge(arrivals, target, wc, a.nproc > 1) != dev::WAIT_OK) atomicCAS(a.error, 0, 1);
      my->aux_seq[2] = seq + 1u;
    }
  }
}

}  // namespace
}  // namespace rbv

extern "C" int rbv_transpose_exchange(rbv_ctx_t ctx, const void* src, unsigned long long dst_off, int elem_size,
                                      const rbv_box* boxes, int* error_flag, int max_ctas, void* stream) {
  using namespace rbv;
  const Context& c = *ctx->c;
  if (c.L() != 1 || (elem_size != 4 && elem_size != 8 && elem_size != 16)) return (int)cudaErrorInvalidValue;
  TransposeArgs a;
  a.nproc = c.nproc(); a.proc = c.proc();
  a.ctrl_off = c.layout().ctrl_off; a.timeout_ns = c.timeout_ns();
  a.error = error_flag;
  a.aux_self = c.nvls_aux_self();
  a.aux_mc = c.nvls_aux_mc();
  for (int q = 0; q < kMaxProcs; q++) {
    a.heap[q] = q < c.nproc() ? c.peer_heap(q) : nullptr;
    if (q < c.nproc()) a.box[q] = boxes[q]; else a.box[q] = rbv_box{};
  }
  a.src = static_cast<const char*>(src);
  a.dst_off = dst_off;
  a.elem_size = elem_size;
  int grid = max_ctas > 0 ? max_ctas : c.sm_count() * 6;
  transpose_exchange_kernel<<<grid, kThreadsT, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}
