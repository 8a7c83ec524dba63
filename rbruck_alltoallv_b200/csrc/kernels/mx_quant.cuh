// The MXFP8 scale rule shared by every kernel that quantises (row quantiser, quantising dispatch, quantising GEMM
// epilogue), so that they agree bit for bit: a block of 32 values with largest magnitude amax gets the scale 2^e with
// the smallest e such that amax / 2^e <= 448 (the largest e4m3 value), stored as the UE8M0 byte e + 127.
#pragma once
#include <cuda_runtime.h>

namespace rbv {

// e = ceil(log2(amax / 448)) from the bits of the quotient, clamped to the UE8M0 range; 0 for amax == 0 (or NaN).
__device__ __forceinline__ int mx_exponent(float amax) {
  if (!(amax > 0.0f)) return 0;
  const unsigned b = __float_as_uint(amax * (1.0f / 448.0f));
  const int e = (int)((b >> 23) & 0xffu) - 127 + ((b & 0x7fffffu) ? 1 : 0);
  return max(-127, min(127, e));
}

// 2^-e for e in [-127, 126] (finite inputs never reach 127: the largest float / 448 is below 2^120).
__device__ __forceinline__ float mx_inv_scale(int e) { return __uint_as_float((unsigned)(127 - e) << 23); }

}  // namespace rbv
