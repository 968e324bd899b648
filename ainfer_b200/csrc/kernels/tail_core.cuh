// Block-level first-max-wins argmax helpers (tools/cmdlist/kernels.cpp:492-509 tie rule).
#pragma once
#include "common.cuh"

namespace ainfer {

__device__ __forceinline__ void argmax_merge(float &bv, int &bi, float ov, int oi) {
  if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}
__device__ __forceinline__ void block_argmax(float &bv, int &bi, float *sv, int *si) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
    argmax_merge(bv, bi, __shfl_xor_sync(kFull, bv, off), __shfl_xor_sync(kFull, bi, off));
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = lane < (int)(blockDim.x >> 5) ? sv[lane] : -INFINITY;
    bi = lane < (int)(blockDim.x >> 5) ? si[lane] : 0x7FFFFFFF;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      argmax_merge(bv, bi, __shfl_xor_sync(kFull, bv, off), __shfl_xor_sync(kFull, bi, off));
  }
}

}  // namespace ainfer
