// Device helpers shared by the decode kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "../common/detmath.h"
#include "registry.h"

// Optional fine-grained stage clock: a translation unit that wants time stamps
// inside the shared stage code defines AINFER_STAMP(id) before including it.
#ifndef AINFER_STAMP
#define AINFER_STAMP(id)
#endif

namespace ainfer {

// Programmatic dependent launch: a kernel first lets its successor start launching,
// and waits for its predecessor (completion and memory flush) before it reads or
// writes anything the predecessor touches. Both are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }


constexpr unsigned kFull = 0xFFFFFFFFu;

// Control block words, tools/decode/decode_l0.cpp:41-43.
enum { CTRL_TOKEN = 0, CTRL_POS = 1, CTRL_LEN = 2, CTRL_SELECTED = 3 };

// Sum over the 32 lanes by the xor butterfly 16,8,4,2,1. Because IEEE addition
// is commutative every lane ends with the value of the stride-halving tree
// p[l] += p[l+st] (st = 16..1) evaluated at lane 0.
__device__ __forceinline__ float warp_tree_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = v + __shfl_xor_sync(kFull, v, off);
  return v;
}
__device__ __forceinline__ double warp_tree_sum(double v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = v + __shfl_xor_sync(kFull, v, off);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, off));
  return v;
}
__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(kFull, v, off);
  return v;
}

// Activation quantiser element rule (tools/cmdlist/kernels.cpp:574-577):
// q = trunc(x/s +- 0.5), clamped to +-127.
__device__ __forceinline__ int quant_round(float x, float s) {
  float v = x / s;
  int qi = (int)(v >= 0 ? v + 0.5f : v - 0.5f);
  return qi < -127 ? -127 : (qi > 127 ? 127 : qi);
}

}  // namespace ainfer
