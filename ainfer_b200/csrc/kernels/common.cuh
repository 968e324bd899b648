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

// Streaming 16-byte load: weights are read once per token, keep them out of L1.
__device__ __forceinline__ uint4 ldg_stream16(const void *p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const void *p) {
  uint2 v;
  asm("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// Activation quantiser element rule (tools/cmdlist/kernels.cpp:574-577):
// q = trunc(x/s +- 0.5), clamped to +-127.
__device__ __forceinline__ int quant_round(float x, float s) {
  float v = x / s;
  int qi = (int)(v >= 0 ? v + 0.5f : v - 0.5f);
  return qi < -127 ? -127 : (qi > 127 ? 127 : qi);
}

// Dot of one 16-byte chunk of packed INT4 (32 weights, low nibble = even k)
// with 32 INT8 activations held de-interleaved: xe[i] = bytes (x0,x2,x4,x6) and
// xo[i] = (x1,x3,x5,x7) of the i-th 8-weight word. Nibbles are biased by xor 8
// to unsigned 0..15; the caller subtracts 8 * sum(x) per group.
__device__ __forceinline__ int dot_chunk_biased(const uint4 w, const uint4 xa, const uint4 xb,
                                                int acc) {
  // xa = {e0, o0, e1, o1}, xb = {e2, o2, e3, o3}
  uint32_t b;
  b = w.x ^ 0x88888888u;
  acc = __dp4a((int)(b & 0x0F0F0F0Fu), (int)xa.x, acc);
  acc = __dp4a((int)((b >> 4) & 0x0F0F0F0Fu), (int)xa.y, acc);
  b = w.y ^ 0x88888888u;
  acc = __dp4a((int)(b & 0x0F0F0F0Fu), (int)xa.z, acc);
  acc = __dp4a((int)((b >> 4) & 0x0F0F0F0Fu), (int)xa.w, acc);
  b = w.z ^ 0x88888888u;
  acc = __dp4a((int)(b & 0x0F0F0F0Fu), (int)xb.x, acc);
  acc = __dp4a((int)((b >> 4) & 0x0F0F0F0Fu), (int)xb.y, acc);
  b = w.w ^ 0x88888888u;
  acc = __dp4a((int)(b & 0x0F0F0F0Fu), (int)xb.z, acc);
  acc = __dp4a((int)((b >> 4) & 0x0F0F0F0Fu), (int)xb.w, acc);
  return acc;
}

// Stages K INT8 activations into shared memory de-interleaved for
// dot_chunk_biased, and the per-group sums of the activations.
// xs_e_o: K bytes, laid out as K/8 pairs {even word, odd word}. gsum: K/128 ints.
__device__ __forceinline__ void stage_activations(const int8_t *__restrict__ xq, int K,
                                                  uint32_t *xs_e_o, int *gsum) {
  const uint2 *src = reinterpret_cast<const uint2 *>(xq);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
    uint2 v = src[i];
    xs_e_o[2 * i] = __byte_perm(v.x, v.y, 0x6420);
    xs_e_o[2 * i + 1] = __byte_perm(v.x, v.y, 0x7531);
  }
  __syncthreads();
  for (int g = threadIdx.x; g < K / 128; g += blockDim.x) {
    int s = 0;
    for (int i = 0; i < 32; ++i) s = __dp4a((int)xs_e_o[g * 32 + i], 0x01010101, s);
    gsum[g] = s;
  }
  __syncthreads();
}

}  // namespace ainfer
