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
#ifndef AINFER_TIMELINE
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#define AINFER_MARK(id)
#define AINFER_MARK_ANY(id)
#else
#define AINFER_MARK_ANY(id) ::ainfer::timeline_mark(id, true)
#define AINFER_MARK(id) ::ainfer::timeline_mark(id)
// Timeline build (-DAINFER_TIMELINE): block 0 of every kernel records the global
// timer when it reaches its dependency wait and when the wait returns (its
// predecessor has completed), in launch order, into one device buffer:
// word 0 = events so far, word 1 = capacity, then (enter, go) pairs. The time
// between the `go` of consecutive kernels is what each costs on the chain.
static __device__ unsigned long long *g_timeline;
static int set_timeline_buffer(unsigned long long *device_ptr) {
  return cudaMemcpyToSymbol(g_timeline, &device_ptr, sizeof device_ptr) == cudaSuccess ? 0 : 1;
}
static TimelineRegistrar g_timeline_registrar(set_timeline_buffer);
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void pdl_wait() {
  const bool rec = blockIdx.x == 0 && threadIdx.x == 0 && g_timeline != nullptr;
  unsigned long long t0 = 0;
  if (rec) t0 = global_timer_ns();
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (rec) {
    const unsigned long long t1 = global_timer_ns();
    const unsigned long long slot = atomicAdd(g_timeline, 1ull);
    if (slot < g_timeline[1]) {
      g_timeline[2 + 2 * slot] = t0;
      g_timeline[3 + 2 * slot] = t1;
    }
  }
}
// A point inside a kernel (block 0, thread 0): stored in the same buffer as (id | 1 << 63, time).
// any_block: for code that only one block of the grid runs (a last-block section).
__device__ __forceinline__ void timeline_mark(int id, bool any_block = false) {
  if ((blockIdx.x == 0 || any_block) && threadIdx.x == 0 && g_timeline != nullptr) {
    const unsigned long long t = global_timer_ns();
    const unsigned long long slot = atomicAdd(g_timeline, 1ull);
    if (slot < g_timeline[1]) {
      g_timeline[2 + 2 * slot] = (1ull << 63) | (unsigned long long)id;
      g_timeline[3 + 2 * slot] = t;
    }
  }
}
#endif


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
// warp_tree_sum of N values at once (N = 2, 4 or 8; other N: one by one). The butterfly's first
// log2(N) levels exchange HALF of the values a lane still holds instead of all of them: at the
// level with offset `off` a lane keeps the values whose index bit matches its own lane bit and
// adds its partner's copy of them (the same two operands the plain butterfly adds at that level,
// and a + b == b + a), so after those levels it holds ONE value, summed over the same lanes in the
// same association as the plain butterfly; the remaining levels are plain. Shuffles: N - 1 +
// (5 - log2 N) instead of 5 N. On return the sum of value g is in `out` on every lane whose bits
// (16, 8, 4 for N = 8) spell g; warp_tree_owner<N>(lane) is that g.
template <int N>
__device__ __forceinline__ int warp_tree_owner(int lane) {
  return N == 8 ? ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1)
       : N == 4 ? ((lane >> 4) & 1) * 2 + ((lane >> 3) & 1)
       : N == 2 ? ((lane >> 4) & 1) : 0;
}
template <int N>
__device__ __forceinline__ float warp_tree_sum_multi(const float (&v)[N], int lane) {
  static_assert(N == 2 || N == 4 || N == 8, "2, 4 or 8 values");
  float a[N];
#pragma unroll
  for (int i = 0; i < N; ++i) a[i] = v[i];
  int n = N, off = 16;
#pragma unroll
  for (int lvl = 0; lvl < (N == 8 ? 3 : N == 4 ? 2 : 1); ++lvl) {
    const bool hi = (lane & off) != 0;
    const int half = n >> 1;
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
      if (i < half) {
        const float send = hi ? a[i] : a[i + half], keep = hi ? a[i + half] : a[i];
        a[i] = keep + __shfl_xor_sync(kFull, send, off);
      }
    }
    n = half;
    off >>= 1;
  }
  float r = a[0];
#pragma unroll
  for (int o = (N == 8 ? 2 : N == 4 ? 4 : 8); o > 0; o >>= 1) r = r + __shfl_xor_sync(kFull, r, o);
  return r;
}
// warp_tree_sum_multi for a caller that can choose which value sits in which slot: lane l passes
// value (i ^ warp_tree_owner<N>(l)) in slot i. The values a lane keeps at each level are then
// always the lower half of its slots and the ones it sends the upper half, so no selection by
// lane bit is needed; the additions are the same pairs as in warp_tree_sum_multi. Returns the
// sum of value warp_tree_owner<N>(lane).
template <int N>
__device__ __forceinline__ float warp_tree_sum_multi_permuted(const float (&v)[N], int lane) {
  static_assert(N == 2 || N == 4 || N == 8, "2, 4 or 8 values");
  float a[N];
#pragma unroll
  for (int i = 0; i < N; ++i) a[i] = v[i];
  int off = 16;
#pragma unroll
  for (int half = N / 2; half > 0; half >>= 1) {
#pragma unroll
    for (int i = 0; i < N / 2; ++i)
      if (i < half) a[i] = a[i] + __shfl_xor_sync(kFull, a[i + half], off);
    off >>= 1;
  }
  float r = a[0];
#pragma unroll
  for (int o = (N == 8 ? 2 : N == 4 ? 4 : 8); o > 0; o >>= 1) r = r + __shfl_xor_sync(kFull, r, o);
  return r;
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

// The same element rule with the group's reciprocal r = 1/s computed once: x * r is within
// 2.3e-5 of the correctly rounded quotient (|x/s| <= 127), so away from a rounding boundary
// (the fractional part of |x*r| + 0.5 neither below 1e-3 nor above 0.999) both give the same
// integer; at a boundary, and for a scale too small for a finite reciprocal, the exact division
// decides. Bit-identical to quant_round at a quarter of its instructions.
__device__ __forceinline__ float quant_recip(float s) { return s < 1e-30f ? 0.0f : 1.0f / s; }
__device__ __forceinline__ int quant_round_r(float x, float s, float r) {
  const float vp = x * r;
  const float t = fabsf(vp) + 0.5f;
  const float f = t - truncf(t);
  if (r == 0.0f || !(f >= 1e-3f && f <= 0.999f)) return quant_round(x, s);
  int qi = (int)t;
  qi = qi > 127 ? 127 : qi;
  return vp < 0.0f ? -qi : qi;
}

}  // namespace ainfer
