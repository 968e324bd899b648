// DeltaNetStep (device body): one decode step of the gated delta rule, state streamed once.
// Replaces SplitRepeat + L2NormQK + SsmRecur of the reference
// (tools/cmdlist/kernels.cpp:340-410,581-604; recorded at
// tools/decode/decode_l0.cpp:622-649). The reference walks the 128x128 state
// of a head four times from one work-item; here a head is split into column
// slices (columns of S are independent), every slice is one thread block that
// holds its part of S in registers, reads it once and writes it once.
//
// Arithmetic per column v (bit-identical to the CPU oracle):
//   S' = S * exp(g)
//   kv = tree8 over 8 row segments of fma chains  sum_k S'[k][v] * key[k]
//   d  = (val[v] - kv) * beta
//   S''[k][v] = fma(key[k], d, S'[k][v])
//   o[v] = tree8 of fma chains sum_k S''[k][v] * q[k]
// with q, key l2-normalised per head (eps inside the root; q also scaled by
// head_dim^-1/2), sums of squares over 32 strided lanes + tree.
#pragma once
#include "common.cuh"

namespace ainfer {

struct DeltaNetStepArgs {
  float *Out;        // [nV][128] head outputs
  const float *Mx;   // conv output [q: nK*128 | k: nK*128 | v: nV*128]
  float *S;          // [nV][128][128] state, row-major [k][v]
  const float *Bt;   // [nV] beta
  const float *Gt;   // [nV] log decay g
  int32_t nK;
  int32_t nV;
};

constexpr int kDnSlices = 4;  // column slices per head (32 columns each)

constexpr int kDnSeg = 16;  // state rows per warp
// This thread's state values of item `item` (rows warp*16 .. +15, its column). The state is written
// only by this kernel, so a caller may fetch the first item's values before it waits for its
// predecessor.
__device__ __forceinline__ void deltanet_load_state(const DeltaNetStepArgs &a, int item, float (&s)[kDnSeg]) {
  const int h = item / kDnSlices, slice = item % kDnSlices;
  const int warp = threadIdx.x >> 5, col = slice * 32 + (threadIdx.x & 31);
  const float *Sh = a.S + (size_t)h * 128 * 128;
#pragma unroll
  for (int r = 0; r < kDnSeg; ++r) s[r] = __ldcg(Sh + (size_t)(warp * kDnSeg + r) * 128 + col);
}

// Body for a 256-thread block; blk/nblk give the block its share of the (head, slice) items.
// first: state values of item `blk` already loaded (or null).
__device__ __forceinline__ void deltanet_step_body(const DeltaNetStepArgs &a, int blk, int nblk,
                                                   const float (*first)[kDnSeg] = nullptr) {
  constexpr int D = 128, SEG = kDnSeg;
  __shared__ float qs[D], ks[D];
  __shared__ float part[8][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int item = blk; item < a.nV * kDnSlices; item += nblk) {
    const int h = item / kDnSlices, slice = item % kDnSlices;
    const int kh = h / (a.nV / a.nK);
    const int col = slice * 32 + lane;
    // issue the state loads first: 16 rows per warp, one column per lane
    float *Sh = a.S + (size_t)h * D * D;
    float s[SEG];
    if (first && item == blk) {
#pragma unroll
      for (int r = 0; r < SEG; ++r) s[r] = (*first)[r];
    } else {
      deltanet_load_state(a, item, s);
    }
    // l2norm of q (warp 0) and k (warp 1)
    if (warp < 2) {
      const float *src = a.Mx + (warp == 0 ? (size_t)kh * D : (size_t)a.nK * D + (size_t)kh * D);
      float x[4];
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[i] = __ldcg(src + lane + 32 * i);
        ss = fmaf(x[i], x[i], ss);
      }
      ss = warp_tree_sum(ss);
      float inv = 1.0f / sqrtf(ss + 1e-6f);
      float f = inv * (warp == 0 ? 0.0883883476483184405f : 1.0f);  // 128^-1/2 for q
      float *dst = warp == 0 ? qs : ks;
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = x[i] * f;
    }
    const float val = __ldcg(a.Mx + (size_t)2 * a.nK * D + (size_t)h * D + col);
    const float beta = __ldcg(a.Bt + h);
    const float gt = det_expf(__ldcg(a.Gt + h));
    __syncthreads();
    float acc = 0.0f;
#pragma unroll
    for (int r = 0; r < SEG; ++r) {
      s[r] = s[r] * gt;
      acc = fmaf(s[r], ks[warp * SEG + r], acc);
    }
    part[warp][lane] = acc;
    __syncthreads();
    float kv = ((part[0][lane] + part[1][lane]) + (part[2][lane] + part[3][lane])) +
               ((part[4][lane] + part[5][lane]) + (part[6][lane] + part[7][lane]));
    float dl = (val - kv) * beta;
    __syncthreads();  // part is reused below
    acc = 0.0f;
#pragma unroll
    for (int r = 0; r < SEG; ++r) {
      s[r] = fmaf(ks[warp * SEG + r], dl, s[r]);
      acc = fmaf(s[r], qs[warp * SEG + r], acc);
      Sh[(size_t)(warp * SEG + r) * D + col] = s[r];
    }
    part[warp][lane] = acc;
    __syncthreads();
    if (warp == 0) {
      float o = ((part[0][lane] + part[1][lane]) + (part[2][lane] + part[3][lane])) +
                ((part[4][lane] + part[5][lane]) + (part[6][lane] + part[7][lane]));
      a.Out[(size_t)h * D + col] = o;
    }
    __syncthreads();  // qs/ks/part are rewritten by the next item
  }
}
}  // namespace ainfer
