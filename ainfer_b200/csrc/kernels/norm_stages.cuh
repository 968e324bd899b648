// Vector stages of the persistent decode step that run redundantly in every
// block ahead of a weight-streaming stage: (1+w) RMSNorm + activation quantiser,
// per-head gated RMSNorm + quantiser, and router logits from a normalised vector
// held in shared memory. (Fusing them into the stand-alone GEMV kernels as well
// was measured and dropped: with programmatic dependent launches the separate
// one-block norm kernel overlaps the next kernel's weight prefetch, and the fused
// form was no faster.)
#pragma once
#include "block_dot.cuh"
#include "../common/detmath.h"

namespace ainfer {

constexpr int kYsFloats = 4096;  // largest fp32 vector of a norm stage (hidden, value_dim, q_heads*256)

// (1+w) RMSNorm + activation quantiser of one fp32 vector, result staged in
// shared memory for the GEMV rows; ys keeps the normalised fp32 vector (the
// router reads it). Same arithmetic as RmsNormQuant (k_norm.cu). src is either
// a global fp32 vector or a BF16 embedding row.
static __device__ __noinline__ StagedAct4 norm_quant_stage(const float *xg, const uint16_t *emb_row,
                                                      const float *w, int N, float eps,
                                                      unsigned char *stage, float *ys,
                                                      float *x_copy_out) {
  __shared__ double ps[256];
  __shared__ float s_inv;
  const int lid = threadIdx.x;
  constexpr int kPer = kYsFloats / 256;  // elements per lane at the largest N
  // every load of this lane is issued before the first use: one round trip to L2
  float xv[kPer], wv[kPer];
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int j = lid + 256 * i;
    if (j < N) {
      xv[i] = emb_row ? bf16_to_f32(emb_row[j]) : __ldcg(xg + j);
      wv[i] = __ldg(w + j);
    }
  }
  __syncthreads();  // ys / stage may still be in use by the previous stage
  double ss = 0;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int j = lid + 256 * i;
    if (j < N) {
      if (x_copy_out) x_copy_out[j] = xv[i];
      double d = (double)xv[i];
      ss = ss + d * d;
    }
  }
  ps[lid] = ss;
  __syncthreads();
  AINFER_STAMP(1);
  for (int st = 128; st >= 32; st >>= 1) {
    if (lid < st) ps[lid] = ps[lid] + ps[lid + st];
    __syncthreads();
  }
  if (lid < 32) {
    double v = ps[lid];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = v + __shfl_xor_sync(kFull, v, off);
    if (lid == 0) s_inv = 1.0f / sqrtf((float)(v / (double)N) + eps);
  }
  __syncthreads();
  const float inv = s_inv;
  AINFER_STAMP(2);
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int j = lid + 256 * i;
    if (j < N) ys[j] = (xv[i] * inv) * (1.0f + wv[i]);
  }
  __syncthreads();
  AINFER_STAMP(3);
  StagedAct4 r = stage4_from_f32<false>(stage, ys, N, 1, N);
  AINFER_STAMP(4);
  return r;
}

// Per-head gated RMSNorm (RmsInv + NormGated, tools/cmdlist/kernels.cpp:619-644)
// of all heads into ys, then the activation quantiser staged for out_proj.
// Same arithmetic as GatedNormQuant (k_norm.cu).
// One head of the gated norm: 128 values, four per lane.
static __device__ __noinline__ void gated_norm_head(float4 o, float4 z, float4 w, float eps, float *out) {
  const int lane = threadIdx.x & 31;
  float ss = 0.0f;
  ss = fmaf(o.x, o.x, ss);
  ss = fmaf(o.y, o.y, ss);
  ss = fmaf(o.z, o.z, ss);
  ss = fmaf(o.w, o.w, ss);
  ss = warp_tree_sum(ss);
  const float inv = 1.0f / sqrtf(ss / 128.0f + eps);
  out[lane] = ((w.x * o.x) * inv) * (z.x / (1.0f + det_expf(-z.x)));
  out[lane + 32] = ((w.y * o.y) * inv) * (z.y / (1.0f + det_expf(-z.y)));
  out[lane + 64] = ((w.z * o.z) * inv) * (z.z / (1.0f + det_expf(-z.z)));
  out[lane + 96] = ((w.w * o.w) * inv) * (z.w / (1.0f + det_expf(-z.w)));
}

static __device__ __noinline__ StagedAct4 gated_norm_stage(const float *O, const float *Z, const float *W,
                                                      int heads, float eps, unsigned char *stage,
                                                      float *ys) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kHB = 4;  // heads a warp fetches together (one round trip to L2 for all of them)
  // lane l holds elements l, l+32, l+64, l+96 of a head (.x .y .z .w)
  const float4 wl = make_float4(__ldg(W + lane), __ldg(W + lane + 32), __ldg(W + lane + 64), __ldg(W + lane + 96));
  __syncthreads();
#pragma unroll 1
  for (int h0 = warp; h0 < heads; h0 += 8 * kHB) {
    float4 ov[kHB], zv[kHB];
#pragma unroll
    for (int b = 0; b < kHB; ++b) {
      const int h = h0 + 8 * b;
      if (h < heads) {
        const float *o = O + (size_t)h * 128 + lane, *z = Z + (size_t)h * 128 + lane;
        ov[b] = make_float4(__ldcg(o), __ldcg(o + 32), __ldcg(o + 64), __ldcg(o + 96));
        zv[b] = make_float4(__ldcg(z), __ldcg(z + 32), __ldcg(z + 64), __ldcg(z + 96));
      }
    }
#pragma unroll
    for (int b = 0; b < kHB; ++b) {
      const int h = h0 + 8 * b;
      if (h < heads) gated_norm_head(ov[b], zv[b], wl, eps, ys + h * 128);
    }
  }
  __syncthreads();
  AINFER_STAMP(5);
  StagedAct4 r = stage4_from_f32<false>(stage, ys, heads * 128, 1, heads * 128);
  AINFER_STAMP(6);
  return r;
}

// Router logits with the normalised activations held in shared memory.
static __device__ __noinline__ void router_rows_smem(const uint16_t *Wr, const uint16_t *Wsg, const float *hn,
                                                 float *logits, int E, int H, int blk, int nblk) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = E + (Wsg ? 1 : 0);
  for (int e = blk * 8 + warp; e < rows; e += nblk * 8) {
    const uint16_t *w = e < E ? Wr + (size_t)e * H : Wsg;
    float acc = 0.0f;
    for (int i = 0; i < H / 256; ++i) {
      int k0 = (i * 32 + lane) * 8;
      uint4 wv = *reinterpret_cast<const uint4 *>(w + k0);
      float4 x0 = *reinterpret_cast<const float4 *>(hn + k0);
      float4 x1 = *reinterpret_cast<const float4 *>(hn + k0 + 4);
      acc = fmaf(u2f(wv.x << 16), x0.x, acc);
      acc = fmaf(u2f(wv.x & 0xFFFF0000u), x0.y, acc);
      acc = fmaf(u2f(wv.y << 16), x0.z, acc);
      acc = fmaf(u2f(wv.y & 0xFFFF0000u), x0.w, acc);
      acc = fmaf(u2f(wv.z << 16), x1.x, acc);
      acc = fmaf(u2f(wv.z & 0xFFFF0000u), x1.y, acc);
      acc = fmaf(u2f(wv.w << 16), x1.z, acc);
      acc = fmaf(u2f(wv.w & 0xFFFF0000u), x1.w, acc);
    }
    acc = warp_tree_sum(acc);
    if (lane == 0) logits[e] = acc;
  }
}

}  // namespace ainfer
