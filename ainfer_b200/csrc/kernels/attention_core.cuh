// Gated GQA decode attention over an INT8 KV cache, split over the sequence.
//   AttnPrep    = SplitQK + BatchNorm(q,k) + RopeApply + KvAppend of the
//                 reference (tools/cmdlist/kernels.cpp:429-462,656-684; recorded
//                 at tools/decode/decode_l0.cpp:567-597), with the BF16 append
//                 replaced by the per-token-per-head INT8 quantiser.
//   AttnSplit   = the score/softmax/weighted-V body of AttnCore
//                 (kernels.cpp:210-304) for one 64-token chunk of one KV head,
//                 all query heads of the group sharing each K/V row read.
//   AttnCombine = merges the chunk partials in ascending order, applies the
//                 sigmoid output gate (kernels.cpp:291-302) and the activation
//                 quantiser that feeds o_proj.
// The reference runs one work-item per query head and re-reads K/V per head;
// here a K/V row is read once per KV head and the sequence is spread over SMs.
#pragma once
#include "common.cuh"

namespace ainfer {

constexpr int kAttnChunk = 64;  // tokens per split (fixed: part of the arithmetic contract)
constexpr int kHeadDim = 256;

// ------------------------------------------------------------- AttnPrep ---
struct AttnPrepArgs {
  const float *Q16;     // [nQ][2*D]: per head content D | gate D
  const float *K16;     // [nKV][D]
  const float *V16;     // [nKV][D]
  const float *QNW;     // [D] q_norm weight
  const float *KNW;     // [D] k_norm weight
  const float *Cos;     // [max_ctx][rot]
  const float *Sin;
  const int32_t *Ctrl;  // position = Ctrl[1]
  float *Qn;            // out [nQ][D]
  int8_t *Kc;           // [max_ctx][nKV][D]
  int8_t *Vc;
  uint16_t *Ks;         // fp16 scales [max_ctx][nKV]
  uint16_t *Vs;
  int32_t nQ, nKV, rot, max_ctx;
  float eps;
};

// quantise one 256-wide row held as x[i] = row[lane + 32*i]
__device__ __forceinline__ void kv_quant_store(const float (&x)[8], int lane, int8_t *dst,
                                               uint16_t *sdst) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(x[i]));
  m = warp_max(m);
  float s = m / 127.0f;
  if (s == 0.0f) s = 1.0f;
  uint16_t h = f32_to_f16(s);
  float sf = f16_to_f32(h);
  if (sf == 0.0f) { sf = 1.0f; h = 0x3C00u; }
  if (lane == 0) *sdst = h;
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[lane + 32 * i] = (int8_t)quant_round(x[i], sf);
}

__device__ __forceinline__ void attn_prep_body(const AttnPrepArgs &a, int blk, int nblk) {
  constexpr int D = kHeadDim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = a.nQ + 2 * a.nKV;
  int pos = __ldcg(a.Ctrl + CTRL_POS);
  int p = pos < a.max_ctx ? pos : a.max_ctx - 1;  // clamp, kernels.cpp:456
  for (int r = blk * 8 + warp; r < rows; r += nblk * 8) {
    float x[8];
    if (r >= a.nQ + a.nKV) {  // V row: quantise only
      int h = r - a.nQ - a.nKV;
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = __ldcg(a.V16 + (size_t)h * D + lane + 32 * i);
      kv_quant_store(x, lane, a.Vc + ((size_t)p * a.nKV + h) * D, a.Vs + (size_t)p * a.nKV + h);
      continue;
    }
    const bool isq = r < a.nQ;
    const int h = isq ? r : r - a.nQ;
    const float *src = isq ? a.Q16 + (size_t)h * 2 * D : a.K16 + (size_t)h * D;
    const float *w = isq ? a.QNW : a.KNW;
    double ss = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x[i] = __ldcg(src + lane + 32 * i);
      double d = (double)x[i];
      ss = ss + d * d;
    }
    ss = warp_tree_sum(ss);
    float inv = 1.0f / sqrtf((float)(ss / (double)D) + a.eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = (x[i] * inv) * (1.0f + w[lane + 32 * i]);
    // NeoX half rotation on the leading rot dims: pairs (d, d + rot/2). With
    // rot = 64 both members of a pair sit in the same lane (i = 0 and 1).
    const int half = a.rot / 2;
    if (half == 32) {
      float c = a.Cos[(size_t)pos * a.rot + lane], s = a.Sin[(size_t)pos * a.rot + lane];
      float x0 = x[0], x1 = x[1];
      x[0] = x0 * c - x1 * s;
      x[1] = x0 * s + x1 * c;
    }
    if (isq) {
#pragma unroll
      for (int i = 0; i < 8; ++i) a.Qn[(size_t)h * D + lane + 32 * i] = x[i];
    } else {
      kv_quant_store(x, lane, a.Kc + ((size_t)p * a.nKV + h) * D, a.Ks + (size_t)p * a.nKV + h);
    }
  }
}

// ------------------------------------------------------------ AttnSplit ---
struct AttnSplitArgs {
  const float *Qn;      // [nQ][D]
  const int8_t *Kc;     // [max_ctx][nKV][D]
  const int8_t *Vc;
  const uint16_t *Ks;   // [max_ctx][nKV]
  const uint16_t *Vs;
  const int32_t *Ctrl;  // T = Ctrl[2] (active_length)
  float *Pm;            // [nQ][max_chunks]   chunk max
  float *Pse;           // [nQ][max_chunks]   chunk sum of exp
  float *Pacc;          // [nQ][max_chunks][D] chunk weighted V
  int32_t nQ, nKV, max_ctx, max_chunks;
};

// kStage: the chunk's K and V rows and their scales are first copied to shared memory by the
// whole block (every global load of the item in flight at once: one round trip), and the token
// loops run rolled over shared memory. A kernel of this chain runs once per layer with a cold
// instruction cache, so its time follows the amount of distinct code it executes: the rolled
// loops are several times faster here than the same work unrolled over registers.
// kvs: 2*C*D bytes (K rows, then V rows), kss/vss: C scales each; shared memory of the caller.
// The heads' score sums of one token: lane partials -> warp_tree_sum per head -> (sum * k_scale) * scale,
// stored at dst[head]. With 2, 4 or 8 heads the sums of all heads share one butterfly
// (warp_tree_sum_multi: the same additions, a fraction of the shuffles).
template <int GQ>
__device__ __forceinline__ void attn_store_scores(const float (&part)[GQ], int lane, float *dst, float ks, float scale) {
  if constexpr (GQ == 2 || GQ == 4 || GQ == 8) {
    const float r = warp_tree_sum_multi<GQ>(part, lane);
    if ((lane & (32 / GQ - 1)) == 0) dst[warp_tree_owner<GQ>(lane)] = (r * ks) * scale;
  } else {
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      const float r = warp_tree_sum(part[g]);
      if (lane == 0) dst[g] = (r * ks) * scale;
    }
  }
}

template <int GQ, bool kStage>  // query heads per KV head
__device__ __forceinline__ void attn_split_body(const AttnSplitArgs &a, int blk, int nblk, unsigned char *kvs,
                                                uint16_t *kss, uint16_t *vss) {
  constexpr int D = kHeadDim, C = kAttnChunk;
  __shared__ __align__(16) float sc[C][GQ];   // per token the heads' scores, then p = w * v_scale
  __shared__ float hmax[GQ], hse[GQ];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  int T = __ldcg(a.Ctrl + CTRL_LEN);
  if (T > a.max_ctx) T = a.max_ctx;  // clamp, kernels.cpp:227-228
  const int nch = (T + C - 1) / C;
  const float scale = 1.0f / sqrtf((float)D);
  for (int item = blk; item < nch * a.nKV; item += nblk) {
    const int c = item / a.nKV, kv = item % a.nKV;
    const int t0 = c * C, t1 = min(T, t0 + C), nt = t1 - t0;
    // q rows of this group: lane holds dims 8*lane .. 8*lane+7 of each head
    float q[GQ][8];
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      const float4 *qp = reinterpret_cast<const float4 *>(a.Qn + (size_t)(kv * GQ + g) * D + lane * 8);
      float4 v0 = __ldcg(qp), v1 = __ldcg(qp + 1);
      q[g][0] = v0.x; q[g][1] = v0.y; q[g][2] = v0.z; q[g][3] = v0.w;
      q[g][4] = v1.x; q[g][5] = v1.y; q[g][6] = v1.z; q[g][7] = v1.w;
    }
    if (kStage) {
      const uint4 *kg = reinterpret_cast<const uint4 *>(a.Kc + ((size_t)t0 * a.nKV + kv) * D);
      const uint4 *vg = reinterpret_cast<const uint4 *>(a.Vc + ((size_t)t0 * a.nKV + kv) * D);
      const size_t rs = (size_t)a.nKV * (D / 16);  // 16-byte pieces between consecutive tokens' rows
      uint4 kr[C * D / 16 / 256], vr[C * D / 16 / 256];
#pragma unroll
      for (int u = 0; u < C * D / 16 / 256; ++u) {
        const int i = tid + 256 * u, row = i / (D / 16), pc = i % (D / 16);
        kr[u] = make_uint4(0, 0, 0, 0);
        vr[u] = make_uint4(0, 0, 0, 0);
        if (row < nt) {
          kr[u] = __ldcg(kg + row * rs + pc);
          vr[u] = __ldcg(vg + row * rs + pc);
        }
      }
      uint16_t ksc = 0, vsc = 0;
      if (tid < nt) {
        ksc = __ldcg(a.Ks + (size_t)(t0 + tid) * a.nKV + kv);
        vsc = __ldcg(a.Vs + (size_t)(t0 + tid) * a.nKV + kv);
      }
#pragma unroll
      for (int u = 0; u < C * D / 16 / 256; ++u) {
        reinterpret_cast<uint4 *>(kvs)[tid + 256 * u] = kr[u];
        reinterpret_cast<uint4 *>(kvs + C * D)[tid + 256 * u] = vr[u];
      }
      if (tid < C) {
        kss[tid] = ksc;
        vss[tid] = vsc;
      }
      __syncthreads();
      // phase 1: scores. warp w takes tokens t0+w, t0+w+8, ...
#pragma unroll 1
      for (int tt = warp; tt < nt; tt += 8) {
        const uint2 kw = reinterpret_cast<const uint2 *>(kvs)[tt * (D / 8) + lane];
        const float ks = f16_to_f32(kss[tt]);
        float kf[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          kf[j] = (float)(int)(int8_t)((kw.x >> (8 * j)) & 0xFF);
          kf[4 + j] = (float)(int)(int8_t)((kw.y >> (8 * j)) & 0xFF);
        }
        float part[GQ];
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
          float acc = 0.0f;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc = fmaf(q[g][j], kf[j], acc);
          part[g] = acc;
        }
        attn_store_scores<GQ>(part, lane, &sc[tt][0], ks, scale);
      }
    } else {
    // phase 1: scores. warp w takes tokens t0+w, t0+w+8, ...; all its K rows (C/8 of them) are
      // fetched before the first is used, so the warp pays one round trip, not one per token
      constexpr int kTok = C / 8;
      uint2 kwv[kTok];
      uint16_t ksv[kTok];
#pragma unroll
      for (int i = 0; i < kTok; ++i) {
        const int tt = warp + 8 * i;
        kwv[i] = make_uint2(0, 0);
        ksv[i] = 0;
        if (tt < nt) {
          const int t = t0 + tt;
          kwv[i] = __ldcg(reinterpret_cast<const uint2 *>(a.Kc + ((size_t)t * a.nKV + kv) * D + lane * 8));
          ksv[i] = __ldcg(a.Ks + (size_t)t * a.nKV + kv);
        }
      }
#pragma unroll
      for (int i = 0; i < kTok; ++i) {
        const int tt = warp + 8 * i;
        if (tt < nt) {
          const uint2 kw = kwv[i];
          const float ks = f16_to_f32(ksv[i]);
          float kf[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            kf[j] = (float)(int)(int8_t)((kw.x >> (8 * j)) & 0xFF);
            kf[4 + j] = (float)(int)(int8_t)((kw.y >> (8 * j)) & 0xFF);
          }
          float part[GQ];
#pragma unroll
          for (int g = 0; g < GQ; ++g) {
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = fmaf(q[g][j], kf[j], acc);
            part[g] = acc;
          }
          attn_store_scores<GQ>(part, lane, &sc[tt][0], ks, scale);
        }
      }
    }
    __syncthreads();
    AINFER_MARK(1);
    // phase 2: per head max, weights, sum of exp (ascending t)
    if (tid < GQ) {
      float mx = -INFINITY;
      for (int tt = 0; tt < nt; ++tt) mx = fmaxf(mx, sc[tt][tid]);
      hmax[tid] = mx;
    }
    __syncthreads();
    for (int i = tid; i < GQ * nt; i += 256) {
      int tt = i / GQ, g = i % GQ;
      sc[tt][g] = det_expf(sc[tt][g] - hmax[g]);
    }
    __syncthreads();
    if (tid < GQ) {
      float se = 0.0f;
      for (int tt = 0; tt < nt; ++tt) se = se + sc[tt][tid];
      hse[tid] = se;
    }
    __syncthreads();
    for (int i = tid; i < GQ * nt; i += 256) {
      int tt = i / GQ, g = i % GQ;
      sc[tt][g] = sc[tt][g] * f16_to_f32(kStage ? vss[tt] : __ldcg(a.Vs + (size_t)(t0 + tt) * a.nKV + kv));
    }
    __syncthreads();
    AINFER_MARK(2);
    // phase 3: every (head, dim) sum runs over the tokens in ascending order. With the heads in
    // fours (one 16-byte read gives a token's weights for four heads) a thread owns four heads
    // of one or two dims; otherwise thread d owns dim d of every head.
    if constexpr (kStage && GQ % 4 == 0) {
      constexpr int HQ = GQ / 4 > 0 ? GQ / 4 : 1, DPT = D * HQ / 256 > 0 ? D * HQ / 256 : 1;
      const int hq = tid / (256 / HQ), d0 = (tid % (256 / HQ)) * DPT;
      float a4[DPT][4];
#pragma unroll
      for (int j = 0; j < DPT; ++j) a4[j][0] = a4[j][1] = a4[j][2] = a4[j][3] = 0.0f;
      const int8_t *vs = reinterpret_cast<const int8_t *>(kvs + C * D) + d0;
#pragma unroll 2
      for (int tt = 0; tt < nt; ++tt) {
        const float4 pw = *reinterpret_cast<const float4 *>(&sc[tt][(4 * hq) % GQ]);
#pragma unroll
        for (int j = 0; j < DPT; ++j) {
          const float v = (float)(int)vs[tt * D + j];
          a4[j][0] = fmaf(pw.x, v, a4[j][0]);
          a4[j][1] = fmaf(pw.y, v, a4[j][1]);
          a4[j][2] = fmaf(pw.z, v, a4[j][2]);
          a4[j][3] = fmaf(pw.w, v, a4[j][3]);
        }
      }
#pragma unroll
      for (int hh = 0; hh < 4; ++hh) {
        const size_t slot = (size_t)(kv * GQ + 4 * hq + hh) * a.max_chunks + c;
#pragma unroll
        for (int j = 0; j < DPT; ++j) a.Pacc[slot * D + d0 + j] = a4[j][hh];
      }
      if (tid < GQ) {
        const size_t slot = (size_t)(kv * GQ + tid) * a.max_chunks + c;
        a.Pm[slot] = hmax[tid];
        a.Pse[slot] = hse[tid];
      }
    } else {
    float acc[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) acc[g] = 0.0f;
    if (kStage) {
      const int8_t *vs = reinterpret_cast<const int8_t *>(kvs + C * D) + tid;
#pragma unroll 2
      for (int tt = 0; tt < nt; ++tt) {
        const float v = (float)(int)vs[tt * D];
#pragma unroll
        for (int g = 0; g < GQ; ++g) acc[g] = fmaf(sc[tt][g], v, acc[g]);
      }
    } else {
      const int8_t *vp = a.Vc + ((size_t)t0 * a.nKV + kv) * D + tid;
#pragma unroll 16
      for (int tt = 0; tt < nt; ++tt) {
        float v = (float)(int)__ldcg(vp + (size_t)tt * a.nKV * D);
#pragma unroll
        for (int g = 0; g < GQ; ++g) acc[g] = fmaf(sc[tt][g], v, acc[g]);
      }
    }
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      size_t slot = (size_t)(kv * GQ + g) * a.max_chunks + c;
      a.Pacc[slot * D + tid] = acc[g];
      if (tid == 0) {
        a.Pm[slot] = hmax[g];
        a.Pse[slot] = hse[g];
      }
    }
    }
    AINFER_MARK(3);
    __syncthreads();
  }
}

// Eight INT8 values (a row's bytes 8*lane .. 8*lane+7) as floats, exactly: a byte b with its
// sign bit flipped is b + 128 in 0..255; placed in the low mantissa byte of 2^23 it reads as the
// float 8388608 + 128 + b, and subtracting 8388736 leaves b. One byte permute and one addition
// per value on the full-rate pipes, where the integer-to-float conversion has a quarter-rate unit.
__device__ __forceinline__ void s8x8_to_f32(uint2 w, float (&f)[8]) {
  const uint32_t lo = w.x ^ 0x80808080u, hi = w.y ^ 0x80808080u;
  f[0] = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7650)) - 8388736.0f;
  f[1] = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7651)) - 8388736.0f;
  f[2] = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7652)) - 8388736.0f;
  f[3] = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7653)) - 8388736.0f;
  f[4] = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7650)) - 8388736.0f;
  f[5] = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7651)) - 8388736.0f;
  f[6] = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7652)) - 8388736.0f;
  f[7] = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7653)) - 8388736.0f;
}

// One (chunk c, KV head kv) item by one warp. kFull: the chunk holds all 64 tokens (every chunk of
// a sequence but its last), so the token bounds are compile-time constants.
template <int GQ, bool kFull>
__device__ __forceinline__ void attn_warp_item(const AttnSplitArgs &a, int c, int kv, int nt_rt, float (*sc)[GQ], float *vsf,
                                               float *ksf, float scale, size_t rs, int lane) {
  constexpr int D = kHeadDim, C = kAttnChunk, PF = 8;
  const int t0 = c * C, nt = kFull ? C : nt_rt;
  float *scf = &sc[0][0];
  const int8_t *kb = a.Kc + ((size_t)t0 * a.nKV + kv) * D + lane * 8;
  const int8_t *vb = a.Vc + ((size_t)t0 * a.nKV + kv) * D + lane * 8;
  uint2 ring[PF];
#pragma unroll
  for (int i = 0; i < PF; ++i) {
    ring[i] = __ldcg(reinterpret_cast<const uint2 *>(kb + (size_t)min(i, nt - 1) * rs));
  }
  {  // scales: lane l fetches those of tokens l and l + 32
    uint16_t ks0 = 0, ks1 = 0, vs0 = 0, vs1 = 0;
    if (lane < nt) {
      ks0 = __ldcg(a.Ks + (size_t)(t0 + lane) * a.nKV + kv);
      vs0 = __ldcg(a.Vs + (size_t)(t0 + lane) * a.nKV + kv);
    }
    if (lane + 32 < nt) {
      ks1 = __ldcg(a.Ks + (size_t)(t0 + lane + 32) * a.nKV + kv);
      vs1 = __ldcg(a.Vs + (size_t)(t0 + lane + 32) * a.nKV + kv);
    }
    ksf[lane] = f16_to_f32(ks0);
    ksf[lane + 32] = f16_to_f32(ks1);
    vsf[lane] = f16_to_f32(vs0);
    vsf[lane + 32] = f16_to_f32(vs1);
  }
  {
    // ---- phase 1: scores; lane holds dims 8*lane .. 8*lane+7 of each query head of the group
    // slot g of this lane holds head g ^ own, where `own` is the head whose score sum the lane ends
    // up with: the shared butterfly then needs no selection by lane (warp_tree_sum_multi_permuted)
    const int own = warp_tree_owner<GQ>(lane);
    float q[GQ][8];
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
      const float4 *qp = reinterpret_cast<const float4 *>(a.Qn + (size_t)(kv * GQ + (g ^ own)) * D + lane * 8);
      const float4 v0 = __ldcg(qp), v1 = __ldcg(qp + 1);
      q[g][0] = v0.x; q[g][1] = v0.y; q[g][2] = v0.z; q[g][3] = v0.w;
      q[g][4] = v1.x; q[g][5] = v1.y; q[g][6] = v1.z; q[g][7] = v1.w;
    }
    const bool writer = (lane & (32 / GQ - 1)) == 0;
    __syncwarp();
#pragma unroll 1
    for (int b0 = 0; b0 < nt; b0 += PF) {
#pragma unroll
      for (int i = 0; i < PF; ++i) {
        const int tt = b0 + i;
        const uint2 cur = ring[i];
        ring[i] = __ldcg(reinterpret_cast<const uint2 *>(kb + (size_t)min(tt + PF, nt - 1) * rs));
        if (tt < nt) {
          float kf[8];
          s8x8_to_f32(cur, kf);
          const float ks = ksf[tt];
          float part[GQ];
#pragma unroll
          for (int g = 0; g < GQ; ++g) {
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = fmaf(q[g][j], kf[j], acc);
            part[g] = acc;
          }
          const float r = warp_tree_sum_multi_permuted<GQ>(part, lane);
          if (writer) sc[tt][own] = (r * ks) * scale;
        }
      }
    }
  }
  // the first V rows travel during the softmax
#pragma unroll
  for (int i = 0; i < PF; ++i) {
    ring[i] = __ldcg(reinterpret_cast<const uint2 *>(vb + (size_t)min(i, nt - 1) * rs));
  }
  __syncwarp();
  // ---- phase 2: per head max, weights, sum of exp (ascending t), p = w * v_scale.
  // Element i = lane + 32 k of the [token][head] array belongs to head lane % GQ for every k.
  float mx = -INFINITY;
  for (int i = lane; i < GQ * nt; i += 32) mx = fmaxf(mx, scf[i]);
#pragma unroll
  for (int off = GQ; off < 32; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(kFull, mx, off));
  for (int i = lane; i < GQ * nt; i += 32) scf[i] = det_expf(scf[i] - mx);
  __syncwarp();
  float se = 0.0f;
  if (lane < GQ)
    for (int tt = 0; tt < nt; ++tt) se = se + sc[tt][lane];
  __syncwarp();
  for (int i = lane; i < GQ * nt; i += 32) scf[i] = scf[i] * vsf[i / GQ];
  __syncwarp();
  // ---- phase 3: every (head, dim) sum runs over the tokens in ascending order
  float acc[GQ][8];
#pragma unroll
  for (int g = 0; g < GQ; ++g)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[g][j] = 0.0f;
#pragma unroll 1
  for (int b0 = 0; b0 < nt; b0 += PF) {
#pragma unroll
    for (int i = 0; i < PF; ++i) {
      const int tt = b0 + i;
      const uint2 cur = ring[i];
      ring[i] = __ldcg(reinterpret_cast<const uint2 *>(vb + (size_t)min(tt + PF, nt - 1) * rs));
      if (tt < nt) {
        float vf[8];
        s8x8_to_f32(cur, vf);
#pragma unroll
        for (int g4 = 0; g4 < GQ / 4; ++g4) {
          const float4 pw = *reinterpret_cast<const float4 *>(&sc[tt][4 * g4]);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc[4 * g4 + 0][j] = fmaf(pw.x, vf[j], acc[4 * g4 + 0][j]);
            acc[4 * g4 + 1][j] = fmaf(pw.y, vf[j], acc[4 * g4 + 1][j]);
            acc[4 * g4 + 2][j] = fmaf(pw.z, vf[j], acc[4 * g4 + 2][j]);
            acc[4 * g4 + 3][j] = fmaf(pw.w, vf[j], acc[4 * g4 + 3][j]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    const size_t slot = (size_t)(kv * GQ + g) * a.max_chunks + c;
    float4 *dst = reinterpret_cast<float4 *>(a.Pacc + slot * D + lane * 8);
    dst[0] = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    dst[1] = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
  }
  if (lane < GQ) {
    const size_t slot = (size_t)(kv * GQ + lane) * a.max_chunks + c;
    a.Pm[slot] = mx;
    a.Pse[slot] = se;
  }
}

// The same chunk arithmetic as attn_split_body with ONE WARP per (chunk, KV head) item, for
// launches with thousands of items (batched decode at long contexts, prefill passes). A chunk's
// result depends on nothing outside the chunk, so who computes it is free; a warp on its own
// needs no block barrier between the phases, never idles while eight threads run the softmax
// sums, and reads every K and V row straight into registers (lane l: bytes 8l..8l+7 of a row,
// eight rows in flight) without a pass through shared memory. The row loads are unconditional
// (past the chunk's end the last row is fetched again): a load under a condition into a register
// that lives across iterations was measured to be waited for at once. In the value pass a lane owns its
// eight dims of every head: 64 sums fed by one 8-byte row piece and the token's weights.
template <int GQ>
__device__ __forceinline__ void attn_split_warp_body(const AttnSplitArgs &a, int blk, int nblk, unsigned char *scratch) {
  constexpr int D = kHeadDim, C = kAttnChunk, W = 8;
  static_assert(GQ % 4 == 0 && 32 % GQ == 0 && C == 64, "lane partition of the warp form");
  static_assert(W * C * (GQ + 2) * 4 <= 2 * C * D, "fits the block form's K/V staging area");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // per warp: [C][GQ] scores (then p = w * v_scale) and the C key and C value scales as floats
  float(*sc)[GQ] = reinterpret_cast<float(*)[GQ]>(scratch) + (size_t)warp * C;
  float *vsf = reinterpret_cast<float *>(scratch) + W * C * GQ + warp * 2 * C, *ksf = vsf + C;
  int T = __ldcg(a.Ctrl + CTRL_LEN);
  if (T > a.max_ctx) T = a.max_ctx;  // clamp, kernels.cpp:227-228
  const int nch = (T + C - 1) / C;
  const float scale = 1.0f / sqrtf((float)D);
  const size_t rs = (size_t)a.nKV * D;   // bytes between consecutive tokens' rows
#pragma unroll 1
  for (int item = blk * W + warp; item < nch * a.nKV; item += nblk * W) {
    const int c = item / a.nKV, kv = item % a.nKV;
    const int t0 = c * C, nt = min(T, t0 + C) - t0;
    if (nt == C) attn_warp_item<GQ, true>(a, c, kv, nt, sc, vsf, ksf, scale, rs, lane);
    else attn_warp_item<GQ, false>(a, c, kv, nt, sc, vsf, ksf, scale, rs, lane);
    __syncwarp();   // the next item overwrites sc and vsf
  }
}

// warp_form_items > 0: launches of the batched kernels, whose rows take the one-warp-per-item
// form when the launch holds at least that many (chunk, KV head) items (rows x chunks x KV heads;
// the same bits either way, so rows of one launch may differ in the form they take).
template <bool kStage>
__device__ __forceinline__ void attn_split_dispatch(const AttnSplitArgs &a, int blk, int nblk, long rows = 0,
                                                    long warp_form_items = 0) {
  __shared__ __align__(16) unsigned char kvs[kStage ? 2 * kAttnChunk * kHeadDim : 16];
  __shared__ uint16_t kss[kStage ? kAttnChunk : 1], vss[kStage ? kAttnChunk : 1];
  if constexpr (kStage) {
    const int gq = a.nQ / a.nKV;
    if (warp_form_items > 0 && (gq == 8 || gq == 4)) {
      int T = __ldcg(a.Ctrl + CTRL_LEN);
      if (T > a.max_ctx) T = a.max_ctx;
      if (rows * ((T + kAttnChunk - 1) / kAttnChunk) * a.nKV >= warp_form_items) {
        if (gq == 8) attn_split_warp_body<8>(a, blk, nblk, kvs);
        else attn_split_warp_body<4>(a, blk, nblk, kvs);
        return;
      }
    }
  }
  switch (a.nQ / a.nKV) {
    case 1: attn_split_body<1, kStage>(a, blk, nblk, kvs, kss, vss); break;
    case 2: attn_split_body<2, kStage>(a, blk, nblk, kvs, kss, vss); break;
    case 4: attn_split_body<4, kStage>(a, blk, nblk, kvs, kss, vss); break;
    case 6: attn_split_body<6, kStage>(a, blk, nblk, kvs, kss, vss); break;
    case 8: attn_split_body<8, kStage>(a, blk, nblk, kvs, kss, vss); break;
    default: break;  // rejected on the host
  }
}

// ---------------------------------------------------------- AttnCombine ---
struct AttnCombineArgs {
  const float *Pm, *Pse, *Pacc;
  const float *Q16;     // gate = Q16[h][D + d]
  const int32_t *Ctrl;
  int8_t *Q8;           // [nQ*D] quantised gated output
  float *SQ;            // [nQ*D/128]
  float *Att;           // optional fp32 copy
  int32_t nQ, max_ctx, max_chunks;
};
__device__ __forceinline__ void attn_combine_body(const AttnCombineArgs &a, int blk, int nblk) {
  constexpr int D = kHeadDim, C = kAttnChunk;
  constexpr int kCombineChunks = 1024;  // contexts up to 65536 tokens take the shared-memory path
  __shared__ float wmax[8];
  __shared__ float s_pm[kCombineChunks], s_pf[kCombineChunks];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int T = __ldcg(a.Ctrl + CTRL_LEN);
  if (T > a.max_ctx) T = a.max_ctx;
  const int nch = (T + C - 1) / C;
  for (int h = blk; h < a.nQ; h += nblk) {
    const float *pm = a.Pm + (size_t)h * a.max_chunks;
    const float *pse = a.Pse + (size_t)h * a.max_chunks;
    const float *pacc = a.Pacc + (size_t)h * a.max_chunks * D;
    const float gate = __ldcg(a.Q16 + (size_t)h * 2 * D + D + tid);  // in flight during the sums below
    float M = -INFINITY, se = 0.0f, acc = 0.0f;
    if (nch <= kCombineChunks) {
      // The chunk maxima and sums are fetched once by the block (thread c takes chunk c) and the
      // rescale factors exp(m_c - M) are computed once; every thread then runs the same sums in
      // ascending chunk order from shared memory, with its partial-output loads 16 in flight.
      __syncthreads();  // s_pm/s_pf of the previous head are no longer read
      for (int c = tid; c < nch; c += 256) {
        s_pm[c] = __ldcg(pm + c);
        s_pf[c] = __ldcg(pse + c);
      }
      __syncthreads();
      for (int c = 0; c < nch; ++c) M = fmaxf(M, s_pm[c]);
      __syncthreads();  // every thread has M: s_pm may be overwritten with the factors
      for (int c = tid; c < nch; c += 256) s_pm[c] = det_expf(s_pm[c] - M);
      __syncthreads();
      for (int c = 0; c < nch; ++c) se = fmaf(s_pf[c], s_pm[c], se);
#pragma unroll 32
      for (int c = 0; c < nch; ++c) acc = fmaf(__ldcg(pacc + (size_t)c * D + tid), s_pm[c], acc);
    } else {
#pragma unroll 8
      for (int c = 0; c < nch; ++c) M = fmaxf(M, __ldcg(pm + c));
#pragma unroll 8
      for (int c = 0; c < nch; ++c) {
        float f = det_expf(__ldcg(pm + c) - M);
        se = fmaf(__ldcg(pse + c), f, se);
        acc = fmaf(__ldcg(pacc + (size_t)c * D + tid), f, acc);
      }
    }
    float o = acc / se;
    float y = o / (1.0f + det_expf(-gate));
    if (a.Att) a.Att[(size_t)h * D + tid] = y;
    // activation quantiser: groups of 128 = 4 warps
    float m = warp_max(fabsf(y));
    if (lane == 0) wmax[warp] = m;
    __syncthreads();
    int g0 = (warp >> 2) * 4;
    m = fmaxf(fmaxf(wmax[g0], wmax[g0 + 1]), fmaxf(wmax[g0 + 2], wmax[g0 + 3]));
    float s = m / 127.0f;
    if (s == 0.0f) s = 1.0f;
    if ((tid & 127) == 0) a.SQ[(size_t)h * 2 + (tid >> 7)] = s;
    a.Q8[(size_t)h * D + tid] = (int8_t)quant_round(y, s);
    __syncthreads();
  }
}

}  // namespace ainfer
