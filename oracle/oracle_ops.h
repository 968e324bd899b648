// TEST INFRASTRUCTURE ONLY (see oracle_math.h). Operator restatements of the
// reference's decode path, each citing the reference lines it follows. Paths
// are relative to the reference project root.
//
// Where the reference sums sequentially inside one work-item, a fixed lane
// partition and combine tree is stated instead, so that a parallel
// implementation can reproduce the result bit for bit. The partition never
// depends on the machine (SM count, thread count): it is part of the contract.
#pragma once
#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <vector>

#include "oracle_math.h"

namespace orc {

// ---------------------------------------------------------------- weights ---
// Symmetric INT4, group 128 along K, scale = amax/7 in fp32 (1.0 if amax==0),
// q = clip(rint(w/scale), -8, 7) with the fp32 scale, scale stored as BF16.
// Two nibbles per byte, low nibble = even index. (tools/binfer.py:76-91;
// C++ twin tools/gemv/gemv.cpp:46-71.)
static inline void quantize_int4_g128(const float *w, size_t numel, uint8_t *packed,
                                      uint16_t *scales) {
  size_t ng = (numel + 127) / 128;
  for (size_t g = 0; g < ng; ++g) {
    float v[128];
    float amax = 0.0f;
    for (int j = 0; j < 128; ++j) {
      size_t i = g * 128 + j;
      v[j] = i < numel ? w[i] : 0.0f;
      float a = fabsf(v[j]);
      amax = a > amax ? a : amax;
    }
    float sc = amax == 0.0f ? 1.0f : amax / 7.0f;
    scales[g] = f32_to_bf16(sc);
    for (int j = 0; j < 128; j += 2) {
      int q0 = (int)rintf(v[j] / sc), q1 = (int)rintf(v[j + 1] / sc);
      q0 = q0 < -8 ? -8 : (q0 > 7 ? 7 : q0);
      q1 = q1 < -8 ? -8 : (q1 > 7 ? 7 : q1);
      packed[g * 64 + j / 2] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
    }
  }
}
static inline int nibble_at(const uint8_t *packed, size_t idx) {
  uint8_t b = packed[idx >> 1];
  int nib = (idx & 1) ? (b >> 4) : (b & 0xF);
  return nib >= 8 ? nib - 16 : nib;
}

// ------------------------------------------------------------ activations ---
// Per-128 group INT8: s = max|x|/127 (1 if 0); q = trunc(x/s +- 0.5), clamp
// +-127. (tools/cmdlist/kernels.cpp:551-579; host mirror
// tools/cmdlist/layerlin_replay.cpp:408-423.)
static inline void aquant_g128(const float *x, int n, int8_t *q8, float *sq) {
  for (int g = 0; g < n / 128; ++g) {
    float m = 0.0f;
    for (int j = 0; j < 128; ++j) {
      float a = fabsf(x[g * 128 + j]);
      m = a > m ? a : m;
    }
    float s = m / 127.0f;
    if (s == 0.0f) s = 1.0f;
    sq[g] = s;
    for (int j = 0; j < 128; ++j) {
      float v = x[g * 128 + j] / s;
      int qi = (int)(v >= 0 ? v + 0.5f : v - 0.5f);
      q8[g * 128 + j] = (int8_t)(qi < -127 ? -127 : (qi > 127 ? 127 : qi));
    }
  }
}

// ------------------------------------------------------------------ GEMV ---
// W4A8: exact int32 group dot, then acc += (float)gs * sc * sq[g] in ascending
// group order, fp32. (tools/cmdlist/kernels.cpp:157-191; host mirror
// tools/cmdlist/gemv_replay.cpp:214-229.)
static inline float gemv_a8_row(const uint8_t *P, const uint16_t *S, size_t row, int K,
                                const int8_t *xq, const float *sq) {
  int G = K / 128;
  float acc = 0.0f;
  for (int g = 0; g < G; ++g) {
    float sc = bf16_to_f32(S[row * G + g]);
    const uint8_t *p = P + (row * (size_t)K + (size_t)g * 128) / 2;
    const int8_t *x = xq + g * 128;
    // two's-complement nibbles widened without a branch ((v ^ 8) - 8), then the exact
    // int32 sum of the 128 products; two loops so that the compiler vectorises both
    int8_t w[128];
    for (int j = 0; j < 64; ++j) {
      w[2 * j] = (int8_t)(((p[j] & 0xF) ^ 8) - 8);
      w[2 * j + 1] = (int8_t)(((p[j] >> 4) ^ 8) - 8);
    }
    int gs = 0;
    for (int j = 0; j < 128; ++j) gs += (int)w[j] * (int)x[j];
    float t = (float)gs * sc;
    t = t * sq[g];
    acc = acc + t;
  }
  return acc;
}
static inline void gemv_a8(const uint8_t *P, const uint16_t *S, int N, int K, const int8_t *xq,
                           const float *sq, float *y) {
  parallel_for((int64_t)(N), [&](int64_t n_) {
    int n = (int)n_;
    y[n] = gemv_a8_row(P, S, (size_t)n, K, xq, sq);
  });
}
// Float-activation policy of the operator sweep: sum over k of
// (float)nib * sc * x[k], accumulated in double, cast to float.
// (tools/gemv/gemv.cpp:480-501.) x holds bf16-representable values.
static inline void gemv_a16(const uint8_t *P, const uint16_t *S, int N, int K, const float *x,
                            int M, float *y /* [M][N] */) {
  parallel_for((int64_t)(N), [&](int64_t n_) {
    int n = (int)n_;
    for (int m = 0; m < M; ++m) {
      double acc = 0;
      for (int g = 0; g < K / 128; ++g) {
        float sc = bf16_to_f32(S[(size_t)n * (K / 128) + g]);
        for (int j = 0; j < 128; ++j) {
          size_t idx = (size_t)n * K + g * 128 + j;
          int nib = nibble_at(P, idx);
          acc += (double)((float)nib * sc * x[(size_t)m * K + g * 128 + j]);
        }
      }
      y[(size_t)m * N + n] = (float)acc;
    }
  });
}

// --------------------------------------------------------------- RMSNorm ---
// (1+w) RMSNorm, fp64 sum of squares over 256 strided lanes combined by the
// stride-halving tree, inv = 1/sqrtf((float)(ss/N) + eps), y = x*inv*(1+w).
// (tools/cmdlist/kernels.cpp:99-114; sequential form :88-95 and
// tools/cmdlist/layerlin_replay.cpp:399-407.)
static inline float rms_inv_256(const float *x, int n, float eps) {
  double ps[256];
  for (int l = 0; l < 256; ++l) {
    double ss = 0;
    for (int j = l; j < n; j += 256) {
      double v = (double)x[j];
      ss = ss + v * v;
    }
    ps[l] = ss;
  }
  double tot = tree_sum(ps, 256);
  return 1.0f / sqrtf((float)(tot / (double)n) + eps);
}
static inline void rmsnorm_1pw(const float *x, const float *w, int n, float eps, float *y) {
  float inv = rms_inv_256(x, n, eps);
  for (int j = 0; j < n; ++j) y[j] = (x[j] * inv) * (1.0f + w[j]);
}
// Per-head (1+w) RMSNorm of the attention q/k rows: fp64 sum over 32 strided
// lanes + tree. (tools/cmdlist/kernels.cpp:667-684.)
static inline void headnorm_1pw(const float *x, const float *w, int n, float eps, float *y) {
  double ps[32];
  for (int l = 0; l < 32; ++l) {
    double ss = 0;
    for (int j = l; j < n; j += 32) {
      double v = (double)x[j];
      ss = ss + v * v;
    }
    ps[l] = ss;
  }
  double tot = tree_sum(ps, 32);
  float inv = 1.0f / sqrtf((float)(tot / (double)n) + eps);
  for (int j = 0; j < n; ++j) y[j] = (x[j] * inv) * (1.0f + w[j]);
}

// ------------------------------------------------------------------ RoPE ---
// NeoX half rotation on the leading rot dims: pairs (d, d+rot/2).
// (tools/cmdlist/kernels.cpp:435-444; table tools/decode/decode_l0.cpp:341-349.)
static inline void rope_table(int pos, int rot, double theta, float *cs, float *sn) {
  for (int i = 0; i < rot; ++i) {
    double inv = 1.0 / std::pow(theta, (double)(2 * (i % (rot / 2))) / (double)rot);
    double ang = (double)pos * inv;
    cs[i] = (float)std::cos(ang);
    sn[i] = (float)std::sin(ang);
  }
}
static inline void rope_apply(float *x, int rot, const float *cs, const float *sn) {
  int h = rot / 2;
  for (int d = 0; d < h; ++d) {
    float x0 = x[d], x1 = x[d + h];
    float c = cs[d], s = sn[d];
    x[d] = x0 * c - x1 * s;
    x[d + h] = x0 * s + x1 * c;
  }
}

// ------------------------------------------------------------- attention ---
// Reference form: fp32 scores over a BF16 KV cache, three passes, sigmoid gate.
// (tools/cmdlist/kernels.cpp:225-303; tools/decode/decode.cpp:646-671.) Kept
// to pin the attention math on the reference's own golden vectors.
static inline void attn_decode_bf16kv(const float *q, const uint16_t *Kc, const uint16_t *Vc,
                                      const float *gate, int nQ, int nKV, int D, int T,
                                      float *out, float *wts_out /* [nQ][T] or null */) {
  float scale = 1.0f / sqrtf((float)D);
  std::vector<float> wts(T);
  for (int h = 0; h < nQ; ++h) {
    int kv = h / (nQ / nKV);
    float mx = -1e30f;
    for (int t = 0; t < T; ++t) {
      float s = 0;
      for (int d = 0; d < D; ++d)
        s += q[(size_t)h * D + d] * bf16_to_f32(Kc[((size_t)t * nKV + kv) * D + d]);
      s = s * scale;
      wts[t] = s;
      mx = s > mx ? s : mx;
    }
    float se = 0;
    for (int t = 0; t < T; ++t) {
      wts[t] = det_expf(wts[t] - mx);
      se += wts[t];
    }
    float inv = 1.0f / se;
    for (int d = 0; d < D; ++d) {
      float a = 0;
      for (int t = 0; t < T; ++t)
        a += (wts[t] * inv) * bf16_to_f32(Vc[((size_t)t * nKV + kv) * D + d]);
      out[(size_t)h * D + d] = a / (1.0f + det_expf(-gate[(size_t)h * D + d]));
    }
    if (wts_out)
      for (int t = 0; t < T; ++t) wts_out[(size_t)h * T + t] = wts[t] * inv;
  }
}

// INT8 KV (no reference counterpart: parity unpinned; restated by analogy with
// the activation quantiser, tools/cmdlist/kernels.cpp:551-579). Per token, per
// KV head over D dims: s = max|x|/127 (1 if 0), stored fp16 RNE, quantise with
// the fp16-rounded scale, round half away, clamp +-127.
static inline void kv_quant_row(const float *x, int D, int8_t *q, uint16_t *s16) {
  float m = 0;
  for (int d = 0; d < D; ++d) {
    float a = fabsf(x[d]);
    m = a > m ? a : m;
  }
  float s = m / 127.0f;
  if (s == 0.0f) s = 1.0f;
  uint16_t h = f32_to_f16(s);
  float sf = f16_to_f32(h);
  if (sf == 0.0f) { sf = 1.0f; h = 0x3C00u; }  // scale underflowed in fp16
  *s16 = h;
  for (int d = 0; d < D; ++d) {
    float v = x[d] / sf;
    int qi = (int)(v >= 0 ? v + 0.5f : v - 0.5f);
    q[d] = (int8_t)(qi < -127 ? -127 : (qi > 127 ? 127 : qi));
  }
}

constexpr int kAttnChunk = 64;  // tokens per split; fixed by the contract

// Split attention over the INT8 cache. Per token: dot over 32 lanes of D/32
// consecutive dims each (fma chain) + tree; score = (dot*ks)*scale. Per chunk
// of 64 tokens: local max, w = exp(score-max), se and acc summed in ascending
// t. Chunks combined in ascending order after rescaling to the global max.
// Output (acc/se) / (1 + exp(-gate)).
static inline void attn_decode_int8kv(const float *q, const int8_t *Kc, const uint16_t *Ks,
                                      const int8_t *Vc, const uint16_t *Vs, const float *gate,
                                      int nQ, int nKV, int D, int T, float *out) {
  float scale = 1.0f / sqrtf((float)D);
  int per = D / 32;
  int nch = (T + kAttnChunk - 1) / kAttnChunk;
  parallel_for((int64_t)(nQ), [&](int64_t h_) {
    int h = (int)h_;
    int kv = h / (nQ / nKV);
    std::vector<float> cm(nch), cse(nch), cacc((size_t)nch * D);
    for (int c = 0; c < nch; ++c) {
      int t0 = c * kAttnChunk, t1 = std::min(T, t0 + kAttnChunk);
      float sc[kAttnChunk];
      float mx = -INFINITY;
      for (int t = t0; t < t1; ++t) {
        const int8_t *kr = Kc + ((size_t)t * nKV + kv) * D;
        float ps[32];
        for (int l = 0; l < 32; ++l) {
          float a = 0.0f;
          for (int j = 0; j < per; ++j)
            a = fmaf(q[(size_t)h * D + l * per + j], (float)kr[l * per + j], a);
          ps[l] = a;
        }
        float dot = tree_sum(ps, 32);
        float s = (dot * f16_to_f32(Ks[(size_t)t * nKV + kv])) * scale;
        sc[t - t0] = s;
        mx = s > mx ? s : mx;
      }
      float se = 0.0f;
      float *acc = &cacc[(size_t)c * D];
      for (int d = 0; d < D; ++d) acc[d] = 0.0f;
      for (int t = t0; t < t1; ++t) {
        float w = det_expf(sc[t - t0] - mx);
        se = se + w;
        float pw = w * f16_to_f32(Vs[(size_t)t * nKV + kv]);
        const int8_t *vr = Vc + ((size_t)t * nKV + kv) * D;
        for (int d = 0; d < D; ++d) acc[d] = fmaf(pw, (float)vr[d], acc[d]);
      }
      cm[c] = mx;
      cse[c] = se;
    }
    float M = -INFINITY;
    for (int c = 0; c < nch; ++c) M = cm[c] > M ? cm[c] : M;
    float se = 0.0f;
    std::vector<float> acc(D, 0.0f);
    for (int c = 0; c < nch; ++c) {
      float f = det_expf(cm[c] - M);
      se = fmaf(cse[c], f, se);
      for (int d = 0; d < D; ++d) acc[d] = fmaf(cacc[(size_t)c * D + d], f, acc[d]);
    }
    for (int d = 0; d < D; ++d) {
      float o = acc[d] / se;
      out[(size_t)h * D + d] = o / (1.0f + det_expf(-gate[(size_t)h * D + d]));
    }
  });
}

// ------------------------------------------------------- Gated DeltaNet ---
// Depthwise conv k=4 over [h0,h1,h2,x]*[w0..w3], SiLU, history shift.
// (tools/cmdlist/kernels.cpp:327-337.)
static inline void conv_silu_step(const float *x, float *cs, const float *cw, int C, float *mx) {
  for (int c = 0; c < C; ++c) {
    float acc = cs[c * 3 + 0] * cw[(size_t)c * 4 + 0];
    acc = acc + cs[c * 3 + 1] * cw[(size_t)c * 4 + 1];
    acc = acc + cs[c * 3 + 2] * cw[(size_t)c * 4 + 2];
    acc = acc + x[c] * cw[(size_t)c * 4 + 3];
    mx[c] = acc / (1.0f + det_expf(-acc));
    cs[c * 3 + 0] = cs[c * 3 + 1];
    cs[c * 3 + 1] = cs[c * 3 + 2];
    cs[c * 3 + 2] = x[c];
  }
}
// Sum of squares over one 128-wide head: 32 strided lanes (fma chains) + tree.
static inline float sumsq_head(const float *x, int n) {
  float ps[32];
  for (int l = 0; l < 32; ++l) {
    float a = 0.0f;
    for (int j = l; j < n; j += 32) a = fmaf(x[j], x[j], a);
    ps[l] = a;
  }
  return tree_sum(ps, 32);
}
// l2norm with eps added to the sum; q additionally scaled by head_dim^-1/2.
// (tools/cmdlist/kernels.cpp:592-604.)
static inline void l2norm_head(const float *x, int n, float mul, float *y) {
  float ss = sumsq_head(x, n);
  float inv = 1.0f / sqrtf(ss + 1e-6f);
  float f = inv * mul;
  for (int d = 0; d < n; ++d) y[d] = x[d] * f;
}
// beta = sigmoid(b); g = -exp(A_log) * softplus(a + dt_bias), softplus passes
// through above 20. (tools/cmdlist/kernels.cpp:610-616.)
static inline float dn_beta(float b) { return 1.0f / (1.0f + det_expf(-b)); }
static inline float dn_gdecay(float a, float a_log, float dt) {
  float sa = a + dt;
  float soft = sa > 20.0f ? sa : det_logf(1.0f + det_expf(sa));
  return (-det_expf(a_log)) * soft;
}
// One recurrence step for one head; S is [k][v] row-major, D x D.
// S *= exp(g); kv = S^T k; delta = (v - kv)*beta; S += k delta^T; o = S^T q.
// (tools/cmdlist/kernels.cpp:354-409; host mirror
// tools/cmdlist/layerlin_replay.cpp:483-506.) The k dimension is summed as 8
// segments of D/8 rows (fma chains) combined ((0+1)+(2+3))+((4+5)+(6+7)).
static inline float tree8(const float *p) {
  return ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));
}
static inline void deltanet_head_step(float *S, const float *q, const float *k, const float *v,
                                      float beta, float g, int D, float *o) {
  float gt = det_expf(g);
  int seg = D / 8;
  for (int i = 0; i < D * D; ++i) S[i] = S[i] * gt;
  for (int c = 0; c < D; ++c) {
    float p[8];
    for (int s = 0; s < 8; ++s) {
      float a = 0.0f;
      for (int r = s * seg; r < (s + 1) * seg; ++r) a = fmaf(S[(size_t)r * D + c], k[r], a);
      p[s] = a;
    }
    float kv = tree8(p);
    float dl = (v[c] - kv) * beta;
    for (int r = 0; r < D; ++r) S[(size_t)r * D + c] = fmaf(k[r], dl, S[(size_t)r * D + c]);
    for (int s = 0; s < 8; ++s) {
      float a = 0.0f;
      for (int r = s * seg; r < (s + 1) * seg; ++r) a = fmaf(S[(size_t)r * D + c], q[r], a);
      p[s] = a;
    }
    o[c] = tree8(p);
  }
}
// Per-head inverse RMS and gated norm with the plain weight.
// (tools/cmdlist/kernels.cpp:619-644.)
static inline void gated_norm_head(const float *o, const float *z, const float *w, int D,
                                   float *y) {
  float ss = sumsq_head(o, D);
  float inv = 1.0f / sqrtf(ss / (float)D + 1e-6f);
  for (int d = 0; d < D; ++d) {
    float zv = z[d];
    y[d] = ((w[d] * o[d]) * inv) * (zv / (1.0f + det_expf(-zv)));
  }
}

// ------------------------------------------------------------------- MoE ---
// (No reference counterpart: parity unpinned.) Router logits from a BF16
// matrix and the fp32 normalised activations: 32 lanes, lane l takes k =
// (i*32+l)*8+j, fma chain in (i, j) order, then the tree.
static inline float dot_bf16_row(const uint16_t *w, const float *x, int K) {
  float ps[32];
  for (int l = 0; l < 32; ++l) {
    float a = 0.0f;
    for (int i = 0; i < K / 256; ++i)
      for (int j = 0; j < 8; ++j) {
        int k = (i * 32 + l) * 8 + j;
        a = fmaf(bf16_to_f32(w[k]), x[k], a);
      }
    ps[l] = a;
  }
  return tree_sum(ps, 32);
}
// Softmax over all experts (max-subtracted; sum over 32 strided lanes + tree),
// top-k by (probability desc, index asc), weights renormalised to sum 1 with
// the sum taken in rank order. near_gap returns the relative gap between the
// k-th and (k+1)-th probability (a "near tie" is < 1e-5).
static inline void router_topk(const float *logits, int E, int k, int *idx, float *wt,
                               float *near_gap) {
  float m = -INFINITY;
  for (int e = 0; e < E; ++e) m = logits[e] > m ? logits[e] : m;
  std::vector<float> p(E);
  float ps[32];
  for (int l = 0; l < 32; ++l) ps[l] = 0.0f;
  for (int e = 0; e < E; ++e) p[e] = det_expf(logits[e] - m);
  for (int l = 0; l < 32; ++l) {
    float a = 0.0f;
    for (int e = l; e < E; e += 32) a = a + p[e];
    ps[l] = a;
  }
  float sum = tree_sum(ps, 32);
  for (int e = 0; e < E; ++e) p[e] = p[e] / sum;
  std::vector<char> used(E, 0);
  float s = 0.0f;
  for (int j = 0; j <= k && j < E; ++j) {
    int best = -1;
    for (int e = 0; e < E; ++e)
      if (!used[e] && (best < 0 || p[e] > p[best])) best = e;
    if (j == k) {
      if (near_gap) {
        float lastp = p[idx[k - 1]];
        *near_gap = lastp > 0 ? (lastp - p[best]) / lastp : 0.0f;
      }
      break;
    }
    used[best] = 1;
    idx[j] = best;
    wt[j] = p[best];
    s = s + p[best];
  }
  if (k >= E && near_gap) *near_gap = 1.0f;
  for (int j = 0; j < k; ++j) wt[j] = wt[j] / s;
}

// ---------------------------------------------------------------- argmax ---
// First-max-wins. (tools/cmdlist/kernels.cpp:492-495; tools/sample/sampler.h:63-71.)
static inline int argmax_first(const float *x, int n) {
  int best = 0;
  float bv = x[0];
  for (int i = 1; i < n; ++i)
    if (x[i] > bv) { bv = x[i]; best = i; }
  return best;
}

}  // namespace orc
