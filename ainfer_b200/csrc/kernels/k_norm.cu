// EmbedRow, RmsNormQuant, GatedNormQuant: the row-wise stages between GEMVs.
// One launch each replaces chains of single-purpose kernels in the reference's
// recorded lists (tools/decode/decode_l0.cpp:505-530,547-551,651-660):
//   RmsNormQuant   = [ResAddF] + RMSNormW + ScalesMax + Quantize
//   GatedNormQuant = RmsInv + NormGated + ScalesMax + Quantize
#include "common.cuh"

namespace ainfer {

// ------------------------------------------------------------- EmbedRow ---
// X[i] = bf16 -> f32 of Emb[token*H + i], token = Ctrl[0] (clamped to the
// table). (Embed, tools/cmdlist/kernels.cpp:1035.)
struct EmbedRowArgs {
  float *X;
  const uint16_t *Emb;
  const int32_t *Ctrl;
  int32_t H;
  int32_t V;
  int32_t ctrl_stride;  // ints between control blocks of consecutive batch rows
};
__global__ void __launch_bounds__(256) EmbedRow(const EmbedRowArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  int row = blockIdx.x;  // one group per batch row
  int tok = a.Ctrl[row * a.ctrl_stride + CTRL_TOKEN];
  tok = tok < 0 ? 0 : (tok >= a.V ? a.V - 1 : tok);
  const uint16_t *src = a.Emb + (size_t)tok * a.H;
  for (int i = threadIdx.x; i < a.H; i += blockDim.x)
    a.X[(size_t)row * a.H + i] = bf16_to_f32(src[i]);
}
#define F(f) AINFER_ARG(EmbedRowArgs, f)
AINFER_REGISTER(EmbedRow, EmbedRowArgs, 256, 1, 0, nullptr, F(X), F(Emb), F(Ctrl), F(H), F(V),
                F(ctrl_stride));
#undef F

// --------------------------------------------------------- RmsNormQuant ---
// Optional residual add (Y = A + B, ResAddF kernels.cpp:646-652), (1+w) RMSNorm
// with the fp64 sum of squares over 256 strided lanes and the stride-halving
// tree (RMSNormW, kernels.cpp:99-114), then the per-128 activation quantiser
// (ScalesMax + Quantize, kernels.cpp:551-579). One group per batch row.
struct RmsNormQuantArgs {
  const float *A;     // input row(s) [rows][N]
  const float *B;     // optional second addend (null: none)
  float *Sum;         // optional: A + B written here (the new residual stream)
  const float *W;     // norm weight [N]
  float *Hn;          // optional normalised fp32 output [rows][N]
  int8_t *Q8;         // quantised output [rows][N]
  float *SQ;          // group scales [rows][N/128]
  int32_t N;
  float eps;
};
__global__ void __launch_bounds__(256) RmsNormQuant(const RmsNormQuantArgs a) {
  pdl_launch_dependents();
  // the norm weight does not depend on the predecessor: fetch this lane's share of the first
  // groups of its warp while waiting (groups warp, warp + 8, ...)
  constexpr int kPre = 2;
  float4 wpre[kPre];
#pragma unroll
  for (int i = 0; i < kPre; ++i) {
    const int g = (threadIdx.x >> 5) + 8 * i;
    wpre[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (g < a.N / 128) wpre[i] = __ldg(reinterpret_cast<const float4 *>(a.W + g * 128) + (threadIdx.x & 31));
  }
  pdl_wait();
  extern __shared__ __align__(16) unsigned char norm_smem[];
  float *xs = reinterpret_cast<float *>(norm_smem);  // [N]
  __shared__ double ps[256];
  __shared__ float s_inv;
  const int row = blockIdx.x, lid = threadIdx.x, N = a.N;
  const float *A = a.A + (size_t)row * N;
  const float *B = a.B ? a.B + (size_t)row * N : nullptr;
  double ss = 0;
  for (int j = lid; j < N; j += 256) {
    float v = A[j];
    if (B) v = v + B[j];
    xs[j] = v;
    if (a.Sum) a.Sum[(size_t)row * N + j] = v;
    double d = (double)v;
    ss = ss + d * d;
  }
  ps[lid] = ss;
  __syncthreads();
  for (int st = 128; st >= 32; st >>= 1) {
    if (lid < st) ps[lid] = ps[lid] + ps[lid + st];
    __syncthreads();
  }
  if (lid < 32) {
    double v = ps[lid];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = v + __shfl_xor_sync(kFull, v, off);
    if (lid == 0) s_inv = 1.0f / sqrtf((float)(v / (double)N) + a.eps);
  }
  __syncthreads();
  const float inv = s_inv;
  // one warp per group of 128: lane holds 4 consecutive elements
  const int warp = lid >> 5, lane = lid & 31;
  for (int g = warp; g < N / 128; g += 8) {
    int j = g * 128 + lane * 4;
    float4 x = *reinterpret_cast<const float4 *>(xs + j);
    const int it = (g - warp) >> 3;
    float4 w = it == 0 ? wpre[0] : it == 1 ? wpre[1] : *reinterpret_cast<const float4 *>(a.W + j);
    float4 y;
    y.x = (x.x * inv) * (1.0f + w.x);
    y.y = (x.y * inv) * (1.0f + w.y);
    y.z = (x.z * inv) * (1.0f + w.z);
    y.w = (x.w * inv) * (1.0f + w.w);
    if (a.Hn) *reinterpret_cast<float4 *>(a.Hn + (size_t)row * N + j) = y;
    float m = fmaxf(fmaxf(fabsf(y.x), fabsf(y.y)), fmaxf(fabsf(y.z), fabsf(y.w)));
    m = warp_max(m);
    float s = m / 127.0f;
    if (s == 0.0f) s = 1.0f;
    if (lane == 0) a.SQ[(size_t)row * (N / 128) + g] = s;
    int q0 = quant_round(y.x, s), q1 = quant_round(y.y, s), q2 = quant_round(y.z, s),
        q3 = quant_round(y.w, s);
    uint32_t packed = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) |
                      ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
    *reinterpret_cast<uint32_t *>(a.Q8 + (size_t)row * N + j) = packed;
  }
}
static uint32_t rmsnorm_smem_fn(const void *args) {
  return (uint32_t)((const RmsNormQuantArgs *)args)->N * 4u;
}
#define F(f) AINFER_ARG(RmsNormQuantArgs, f)
AINFER_REGISTER(RmsNormQuant, RmsNormQuantArgs, 256, 1, 0, rmsnorm_smem_fn, F(A), F(B), F(Sum),
                F(W), F(Hn), F(Q8), F(SQ), F(N), F(eps));
#undef F

// ------------------------------------------------------- GatedNormQuant ---
// Per head of 128: inv = 1/sqrtf(sum(o^2)/128 + eps) (RmsInv, kernels.cpp:
// 632-644; sum over 32 strided lanes as fma chains + tree), y = ((w*o)*inv) *
// silu(z) (NormGated, kernels.cpp:619-630, plain weight), then the activation
// quantiser with the head as the group. One warp per head.
struct GatedNormQuantArgs {
  const float *O;   // [heads][128] recurrence output
  const float *Z;   // [heads][128] gate input
  const float *W;   // [128]
  int8_t *Q8;       // [heads*128]
  float *SQ;        // [heads]
  float *Y;         // optional fp32 copy of the gated output
  int32_t heads;
  float eps;
};
__global__ void __launch_bounds__(128) GatedNormQuant(const GatedNormQuantArgs a) {
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float wn[4];  // the norm weight does not depend on the predecessor
#pragma unroll
  for (int i = 0; i < 4; ++i) wn[i] = __ldg(a.W + lane + 32 * i);
  pdl_wait();
  for (int h = blockIdx.x * 4 + warp; h < a.heads; h += gridDim.x * 4) {
    const float *o = a.O + (size_t)h * 128;
    const float *z = a.Z + (size_t)h * 128;
    float ov[4], y[4];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ov[i] = o[lane + 32 * i];
      ss = fmaf(ov[i], ov[i], ss);
    }
    ss = warp_tree_sum(ss);
    float inv = 1.0f / sqrtf(ss / 128.0f + a.eps);
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int d = lane + 32 * i;
      float zv = z[d];
      y[i] = ((wn[i] * ov[i]) * inv) * (zv / (1.0f + det_expf(-zv)));
      m = fmaxf(m, fabsf(y[i]));
    }
    m = warp_max(m);
    float s = m / 127.0f;
    if (s == 0.0f) s = 1.0f;
    if (lane == 0) a.SQ[h] = s;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int d = lane + 32 * i;
      a.Q8[(size_t)h * 128 + d] = (int8_t)quant_round(y[i], s);
      if (a.Y) a.Y[(size_t)h * 128 + d] = y[i];
    }
  }
}
#define F(f) AINFER_ARG(GatedNormQuantArgs, f)
AINFER_REGISTER(GatedNormQuant, GatedNormQuantArgs, 128, 4, 0, nullptr, F(O), F(Z), F(W), F(Q8),
                F(SQ), F(Y), F(heads), F(eps));
#undef F

// ------------------------------------------------------------ QuantRows ---
// Plain activation quantiser (ScalesMax + Quantize, kernels.cpp:551-579) for
// callers that hold fp32 activations: one warp per group of 128.
struct QuantRowsArgs {
  const float *X;
  int8_t *Q8;
  float *SQ;
  int32_t groups;
};
__global__ void __launch_bounds__(256) QuantRows(const QuantRowsArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = blockIdx.x * 8 + warp; g < a.groups; g += gridDim.x * 8) {
    float4 x = *reinterpret_cast<const float4 *>(a.X + (size_t)g * 128 + lane * 4);
    float m = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
    m = warp_max(m);
    float s = m / 127.0f;
    if (s == 0.0f) s = 1.0f;
    if (lane == 0) a.SQ[g] = s;
    uint32_t packed = (uint32_t)(quant_round(x.x, s) & 0xFF) |
                      ((uint32_t)(quant_round(x.y, s) & 0xFF) << 8) |
                      ((uint32_t)(quant_round(x.z, s) & 0xFF) << 16) |
                      ((uint32_t)(quant_round(x.w, s) & 0xFF) << 24);
    *reinterpret_cast<uint32_t *>(a.Q8 + (size_t)g * 128 + lane * 4) = packed;
  }
}
#define F(f) AINFER_ARG(QuantRowsArgs, f)
AINFER_REGISTER(QuantRows, QuantRowsArgs, 256, 8, 0, nullptr, F(X), F(Q8), F(SQ), F(groups));
#undef F

AINFER_EARLY_LAUNCH(EmbedRow);
AINFER_EARLY_LAUNCH(RmsNormQuant);
AINFER_EARLY_LAUNCH(GatedNormQuant);
AINFER_EARLY_LAUNCH(QuantRows);

}  // namespace ainfer
