// Kernels of batched decode: B sequences advance one token each per step, every sequence with
// its own recurrent state, conv history, KV cache and control block. Each is the single-sequence
// decode kernel's body run for sequence blockIdx.x / groups_per_sequence with that sequence's
// pointers (the bodies are shared: deltanet_core.cuh, attention_core.cuh), so a sequence's row
// is bit-identical to decoding it alone. The reference decodes one sequence (its batching was
// dropped); the per-sequence arithmetic follows the same reference kernels as the decode path
// (SsmConv / SsmRecur tools/cmdlist/kernels.cpp:322-410, AttnCore :210-304, Argmax :480-549).
#include "attention_core.cuh"
#include "deltanet_core.cuh"
#include "tail_core.cuh"

namespace ainfer {

// ---- conv k = 4 + SiLU + history shift, one thread per (sequence, channel) ----
struct BatchConvSiluArgs {
  float *Mx;          // [B][C]
  const float *QKV;   // [B][C]
  float *CS;          // sequence b's history [C][3] at CS + b * cs_stride
  const float *CW;    // [C][4]
  int32_t C, B;
  int64_t cs_stride;  // floats between two sequences' histories
};
__global__ void __launch_bounds__(256) BatchConvSilu(const BatchConvSiluArgs a) {
  const long i = (long)blockIdx.x * 256 + threadIdx.x;
  if (i >= (long)a.B * a.C) return;
  const int b = (int)(i / a.C), c = (int)(i % a.C);
  float *cs = a.CS + (size_t)b * a.cs_stride + (size_t)c * 3;
  const float4 w = __ldg(reinterpret_cast<const float4 *>(a.CW) + c);
  const float h0 = cs[0], h1 = cs[1], h2 = cs[2], x = a.QKV[i];
  float acc = h0 * w.x;
  acc = acc + h1 * w.y;
  acc = acc + h2 * w.z;
  acc = acc + x * w.w;
  a.Mx[i] = acc / (1.0f + det_expf(-acc));
  cs[0] = h1; cs[1] = h2; cs[2] = x;
}

// ---- gated delta rule step of every sequence: nV * 4 blocks per sequence ----
struct BatchDeltaNetStepArgs {
  float *Out;        // [B][nV][128]
  const float *Mx;   // [B][C]
  float *S;          // sequence b's state [nV][128][128] at S + b * s_stride
  const float *Bt;   // [B][nV]
  const float *Gt;   // [B][nV]
  int32_t nK, nV, B;
  int64_t s_stride;  // floats between two sequences' states
};
__global__ void __launch_bounds__(256) BatchDeltaNetStep(const BatchDeltaNetStepArgs a) {
  const int per = a.nV * kDnSlices, b = blockIdx.x / per;
  if (b >= a.B) return;
  const int C = 2 * a.nK * 128 + a.nV * 128;
  DeltaNetStepArgs s;
  s.Out = a.Out + (size_t)b * a.nV * 128;
  s.Mx = a.Mx + (size_t)b * C;
  s.S = a.S + (size_t)b * a.s_stride;
  s.Bt = a.Bt + (size_t)b * a.nV;
  s.Gt = a.Gt + (size_t)b * a.nV;
  s.nK = a.nK; s.nV = a.nV;
  deltanet_step_body(s, blockIdx.x % per, per);
}

// ---- attention of every sequence against its own INT8 cache ----
struct BatchAttnArgs {
  const float *Q16, *K16, *V16;   // [B][nQ*2D], [B][nKV*D], [B][nKV*D]
  const float *QNW, *KNW, *Cos, *Sin;
  const int32_t *Ctrl;            // [B][4]
  float *Qn;                      // [B][nQ*D]
  int8_t *Kc, *Vc;                // sequence b's cache of this layer at + b * kv_stride (elements of D bytes: rows)
  uint16_t *Ks, *Vs;
  float *Pm, *Pse, *Pacc;         // [B][nQ*max_chunks], [B][nQ*max_chunks], [B][nQ*max_chunks*D]
  int8_t *Q8;                     // [B][nQ*D]
  float *SQ;                      // [B][nQ*D/128]
  int32_t nQ, nKV, rot, max_ctx, max_chunks, B, groups;   // groups: blocks per sequence of this launch
  float eps;
  int64_t kv_stride;              // cache rows (of nKV heads) between two sequences
};
__global__ void __launch_bounds__(256) BatchAttnPrep(const BatchAttnArgs a) {
  const int b = blockIdx.x / a.groups;
  if (b >= a.B) return;
  AttnPrepArgs p;
  p.Q16 = a.Q16 + (size_t)b * a.nQ * 2 * kHeadDim; p.K16 = a.K16 + (size_t)b * a.nKV * kHeadDim; p.V16 = a.V16 + (size_t)b * a.nKV * kHeadDim;
  p.QNW = a.QNW; p.KNW = a.KNW; p.Cos = a.Cos; p.Sin = a.Sin;
  p.Ctrl = a.Ctrl + 4 * b;
  p.Qn = a.Qn + (size_t)b * a.nQ * kHeadDim;
  p.Kc = a.Kc + (size_t)b * a.kv_stride * a.nKV * kHeadDim; p.Vc = a.Vc + (size_t)b * a.kv_stride * a.nKV * kHeadDim;
  p.Ks = a.Ks + (size_t)b * a.kv_stride * a.nKV; p.Vs = a.Vs + (size_t)b * a.kv_stride * a.nKV;
  p.nQ = a.nQ; p.nKV = a.nKV; p.rot = a.rot; p.max_ctx = a.max_ctx; p.eps = a.eps;
  attn_prep_body(p, blockIdx.x % a.groups, a.groups);
}
// From this many items in a launch the one-warp-per-item form of the split is used.
constexpr long kWarpFormItems = 2048;
__global__ void __launch_bounds__(256, 2) BatchAttnSplit(const BatchAttnArgs a) {
  const int b = blockIdx.x / a.groups;
  if (b >= a.B) return;
  AttnSplitArgs p;
  p.Qn = a.Qn + (size_t)b * a.nQ * kHeadDim;
  p.Kc = a.Kc + (size_t)b * a.kv_stride * a.nKV * kHeadDim; p.Vc = a.Vc + (size_t)b * a.kv_stride * a.nKV * kHeadDim;
  p.Ks = a.Ks + (size_t)b * a.kv_stride * a.nKV; p.Vs = a.Vs + (size_t)b * a.kv_stride * a.nKV;
  p.Ctrl = a.Ctrl + 4 * b;
  p.Pm = a.Pm + (size_t)b * a.nQ * a.max_chunks; p.Pse = a.Pse + (size_t)b * a.nQ * a.max_chunks;
  p.Pacc = a.Pacc + (size_t)b * a.nQ * a.max_chunks * kHeadDim;
  p.nQ = a.nQ; p.nKV = a.nKV; p.max_ctx = a.max_ctx; p.max_chunks = a.max_chunks;
  attn_split_dispatch<true>(p, blockIdx.x % a.groups, a.groups, a.B, kWarpFormItems);
}
__global__ void __launch_bounds__(256) BatchAttnCombine(const BatchAttnArgs a) {
  const int b = blockIdx.x / a.groups;
  if (b >= a.B) return;
  AttnCombineArgs p;
  p.Pm = a.Pm + (size_t)b * a.nQ * a.max_chunks; p.Pse = a.Pse + (size_t)b * a.nQ * a.max_chunks;
  p.Pacc = a.Pacc + (size_t)b * a.nQ * a.max_chunks * kHeadDim;
  p.Q16 = a.Q16 + (size_t)b * a.nQ * 2 * kHeadDim;
  p.Ctrl = a.Ctrl + 4 * b;
  p.Q8 = a.Q8 + (size_t)b * a.nQ * kHeadDim;
  p.SQ = a.SQ + (size_t)b * (a.nQ * kHeadDim / 128);
  p.Att = nullptr;
  p.nQ = a.nQ; p.max_ctx = a.max_ctx; p.max_chunks = a.max_chunks;
  attn_combine_body(p, blockIdx.x % a.groups, a.groups);
}

// ---- greedy token of every sequence (first maximum wins) and its control block's advance ----
struct BatchArgmaxArgs {
  const float *Logits;   // [B][V]
  int32_t *OutT;         // [B]
  int32_t *Ctrl;         // [B][4]: {selected, position + 1, length + 1, selected} when advance != 0
  int32_t V, advance;
};
__global__ void __launch_bounds__(1024) BatchArgmax(const BatchArgmaxArgs a) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int b = blockIdx.x;
  const float *lg = a.Logits + (size_t)b * a.V;
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  for (int i = threadIdx.x; i < a.V; i += 1024) argmax_merge(bv, bi, lg[i], i);
  block_argmax(bv, bi, sv, si);
  if (threadIdx.x == 0) {
    a.OutT[b] = bi;
    int32_t *c = a.Ctrl + 4 * b;
    c[CTRL_SELECTED] = bi;
    if (a.advance) {
      c[CTRL_TOKEN] = bi;
      c[CTRL_POS] = c[CTRL_POS] + 1;
      c[CTRL_LEN] = c[CTRL_LEN] + 1;
    }
  }
}

#define F(f) AINFER_ARG(BatchConvSiluArgs, f)
AINFER_REGISTER(BatchConvSilu, BatchConvSiluArgs, 256, 256, 0, nullptr, F(Mx), F(QKV), F(CS), F(CW), F(C), F(B), F(cs_stride));
#undef F
#define F(f) AINFER_ARG(BatchDeltaNetStepArgs, f)
AINFER_REGISTER(BatchDeltaNetStep, BatchDeltaNetStepArgs, 256, 1, 0, nullptr, F(Out), F(Mx), F(S), F(Bt), F(Gt), F(nK), F(nV), F(B), F(s_stride));
#undef F
#define BATCH_ATTN_FIELDS                                                                                                          \
  F(Q16), F(K16), F(V16), F(QNW), F(KNW), F(Cos), F(Sin), F(Ctrl), F(Qn), F(Kc), F(Vc), F(Ks), F(Vs), F(Pm), F(Pse), F(Pacc), F(Q8), \
      F(SQ), F(nQ), F(nKV), F(rot), F(max_ctx), F(max_chunks), F(B), F(groups), F(eps), F(kv_stride)
#define F(f) AINFER_ARG(BatchAttnArgs, f)
AINFER_REGISTER(BatchAttnPrep, BatchAttnArgs, 256, 1, 0, nullptr, BATCH_ATTN_FIELDS);
AINFER_REGISTER(BatchAttnSplit, BatchAttnArgs, 256, 1, 0, nullptr, BATCH_ATTN_FIELDS);
AINFER_REGISTER(BatchAttnCombine, BatchAttnArgs, 256, 1, 0, nullptr, BATCH_ATTN_FIELDS);
#undef F
#define F(f) AINFER_ARG(BatchArgmaxArgs, f)
AINFER_REGISTER(BatchArgmax, BatchArgmaxArgs, 1024, 1, 0, nullptr, F(Logits), F(OutT), F(Ctrl), F(V), F(advance));
#undef F

}  // namespace ainfer
