// Mixture-of-experts block of the decode loop: RouterTopK, ExpertGateUp,
// ExpertDownCombine. The reference's MLP is dense (gate/up GEMV, SiluMul,
// quantise, down GEMV, ResAddF: tools/decode/decode_l0.cpp:666-674); each
// expert here is that same MLP, the routing around it has no reference
// counterpart and follows the arithmetic stated with each kernel.
#include "../common/tables.h"
#include "gemv_core.cuh"

namespace ainfer {

// ----------------------------------------------------------- RouterTopK ---
// logits[e] = sum_k bf16(Wr[e][k]) * hn[k]: 32 lanes, lane l takes k =
// (i*32+l)*8+j, fma chain in (i, j) order, then the lane tree. The last block
// to finish runs softmax over all experts (max-subtracted, sum over 32 strided
// lanes + tree), top-k by (probability desc, index asc), renormalises the k
// weights in rank order, and evaluates the shared-expert gate sigmoid.
struct RouterTopKArgs {
  const uint16_t *Wr;    // [E][H] bf16 router
  const uint16_t *Wsg;   // [H] bf16 shared-expert gate row (null: no shared expert)
  const float *Hn;       // [H] normalised activations (fp32)
  float *Logits;         // [E+1] scratch
  uint32_t *Counter;     // zero-initialised arrival counter, left at zero
  int32_t *SelIdx;       // [k+1]: routed expert ids in rank order, then E (shared slot)
  float *SelW;           // [k+1]: renormalised weights, then sigmoid(shared gate)
  float *NearGap;        // [1] relative gap between the k-th and (k+1)-th probability
  int32_t E, H, k;
};
__global__ void __launch_bounds__(256) RouterTopK(const RouterTopKArgs a) {
  __shared__ bool is_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = a.E + (a.Wsg ? 1 : 0);
  for (int e = blockIdx.x * 8 + warp; e < rows; e += gridDim.x * 8) {
    const uint16_t *w = e < a.E ? a.Wr + (size_t)e * a.H : a.Wsg;
    float acc = 0.0f;
    for (int i = 0; i < a.H / 256; ++i) {
      int k0 = (i * 32 + lane) * 8;
      uint4 wv = *reinterpret_cast<const uint4 *>(w + k0);
      float4 x0 = *reinterpret_cast<const float4 *>(a.Hn + k0);
      float4 x1 = *reinterpret_cast<const float4 *>(a.Hn + k0 + 4);
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
    if (lane == 0) a.Logits[e] = acc;
  }
  // last block to arrive does the selection
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned prev = atomicAdd(a.Counter, 1u);
    is_last = prev == gridDim.x - 1;
    if (is_last) *a.Counter = 0u;
  }
  __syncthreads();
  if (!is_last || warp != 0) return;
  __threadfence();
  constexpr int NI = 32;  // up to 1024 experts
  const volatile float *lg = a.Logits;
  float p[NI];
  bool used[NI];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    int e = lane + 32 * i;
    p[i] = e < a.E ? lg[e] : -INFINITY;
    used[i] = e >= a.E;
    m = fmaxf(m, p[i]);
  }
  m = warp_max(m);
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    int e = lane + 32 * i;
    if (e < a.E) {
      p[i] = det_expf(p[i] - m);
      sum = sum + p[i];
    }
  }
  sum = warp_tree_sum(sum);
#pragma unroll
  for (int i = 0; i < NI; ++i)
    if (lane + 32 * i < a.E) p[i] = p[i] / sum;
  float s = 0.0f, lastp = 0.0f;
  float wsel = 0.0f;  // lane j keeps the weight of rank j (k <= 32)
  for (int j = 0; j <= a.k && j < a.E; ++j) {
    float bv = -1.0f;
    int bi = 0x7FFFFFFF;
#pragma unroll
    for (int i = 0; i < NI; ++i)
      if (!used[i] && p[i] > bv) { bv = p[i]; bi = lane + 32 * i; }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      float ov = __shfl_xor_sync(kFull, bv, off);
      int oi = __shfl_xor_sync(kFull, bi, off);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (j == a.k) {
      if (lane == 0) *a.NearGap = lastp > 0.0f ? (lastp - bv) / lastp : 0.0f;
      break;
    }
    if ((bi & 31) == lane) {
#pragma unroll
      for (int i = 0; i < NI; ++i)
        if (i == (bi >> 5)) used[i] = true;
    }
    if (lane == j) wsel = bv;
    if (lane == 0) a.SelIdx[j] = bi;
    s = s + bv;
    lastp = bv;
  }
  if (a.k >= a.E && lane == 0) *a.NearGap = 1.0f;
  if (lane < a.k) a.SelW[lane] = wsel / s;
  if (lane == 0) {
    a.SelIdx[a.k] = a.E;
    a.SelW[a.k] = a.Wsg ? 1.0f / (1.0f + det_expf(-lg[a.E])) : 0.0f;
  }
}
#define F(f) AINFER_ARG(RouterTopKArgs, f)
AINFER_REGISTER(RouterTopK, RouterTopKArgs, 256, 8, 0, nullptr, F(Wr), F(Wsg), F(Hn), F(Logits),
                F(Counter), F(SelIdx), F(SelW), F(NearGap), F(E), F(H), F(k));
#undef F

extern __shared__ __align__(16) unsigned char moe_smem[];

// --------------------------------------------------------- ExpertGateUp ---
// For every active slot s (routed experts in rank order, then the shared
// expert) and every intermediate row n: g = gate_e[n].h, u = up_e[n].h (W4A8
// GEMV), Act[s][n] = (g / (1 + exp(-g))) * u  (SiluMul, kernels.cpp:29-37).
struct ExpertGateUpArgs {
  const ExpertW *Experts;  // [E+1]
  const int32_t *SelIdx;   // [slots]
  const int8_t *XQ;        // [H] quantised hidden
  const float *SQ;         // [H/128]
  float *Act;              // [slots][I]
  int32_t slots, I, H;
  int32_t slot_begin;      // first slot this launch handles (expert-parallel ranks)
};
template <int K>
__device__ __forceinline__ void gateup_body(const ExpertGateUpArgs &a) {
  using Gm = RowGeom<K>;
  StagedAct act = stage_act(moe_smem, a.XQ, a.SQ, K, 1, K, K / 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const long total = (long)a.slots * a.I;
  const long tile = (long)warps * Gm::RPW;
  for (long base = (long)blockIdx.x * tile; base < total; base += (long)gridDim.x * tile) {
    long r = base + (long)warp * Gm::RPW + lane / Gm::LPR;
    if (base + (long)warp * Gm::RPW >= total) continue;
    bool ok = r < total;
    int s = ok ? (int)(r / a.I) : 0, n = ok ? (int)(r % a.I) : 0;
    const ExpertW &ew = a.Experts[a.SelIdx[a.slot_begin + s]];
    LaneRows<2> rows;
    rows.ok[0] = rows.ok[1] = ok;
    rows.P[0] = ew.gP + (long)n * (K / 2);
    rows.S[0] = ew.gS + (long)n * Gm::G;
    rows.P[1] = ew.uP + (long)n * (K / 2);
    rows.S[1] = ew.uS + (long)n * Gm::G;
    float acc[2][1];
    warp_rows_dot<K, 1, 2>(rows, act, acc);
    if (ok && (lane % Gm::LPR) == 0) {
      float g = acc[0][0], u = acc[1][0];
      a.Act[(size_t)(a.slot_begin + s) * a.I + n] = (g / (1.0f + det_expf(-g))) * u;
    }
  }
}
__global__ void __launch_bounds__(256) ExpertGateUp(const ExpertGateUpArgs a) {
  switch (a.H) {
    case 256: gateup_body<256>(a); break;
    case 512: gateup_body<512>(a); break;
    case 1024: gateup_body<1024>(a); break;
    case 2048: gateup_body<2048>(a); break;
    case 4096: gateup_body<4096>(a); break;
    default: break;
  }
}
static uint32_t gateup_smem_fn(const void *args) {
  return staged_act_bytes(((const ExpertGateUpArgs *)args)->H, 1);
}
#define F(f) AINFER_ARG(ExpertGateUpArgs, f)
AINFER_REGISTER(ExpertGateUp, ExpertGateUpArgs, 256, 0, 0, gateup_smem_fn, F(Experts), F(SelIdx),
                F(XQ), F(SQ), F(Act), F(slots), F(I), F(H), F(slot_begin));
#undef F

// ---------------------------------------------------- ExpertDownCombine ---
// Quantises each slot's activation (per-128 quantiser), y_s[n] = down_e[n].act_s,
// then out[n] = Res[n] + (sum_s w_s * y_s[n] in rank order, + sg * y_shared[n]),
// products and sums unfused. (Down GEMV + ResAddF, decode_l0.cpp:672-674.)
struct ExpertDownCombineArgs {
  const ExpertW *Experts;
  const int32_t *SelIdx;  // [slots]
  const float *SelW;      // [slots] (last = shared-expert gate when has_shared)
  const float *Act;       // [slots][I]
  const float *Res;       // [H] residual input
  float *X;               // [H] output residual stream
  float *Moe;             // optional [H]: the MoE output before the residual add
  int32_t slots, I, H;
};
template <int K, int RT>
__device__ __forceinline__ void down_body(const ExpertDownCombineArgs &a) {
  using Gm = RowGeom<K>;
  StagedAct act = stage_act_from_f32(moe_smem, a.Act, K, a.slots, K);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const long tile = (long)warps * Gm::RPW;
  for (long base = (long)blockIdx.x * tile; base < a.H; base += (long)gridDim.x * tile) {
    if (base + (long)warp * Gm::RPW >= a.H) continue;
    long n = base + (long)warp * Gm::RPW + lane / Gm::LPR;
    bool ok = n < a.H;
    LaneRows<RT> rows;
#pragma unroll
    for (int p = 0; p < RT; ++p) {
      rows.ok[p] = ok && p < a.slots;
      const ExpertW &ew = a.Experts[a.SelIdx[p < a.slots ? p : 0]];
      rows.P[p] = ew.dP + (ok ? n : 0) * (K / 2);
      rows.S[p] = ew.dS + (ok ? n : 0) * Gm::G;
    }
    float y[RT];
    warp_rows_dot_paired<K, RT>(rows, act, y);
    if (ok && (lane % Gm::LPR) == 0) {
      float acc = 0.0f;
#pragma unroll
      for (int p = 0; p < RT; ++p)
        if (p < a.slots) acc = acc + a.SelW[p] * y[p];
      if (a.Moe) a.Moe[n] = acc;
      a.X[n] = a.Res[n] + acc;
    }
  }
}
template <int K>
__device__ __forceinline__ void down_dispatch(const ExpertDownCombineArgs &a) {
  if (a.slots <= 6) down_body<K, 6>(a);
  else down_body<K, 12>(a);
}
__global__ void __launch_bounds__(256) ExpertDownCombine(const ExpertDownCombineArgs a) {
  switch (a.I) {
    case 128: down_dispatch<128>(a); break;
    case 256: down_dispatch<256>(a); break;
    case 512: down_dispatch<512>(a); break;
    case 1024: down_dispatch<1024>(a); break;
    default: break;
  }
}
static uint32_t down_smem_fn(const void *args) {
  // sized for the template's pass count (6 or 12): passes beyond the active
  // slots are masked but still index the staged arrays
  const ExpertDownCombineArgs *a = (const ExpertDownCombineArgs *)args;
  return staged_act_bytes(a->I, a->slots <= 6 ? 6 : 12);
}
#define F(f) AINFER_ARG(ExpertDownCombineArgs, f)
AINFER_REGISTER(ExpertDownCombine, ExpertDownCombineArgs, 256, 0, 0, down_smem_fn, F(Experts),
                F(SelIdx), F(SelW), F(Act), F(Res), F(X), F(Moe), F(slots), F(I), F(H));
#undef F

}  // namespace ainfer
