// Mixture-of-experts block of the decode loop: RouterTopK, ExpertGateUp,
// ExpertDownCombine. The reference's MLP is dense (gate/up GEMV, SiluMul,
// quantise, down GEMV, ResAddF: tools/decode/decode_l0.cpp:666-674); each
// expert here is that same MLP, the routing around it has no reference
// counterpart and follows the arithmetic stated with each kernel.
#pragma once
#include "../common/router_static.h"
#include "../common/tables.h"
#include "common.cuh"

namespace ainfer {

// (g / (1 + exp(-g))) * u, the reference's SiluMul (tools/cmdlist/kernels.cpp:29-37).
static __device__ __noinline__ float silu_mul(float g, float u) { return (g / (1.0f + det_expf(-g))) * u; }

// ----------------------------------------------------------- RouterTopK ---
// logits[e] = sum_k bf16(Wr[e][k]) * hn[k]: 32 lanes, lane l takes k =
// (i*32+l)*8+j, fma chain in (i, j) order, then the lane tree. The last block
// to finish runs softmax over all experts (max-subtracted, sum over 32 strided
// lanes + tree), top-k by (probability desc, index asc), renormalises the k
// weights in rank order, and evaluates the shared-expert gate sigmoid.
// Scratch of the allocation-free router entry point: logits of up to 1024
// experts plus the shared-expert gate, and a block counter.
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
  // Optional (null: skipped): the layer's expert table [E+1] and a buffer of k+1 records. The
  // selecting block copies the selected experts' pointer records there in slot order (the expert
  // kernels then read them with one load instead of chasing SelIdx through the table) and
  // touches the first line of each selected matrix, so that the address translations of pages
  // this token has not used yet are under way before the expert kernels ask for them.
  const ExpertW *Experts;
  ExpertW *SelRows;
};
__device__ __forceinline__ void prefetch_l2(const void *p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
// Every thread of the selecting block calls, after router_select() returned.
__device__ __forceinline__ void router_publish_rows(const RouterTopKArgs &a) {
  if (!a.Experts || !a.SelRows) return;
  const int t = threadIdx.x;
  if (t < (a.k + 1) * 3) {
    const int idx = __ldcg(a.SelIdx + t / 3);
    const uint4 rec = __ldg(reinterpret_cast<const uint4 *>(a.Experts + idx) + t % 3);  // two pointers
    reinterpret_cast<uint4 *>(a.SelRows + t / 3)[t % 3] = rec;
    prefetch_l2(reinterpret_cast<const void *>(((unsigned long long)rec.y << 32) | rec.x));
    prefetch_l2(reinterpret_cast<const void *>(((unsigned long long)rec.w << 32) | rec.z));
  }
}
// Router logits: one warp per row (experts, then the shared-expert gate row). A lane's share of
// a row is fetched eight 16-byte loads at a time so that the loads of a chunk are all in flight
// together; the sums keep the order stated above. prefetch_router_row/consume split the first
// chunk of a warp's first row so that a caller can issue its weight loads before it waits for
// the producer of Hn.
constexpr int kRouterChunk = 8;  // 16-byte loads in flight per lane
struct RouterRowRegs { uint4 w[kRouterChunk]; };

__device__ __forceinline__ const uint16_t *router_row_ptr(const RouterTopKArgs &a, int e) {
  return e < a.E ? a.Wr + (size_t)e * a.H : a.Wsg;
}
// The loads are unconditional (past the row's end the last piece is fetched again and not used):
// a load under a condition into a register that stays live was measured to be waited for where
// it is issued, which serialises the chunk's round trips.
__device__ __forceinline__ void router_row_load(RouterRowRegs &r, const uint16_t *w, int i0, int n, int lane) {
#pragma unroll
  for (int c = 0; c < kRouterChunk; ++c) {
    const int ic = i0 + c < n ? i0 + c : n - 1;
    r.w[c] = __ldg(reinterpret_cast<const uint4 *>(w + (ic * 32 + lane) * 8));
  }
}
__device__ __forceinline__ float router_row_fma(const RouterRowRegs &r, const float *Hn, int i0, int n, int lane,
                                                float acc) {
  float4 x0[kRouterChunk], x1[kRouterChunk];
#pragma unroll
  for (int c = 0; c < kRouterChunk; ++c) {
    const int ic = i0 + c < n ? i0 + c : n - 1;
    const int k0 = (ic * 32 + lane) * 8;
    x0[c] = __ldcg(reinterpret_cast<const float4 *>(Hn + k0));
    x1[c] = __ldcg(reinterpret_cast<const float4 *>(Hn + k0 + 4));
  }
#pragma unroll
  for (int c = 0; c < kRouterChunk; ++c)
    if (i0 + c < n) {
      const uint4 wv = r.w[c];
      acc = fmaf(u2f(wv.x << 16), x0[c].x, acc);
      acc = fmaf(u2f(wv.x & 0xFFFF0000u), x0[c].y, acc);
      acc = fmaf(u2f(wv.y << 16), x0[c].z, acc);
      acc = fmaf(u2f(wv.y & 0xFFFF0000u), x0[c].w, acc);
      acc = fmaf(u2f(wv.z << 16), x1[c].x, acc);
      acc = fmaf(u2f(wv.z & 0xFFFF0000u), x1[c].y, acc);
      acc = fmaf(u2f(wv.w << 16), x1[c].z, acc);
      acc = fmaf(u2f(wv.w & 0xFFFF0000u), x1[c].w, acc);
    }
  return acc;
}
// first: the chunk already loaded for row (blk*8 + warp), valid when that row exists
__device__ __forceinline__ void router_logits_rows(const RouterTopKArgs &a, int blk, int nblk,
                                                   RouterRowRegs *first = nullptr) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = a.E + (a.Wsg ? 1 : 0);
  const int n = a.H / 256;
  for (int e = blk * 8 + warp; e < rows; e += nblk * 8) {
    const uint16_t *w = router_row_ptr(a, e);
    float acc = 0.0f;
    for (int i0 = 0; i0 < n; i0 += kRouterChunk) {
      RouterRowRegs r;
      if (first && i0 == 0 && e == blk * 8 + warp) r = *first;
      else router_row_load(r, w, i0, n, lane);
      acc = router_row_fma(r, a.Hn, i0, n, lane, acc);
    }
    acc = warp_tree_sum(acc);
    if (lane == 0) a.Logits[e] = acc;
  }
}

// Top-k of the block's probabilities sp[0..E) in two levels. Probabilities are >= 0, so their
// bit patterns order like unsigned integers; key = bits + 1 keeps 0 free for "no candidate".
// Level 1: each of eight warps takes an eighth of the experts (four per lane) and extracts its
// own best k+1 in (value desc, index asc) order: every expert of the global top k+1 is among
// them. Level 2: warp 0 extracts the global order from those 8 (k+1) candidates by the same
// rule. One extraction = the lane's best key and the lowest index holding it, then the warp
// maximum and, among its holders, the lowest index by two hardware warp reductions. The
// result is that of a comparison tournament over all E; only the work per step is small.
constexpr int kTopkWarps = 8, kTopkMaxSel = 33;  // k <= 32
template <int kPerLane>
__device__ __forceinline__ void topk_extract(unsigned (&key)[kPerLane], const unsigned (&idx)[kPerLane],
                                             unsigned &wv, unsigned &wi) {
  unsigned m = key[0];
#pragma unroll
  for (int i = 1; i < kPerLane; ++i) m = key[i] > m ? key[i] : m;
  unsigned bi = 0x7FFFFFFFu;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i)
    if (key[i] == m && m != 0u && idx[i] < bi) bi = idx[i];
  wv = __reduce_max_sync(kFull, m);
  wi = __reduce_min_sync(kFull, m == wv ? bi : 0x7FFFFFFFu);
#pragma unroll
  for (int i = 0; i < kPerLane; ++i)
    if (key[i] == wv && idx[i] == wi) key[i] = 0u;  // never extracted again
}
template <int kPerLane2>
__device__ __forceinline__ void topk_level2(const unsigned *ck, const unsigned *ci, int ncand, float *sp, int E,
                                            int k, bool has_shared, int32_t *sel_idx, float *sel_w,
                                            float *near_gap) {
  const int lane = threadIdx.x & 31;
  unsigned key[kPerLane2], idx[kPerLane2];
#pragma unroll
  for (int i = 0; i < kPerLane2; ++i) {
    const int c = lane + 32 * i;
    key[i] = c < ncand ? ck[c] : 0u;
    idx[i] = c < ncand ? ci[c] : 0x7FFFFFFFu;
  }
  float s = 0.0f, lastp = 0.0f;
  float wsel = 0.0f;  // lane j keeps the weight of rank j (k <= 32)
#pragma unroll 1
  for (int j = 0; j <= k && j < E; ++j) {
    unsigned wv, wi;
    topk_extract<kPerLane2>(key, idx, wv, wi);
    const float p = __uint_as_float(wv - 1u);
    if (j == k) {
      if (lane == 0) *near_gap = lastp > 0.0f ? (lastp - p) / lastp : 0.0f;
      break;
    }
    if (lane == 0) {
      sp[wi] = -1.0f;  // a selected entry is marked in the probability array
      sel_idx[j] = (int32_t)wi;
    }
    if (lane == j) wsel = p;
    s = s + p;
    lastp = p;
  }
  if (k >= E && lane == 0) *near_gap = 1.0f;
  if (lane < k) sel_w[lane] = wsel / s;
  if (lane == 0) {
    sel_idx[k] = E;
    sel_w[k] = has_shared ? 1.0f / (1.0f + det_expf(-sp[E])) : 0.0f;
  }
}
// Every thread of a block of at least 256 threads calls (one __syncthreads inside); E <= 1024.
__device__ __forceinline__ void router_topk_block(float *sp, int E, int k, bool has_shared, int32_t *sel_idx,
                                                  float *sel_w, float *near_gap) {
  __shared__ unsigned ck[kTopkWarps * kTopkMaxSel], ci[kTopkWarps * kTopkMaxSel];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nsel = k + 1 < kTopkMaxSel ? k + 1 : kTopkMaxSel;
  if (warp < kTopkWarps) {
    const int per = (E + kTopkWarps - 1) / kTopkWarps;  // experts of this warp: [warp*per, +per)
    unsigned key[4], idx[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int o = lane + 32 * i, e = warp * per + o;
      const bool ok = o < per && e < E;
      key[i] = ok ? __float_as_uint(sp[e]) + 1u : 0u;
      idx[i] = ok ? (unsigned)e : 0x7FFFFFFFu;
    }
#pragma unroll 1
    for (int j = 0; j < nsel; ++j) {
      unsigned wv, wi;
      topk_extract<4>(key, idx, wv, wi);
      if (lane == 0) {
        ck[warp * nsel + j] = wv;
        ci[warp * nsel + j] = wi;
      }
    }
  }
  __syncthreads();
  if (warp == 0) {
    const int ncand = kTopkWarps * nsel;
    if (ncand <= 128) topk_level2<4>(ck, ci, ncand, sp, E, k, has_shared, sel_idx, sel_w, near_gap);
    else topk_level2<9>(ck, ci, ncand, sp, E, k, has_shared, sel_idx, sel_w, near_gap);
  }
}

// Selection by a whole block (every thread calls; contains __syncthreads):
// softmax over E logits, top-k by (probability desc, index asc), renormalised
// weights, shared-expert gate. sp is E+1 floats of shared-memory scratch
// (probabilities; a selected entry is overwritten by -1). The logits are fetched
// by all threads at once (one round trip to L2) and exponentials are taken
// element-wise by all threads; the sums keep the one-warp partition (lane l
// adds entries l, l+32, ... in ascending order, then an xor butterfly), so the
// result does not depend on how many threads help. Outputs may live in shared
// or global memory; they are complete after the function returns (block-wide).
static __device__ __noinline__ void router_select(const float *lg, int E, int k, bool has_shared, float *sp,
                                           int32_t *sel_idx, float *sel_w, float *near_gap) {
  __shared__ float s_m, s_sum;
  const int tid = threadIdx.x, lane = tid & 31, nthr = blockDim.x;
#pragma unroll 1
  for (int e = tid; e <= E; e += nthr)
    if (e < E || has_shared) sp[e] = __ldcg(lg + e);
  __syncthreads();
  if (tid < 32) {
    float m = -INFINITY;
#pragma unroll 4
    for (int e = lane; e < E; e += 32) m = fmaxf(m, sp[e]);
    m = warp_max(m);
    if (lane == 0) s_m = m;
  }
  __syncthreads();
  const float m = s_m;
#pragma unroll 1
  for (int e = tid; e < E; e += nthr) sp[e] = det_expf(sp[e] - m);
  __syncthreads();
  if (tid < 32) {
    float sum = 0.0f;
#pragma unroll 4
    for (int e = lane; e < E; e += 32) sum = sum + sp[e];
    sum = warp_tree_sum(sum);
    if (lane == 0) s_sum = sum;
  }
  __syncthreads();
  const float sum = s_sum;
#pragma unroll 1
  for (int e = tid; e < E; e += nthr) sp[e] = sp[e] / sum;
  __syncthreads();
  router_topk_block(sp, E, k, has_shared, sel_idx, sel_w, near_gap);
  __syncthreads();
}

// --------------------------------------------------------- ExpertGateUp ---
// For every active slot s (routed experts in rank order, then the shared
// expert) and every intermediate row n: g = gate_e[n].h, u = up_e[n].h (W4A8
// GEMV), Act[s][n] = (g / (1 + exp(-g))) * u  (SiluMul, kernels.cpp:29-37).
struct ExpertGateUpArgs {
  const ExpertW *Experts;  // [E+1]
  const int32_t *SelIdx;   // [slots]; null: Experts already holds the slots' records in slot order
  const int8_t *XQ;        // [H] quantised hidden
  const float *SQ;         // [H/128]
  float *Act;              // [slots][I]
  int32_t slots, I, H;
  int32_t slot_begin;      // first slot this launch handles (expert-parallel ranks)
  int32_t prefetch_down;   // non-zero: also start these slots' down projections towards L2
};
// ---------------------------------------------------- ExpertDownCombine ---
// Quantises each slot's activation (per-128 quantiser), y_s[n] = down_e[n].act_s,
// then out[n] = Res[n] + (sum_s w_s * y_s[n] in rank order, + sg * y_shared[n]),
// products and sums unfused. (Down GEMV + ResAddF, decode_l0.cpp:672-674.)
struct ExpertDownCombineArgs {
  const ExpertW *Experts;
  const int32_t *SelIdx;  // [slots]; null: Experts already holds the slots' records in slot order
  const float *SelW;      // [slots] (last = shared-expert gate when has_shared)
  const float *Act;       // [slots][I]
  const float *Res;       // [H] residual input
  float *X;               // [H] output residual stream
  float *Moe;             // optional [H]: the MoE output before the residual add
  int32_t slots, I, H;
};
// Output rows of the down projections: for row n every active slot's matrix is
// dotted with that slot's quantised activation (slots in groups of four, so that
// four loads are in flight), then combined in rank order.
}  // namespace ainfer
