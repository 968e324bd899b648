// Kernels of the expert-parallel mixture-of-experts block for a decode batch: batched router,
// the dispatch plan and permute (pack (token, slot) items per destination rank), the grouping of
// received items by expert for the grouped tensor-core GEMM, the SiLU-multiply + activation
// quantiser between the two expert GEMMs, the un-permute back to the senders' order and the
// slot-ordered combine. The reference decodes one token on one device and has no counterpart
// (its MLP is dense: tools/decode/decode_l0.cpp:666-674); the arithmetic of every piece is the
// single-token kernels' (moe_core.cuh), so a token's result does not depend on the batch it is
// in nor on how many ranks share the experts.
//
// Exchange buffers. A dispatch buffer has one slot per peer rank:
//   [16 B header: item count][cap x 16 B records {expert, token, slot, 0}][cap x item bytes payload]
// where the payload of an item is the token's quantised hidden vector (H int8) and its group
// scales (H/128 fp32, padded to 16 bytes), and cap = owned tokens x top-k is the most one rank can send to another.
// A return buffer has one slot of cap x H fp32 per peer: the un-weighted expert outputs, in the
// order the items were sent. Slots are exchanged whole (fixed size), so the host never needs the
// counts.
#define AINFER_BLOCK_DOT_INLINE 1

#include "direct_dot.cuh"

namespace ainfer {

__host__ __device__ inline int ep_item_bytes(int H) { return H + ((H / 128 * 4 + 15) & ~15); }

// ---- batched router: logits of every owned token, then one block per token selects ----
struct RouterLogitsRowsArgs {
  const uint16_t *Wr;    // [E][H] bf16 router
  const uint16_t *Wsg;   // [H] bf16 shared-expert gate row (null: none)
  const float *Hn;       // [rows][H] normalised activations
  const float *Bias;     // optional [E]: added to the routed experts' logits (load generators); null: none
  float *Logits;         // [rows][E+1]
  int32_t E, H, rows;
  int32_t tokens_per_block;   // launched with ceil((E + 1) / 8) x ceil(rows / tokens_per_block) blocks
};
// One warp per router row and block of tokens; per token the sums of RouterTopK (router_row_fma
// order, then the lane tree). The row's first chunk of weights is fetched once, and four tokens
// are summed side by side: a token's sum is one chain of dependent additions per lane, so four
// chains in flight is what keeps the lanes busy.
// kSmem: the block's tokens' activations were staged in shared memory (hn points there, token stride H)
template <bool kSmem>
__device__ __forceinline__ void router_rows_compute(const RouterLogitsRowsArgs &a, const uint16_t *w, const RouterRowRegs &r0,
                                                    const float *hn_base, int t_begin, int t_end, int e, bool store, float bias,
                                                    int lane) {
  const int n = a.H / 256;
  for (int t = t_begin; t < t_end; t += 4) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    RouterRowRegs r = r0;
    const float *hn[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) hn[u] = hn_base + (size_t)((t + u < t_end ? t + u : t_end - 1) - (kSmem ? t_begin : 0)) * a.H;   // past the end: the last token again, not stored
    for (int i0 = 0;;) {
#pragma unroll
      for (int c = 0; c < kRouterChunk; ++c) {
        const int ic = i0 + c < n ? i0 + c : n - 1, k0 = (ic * 32 + lane) * 8;
        float4 x0[4], x1[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (kSmem) {
            x0[u] = *reinterpret_cast<const float4 *>(hn[u] + k0);
            x1[u] = *reinterpret_cast<const float4 *>(hn[u] + k0 + 4);
          } else {
            x0[u] = __ldcg(reinterpret_cast<const float4 *>(hn[u] + k0));
            x1[u] = __ldcg(reinterpret_cast<const float4 *>(hn[u] + k0 + 4));
          }
        }
        if (i0 + c < n) {
          const uint4 wv = r.w[c];
          const float w0 = u2f(wv.x << 16), w1 = u2f(wv.x & 0xFFFF0000u), w2 = u2f(wv.y << 16), w3 = u2f(wv.y & 0xFFFF0000u),
                      w4 = u2f(wv.z << 16), w5 = u2f(wv.z & 0xFFFF0000u), w6 = u2f(wv.w << 16), w7 = u2f(wv.w & 0xFFFF0000u);
#pragma unroll
          for (int u = 0; u < 4; ++u) {   // router_row_fma's order for each token
            float s = acc[u];
            s = fmaf(w0, x0[u].x, s);
            s = fmaf(w1, x0[u].y, s);
            s = fmaf(w2, x0[u].z, s);
            s = fmaf(w3, x0[u].w, s);
            s = fmaf(w4, x1[u].x, s);
            s = fmaf(w5, x1[u].y, s);
            s = fmaf(w6, x1[u].z, s);
            s = fmaf(w7, x1[u].w, s);
            acc[u] = s;
          }
        }
      }
      i0 += kRouterChunk;
      if (i0 >= n) break;
      router_row_load(r, w, i0, n, lane);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float sum = warp_tree_sum(acc[u]);
      if (lane == 0 && store && t + u < t_end) a.Logits[(size_t)(t + u) * (a.E + 1) + e] = a.Bias ? sum + bias : sum;
    }
  }
}
constexpr int kRouterStageFloats = 8192;   // 32 KB: four tokens of 2048
__global__ void __launch_bounds__(256, 2) RouterLogitsRows(const RouterLogitsRowsArgs a) {
  // The block's tokens are read by all eight warps: staged once in shared memory they cross from
  // L2 once per block instead of once per warp (at 64 tokens and 513 rows the per-warp reads were
  // 266 MB a launch, and the launch took as long as that takes).
  __shared__ __align__(16) float hs[kRouterStageFloats];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nrows = a.E + (a.Wsg ? 1 : 0), n = a.H / 256;
  const int nrb = (a.E + 1 + 7) / 8, rb = blockIdx.x % nrb, tb = blockIdx.x / nrb;
  const int t_begin = tb * a.tokens_per_block;
  const int t_end = t_begin + a.tokens_per_block < a.rows ? t_begin + a.tokens_per_block : a.rows;
  const int e_raw = rb * 8 + warp, e = e_raw < nrows ? e_raw : nrows - 1;   // a warp past the last row repeats it and stores nothing
  const uint16_t *w = e < a.E ? a.Wr + (size_t)e * a.H : a.Wsg;
  const float bias = a.Bias && e < a.E ? __ldg(a.Bias + e) : 0.0f;
  RouterRowRegs r0;
  router_row_load(r0, w, 0, n, lane);
  const bool staged = (t_end - t_begin) * a.H <= kRouterStageFloats;   // the same for every thread of the block
  if (staged) {
    const float4 *src = reinterpret_cast<const float4 *>(a.Hn + (size_t)t_begin * a.H);
    const int n4 = (t_end - t_begin) * a.H / 4;
    for (int i = threadIdx.x; i < n4; i += 256) reinterpret_cast<float4 *>(hs)[i] = __ldcg(src + i);
    __syncthreads();
    router_rows_compute<true>(a, w, r0, hs, t_begin, t_end, e, e_raw < nrows, bias, lane);
  } else {
    router_rows_compute<false>(a, w, r0, a.Hn, t_begin, t_end, e, e_raw < nrows, bias, lane);
  }
}
struct RouterSelectRowsArgs {
  const float *Logits;   // [rows][E+1]
  int32_t *SelIdx;       // [rows][k+1]
  float *SelW;           // [rows][k+1]
  float *NearGap;        // [rows]
  int32_t E, k, has_shared;
};
__global__ void __launch_bounds__(256) RouterSelectRows(const RouterSelectRowsArgs a) {
  __shared__ float sp[1024 + 1];
  const int t = blockIdx.x;
  router_select(a.Logits + (size_t)t * (a.E + 1), a.E, a.k, a.has_shared != 0, sp, a.SelIdx + (size_t)t * (a.k + 1),
                a.SelW + (size_t)t * (a.k + 1), a.NearGap + t);
}

// ---- dispatch plan: destination rank and position of every (token, slot) item ----
constexpr int kEpMaxItems = 2048;   // owned tokens x top-k, and items a rank can receive
struct EpItemRec { int32_t expert, token, slot, pad; };
struct EpPlanArgs {
  const int32_t *SelIdx;   // [n][k+1]
  unsigned char *Send;     // dispatch buffer (R slots)
  int32_t *ItemDest;       // [n*k]: dest << 16 | position in the destination's slot
  int32_t n, k, experts_per_rank, world, cap;
  uint32_t slot_bytes;
};
// One block. Item i = token * k + slot goes to the rank that holds its expert; its position there
// is the number of earlier items with the same destination (so slots are filled in item order).
__global__ void __launch_bounds__(1024) EpPlan(const EpPlanArgs a) {
  __shared__ unsigned char dest[kEpMaxItems];
  const int items = a.n * a.k;
  for (int i = threadIdx.x; i < items; i += blockDim.x)
    dest[i] = (unsigned char)(a.SelIdx[(size_t)(i / a.k) * (a.k + 1) + i % a.k] / a.experts_per_rank);
  __syncthreads();
  for (int i = threadIdx.x; i < items; i += blockDim.x) {
    const int d = dest[i];
    int pos = 0;
    for (int j = 0; j < i; ++j) pos += dest[j] == d;
    a.ItemDest[i] = (d << 16) | pos;
    EpItemRec rec{a.SelIdx[(size_t)(i / a.k) * (a.k + 1) + i % a.k], i / a.k, i % a.k, 0};
    *reinterpret_cast<EpItemRec *>(a.Send + (size_t)d * a.slot_bytes + 16 + (size_t)pos * 16) = rec;
  }
  for (int d = threadIdx.x; d < a.world; d += blockDim.x) {
    int c = 0;
    for (int j = 0; j < items; ++j) c += dest[j] == d;
    *reinterpret_cast<int4 *>(a.Send + (size_t)d * a.slot_bytes) = make_int4(c, 0, 0, 0);
  }
}
// ---- permute: one block per item copies the token's quantised vector and scales ----
struct EpPackArgs {
  const int8_t *Q8;        // [n][H]
  const float *SQ;         // [n][H/128]
  const int32_t *ItemDest; // [n*k]
  unsigned char *Send;
  int32_t k, H, cap;
  uint32_t slot_bytes;
};
__global__ void __launch_bounds__(128) EpPack(const EpPackArgs a) {
  const int i = blockIdx.x, t = i / a.k;
  const int dp = a.ItemDest[i], d = dp >> 16, pos = dp & 0xFFFF;
  const int item_bytes = ep_item_bytes(a.H);
  unsigned char *dst = a.Send + (size_t)d * a.slot_bytes + 16 + (size_t)a.cap * 16 + (size_t)pos * item_bytes;
  const uint4 *q = reinterpret_cast<const uint4 *>(a.Q8 + (size_t)t * a.H);
  for (int j = threadIdx.x; j < a.H / 16; j += blockDim.x) reinterpret_cast<uint4 *>(dst)[j] = q[j];
  const float *s = a.SQ + (size_t)t * (a.H / 128);
  for (int j = threadIdx.x; j < a.H / 128; j += blockDim.x) reinterpret_cast<float *>(dst + a.H)[j] = s[j];
}

// ---- grouping of the received items by expert, and the problem lists of the grouped GEMMs ----
struct EpTcGroup {           // = TcGroup of the grouped tensor-core GEMM
  const uint8_t *P;
  const uint16_t *S;
  int32_t x_row0, M, y_col, pad;
};
static_assert(sizeof(EpTcGroup) == 32, "layout of the grouped GEMM's problem record");
struct EpGroupArgs {
  const unsigned char *Recv;  // dispatch buffer received (R slots)
  const ExpertW *Experts;     // the layer's table [E+1]
  int32_t *Sorted;            // [R*cap]: src << 16 | index in the source's slot, grouped by expert
  // Problems are listed by size: up to small_rows rows for the dp4a kernel that streams weights
  // once (Int4GemvA8MultiGrouped), more for the tensor-core kernel (Int4GemmA8TcGrouped).
  EpTcGroup *GroupsGateUp;    // [2 * (experts_per_rank + 1)]: gate and up problem of every active expert with few rows
  EpTcGroup *GroupsDown;      // [experts_per_rank + 1]
  EpTcGroup *GroupsGateUpL;   // the same for experts with many rows
  EpTcGroup *GroupsDownL;
  int32_t *Counts;            // [8]: items in total, gate/up and down problems (few rows), gate/up and down problems (many rows)
  int32_t world, rank, experts_per_rank, cap, I;
  uint32_t slot_bytes;
  // The shared expert of this rank's own rows rides in the same launches as one more problem:
  // its activations are rows [shared_row0, shared_row0 + shared_rows) of the grouped layout
  // (the owner's quantiser writes them there). shared_rows == 0: none.
  int32_t shared_row0, shared_rows, shared_expert;
  int32_t small_rows;   // problems up to this many rows go to the first pair of lists (a large value: all of them)
  int32_t max_rows;     // an expert with more rows is cut into problems of at most this many (same weights, consecutive rows)
};
// One block. Items are numbered (source rank, index) in ascending order; an item's row in the
// grouped layout is the start of its expert's range plus the number of earlier items of the same
// expert. Experts with no item produce no problem.
__global__ void __launch_bounds__(1024) EpGroup(const EpGroupArgs a) {
  __shared__ short le[kEpMaxItems];          // local expert of every received item
  __shared__ int base[65];                   // first item number of every source
  __shared__ int hist[1024], start[1024], active[1024];   // active: index in its list, many-row experts offset by 1 << 20
  const int tid = threadIdx.x;
  if (tid == 0) {
    int s = 0;
    for (int r = 0; r < a.world; ++r) {
      base[r] = s;
      s += *reinterpret_cast<const int *>(a.Recv + (size_t)r * a.slot_bytes);
    }
    base[a.world] = s;
  }
  for (int e = tid; e < a.experts_per_rank; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int total = base[a.world] < kEpMaxItems ? base[a.world] : kEpMaxItems;
  for (int it = tid; it < total; it += blockDim.x) {
    int r = 0;
    while (it >= base[r + 1]) ++r;
    const EpItemRec rec = *reinterpret_cast<const EpItemRec *>(a.Recv + (size_t)r * a.slot_bytes + 16 + (size_t)(it - base[r]) * 16);
    const int l = rec.expert - a.rank * a.experts_per_rank;
    le[it] = (short)l;
    atomicAdd(&hist[l], 1);
  }
  __syncthreads();
  if (tid < 32) {   // exclusive scans over the experts (counts, and "has items" flags): one warp, chunks of 32
    int run = 0, nact = 0, nactl = 0;
    for (int e0 = 0; e0 < a.experts_per_rank; e0 += 32) {
      const int e = e0 + tid;
      const int c = e < a.experts_per_rank ? hist[e] : 0, f = c > 0 && c <= a.small_rows;
      const int fl = c > a.small_rows ? (c + a.max_rows - 1) / a.max_rows : 0;   // problems in the many-row lists
      int sc = c, sf = f, sl = fl;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int vc = __shfl_up_sync(kFull, sc, off), vf = __shfl_up_sync(kFull, sf, off), vl = __shfl_up_sync(kFull, sl, off);
        if (tid >= off) { sc += vc; sf += vf; sl += vl; }
      }
      if (e < a.experts_per_rank) { start[e] = run + sc - c; active[e] = fl ? (1 << 20) + nactl + sl - fl : nact + sf - f; }
      run += __shfl_sync(kFull, sc, 31);
      nact += __shfl_sync(kFull, sf, 31);
      nactl += __shfl_sync(kFull, sl, 31);
    }
    if (tid == 0) {
      const int sh = a.shared_rows > 0 && a.shared_rows <= a.small_rows ? 1 : 0;
      const int shl = a.shared_rows > a.small_rows ? (a.shared_rows + a.max_rows - 1) / a.max_rows : 0;
      if (sh || shl) {
        const ExpertW w = a.Experts[a.shared_expert];
        const int cut = sh ? a.shared_rows : a.max_rows;
        for (int j = 0; j < sh + shl; ++j) {
          const int r0 = a.shared_row0 + j * cut, mr = min(cut, a.shared_rows - j * cut);
          EpTcGroup *gu = sh ? a.GroupsGateUp + 2 * nact : a.GroupsGateUpL + 2 * (nactl + j), *gd = sh ? a.GroupsDown + nact : a.GroupsDownL + nactl + j;
          gu[0] = EpTcGroup{w.gP, w.gS, r0, mr, 0, 0};
          gu[1] = EpTcGroup{w.uP, w.uS, r0, mr, a.I, 0};
          gd[0] = EpTcGroup{w.dP, w.dS, r0, mr, 0, 0};
        }
      }
      *reinterpret_cast<int4 *>(a.Counts) = make_int4(total, 2 * (nact + sh), nact + sh, 2 * (nactl + shl));
      *reinterpret_cast<int4 *>(a.Counts + 4) = make_int4(nactl + shl, 0, 0, 0);
    }
  }
  __syncthreads();
  for (int e = tid; e < a.experts_per_rank; e += blockDim.x) {
    const int c = hist[e];
    if (c > 0) {
      const ExpertW w = a.Experts[a.rank * a.experts_per_rank + e];
      const bool large = active[e] >= (1 << 20);
      const int g = active[e] & ((1 << 20) - 1);
      const int cut = large ? a.max_rows : c, np = (c + cut - 1) / cut;
      for (int j = 0; j < np; ++j) {
        const int r0 = start[e] + j * cut, mr = min(cut, c - j * cut);
        EpTcGroup *gu = (large ? a.GroupsGateUpL : a.GroupsGateUp) + 2 * (g + j), *gd = (large ? a.GroupsDownL : a.GroupsDown) + g + j;
        gu[0] = EpTcGroup{w.gP, w.gS, r0, mr, 0, 0};
        gu[1] = EpTcGroup{w.uP, w.uS, r0, mr, a.I, 0};
        gd[0] = EpTcGroup{w.dP, w.dS, r0, mr, 0, 0};
      }
    }
  }
  for (int it = tid; it < total; it += blockDim.x) {
    const int l = le[it];
    int pos = start[l];
    for (int j = 0; j < it; ++j) pos += le[j] == l;
    int r = 0;
    while (it >= base[r + 1]) ++r;
    a.Sorted[pos] = (r << 16) | (it - base[r]);
  }
}
// ---- gather the received payloads into the grouped layout ----
struct EpGatherArgs {
  const unsigned char *Recv;
  const int32_t *Sorted;
  const int32_t *Counts;
  int8_t *XQ;     // [R*cap][H]
  float *SQ;      // [R*cap][H/128]
  int32_t H, cap;
  uint32_t slot_bytes;
};
__global__ void __launch_bounds__(128) EpGather(const EpGatherArgs a) {
  const int pos = blockIdx.x;
  if (pos >= __ldg(a.Counts)) return;
  const int si = a.Sorted[pos], r = si >> 16, i = si & 0xFFFF;
  const int item_bytes = ep_item_bytes(a.H);
  const unsigned char *src = a.Recv + (size_t)r * a.slot_bytes + 16 + (size_t)a.cap * 16 + (size_t)i * item_bytes;
  uint4 *q = reinterpret_cast<uint4 *>(a.XQ + (size_t)pos * a.H);
  for (int j = threadIdx.x; j < a.H / 16; j += blockDim.x) q[j] = reinterpret_cast<const uint4 *>(src)[j];
  float *s = a.SQ + (size_t)pos * (a.H / 128);
  for (int j = threadIdx.x; j < a.H / 128; j += blockDim.x) s[j] = reinterpret_cast<const float *>(src + a.H)[j];
}

// ---- between the expert GEMMs: act = silu(gate) * up, then the per-128 activation quantiser ----
// (SiluMul tools/cmdlist/kernels.cpp:29-37, ScalesMax + Quantize :551-579.) One warp per group of
// 128, a lane holds four consecutive elements.
struct SiluQuantRowsArgs {
  const float *GU;         // [rows][2*I]: gate outputs, then up outputs
  const int32_t *Counts;   // optional device word: rows in use among the first always_from (null: every launched row)
  int8_t *AQ;              // [rows][I]
  float *ASQ;              // [rows][I/128]
  int32_t I;
  int32_t always_from;     // rows from this one on are always in use
};
__global__ void __launch_bounds__(128) SiluQuantRows(const SiluQuantRowsArgs a) {
  const int row = blockIdx.x;
  if (a.Counts && row < a.always_from && row >= __ldg(a.Counts)) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float *g = a.GU + (size_t)row * 2 * a.I, *u = g + a.I;
  for (int grp = warp; grp < a.I / 128; grp += 4) {
    const int j = grp * 128 + lane * 4;
    const float4 gv = *reinterpret_cast<const float4 *>(g + j), uv = *reinterpret_cast<const float4 *>(u + j);
    float4 y;
    y.x = silu_mul(gv.x, uv.x);
    y.y = silu_mul(gv.y, uv.y);
    y.z = silu_mul(gv.z, uv.z);
    y.w = silu_mul(gv.w, uv.w);
    float m = fmaxf(fmaxf(fabsf(y.x), fabsf(y.y)), fmaxf(fabsf(y.z), fabsf(y.w)));
    m = warp_max(m);
    float s = m / 127.0f;
    if (s == 0.0f) s = 1.0f;
    if (lane == 0) a.ASQ[(size_t)row * (a.I / 128) + grp] = s;
    const int q0 = quant_round(y.x, s), q1 = quant_round(y.y, s), q2 = quant_round(y.z, s), q3 = quant_round(y.w, s);
    *reinterpret_cast<uint32_t *>(a.AQ + (size_t)row * a.I + j) =
        (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
  }
}

// ---- un-permute: expert outputs back into the senders' slots, in the order they were sent ----
struct EpScatterArgs {
  const float *Y;          // [R*cap][H] down-projection outputs in the grouped layout
  const int32_t *Sorted;
  const int32_t *Counts;
  unsigned char *Ret;      // return buffer (R slots of cap x H fp32)
  int32_t H;
  uint32_t slot_bytes;
};
__global__ void __launch_bounds__(128) EpScatter(const EpScatterArgs a) {
  const int pos = blockIdx.x;
  if (pos >= __ldg(a.Counts)) return;
  const int si = a.Sorted[pos], r = si >> 16, i = si & 0xFFFF;
  const float4 *src = reinterpret_cast<const float4 *>(a.Y + (size_t)pos * a.H);
  float4 *dst = reinterpret_cast<float4 *>(a.Ret + (size_t)r * a.slot_bytes + (size_t)i * a.H * 4);
  for (int j = threadIdx.x; j < a.H / 4; j += blockDim.x) dst[j] = src[j];
}

// ---- combine on the token's owner: the additions of ExpertDownCombine, in slot order ----
// X[t][n] = Res[t][n] + (sum over routed slots j in rank order of W[t][j] * Y_j[n], then
// + W[t][k] * Ysh[t][n]); products and sums unfused.
struct EpCombineArgs {
  const float *Res;         // [n][H]
  const unsigned char *Back;// return buffer received (R slots)
  const int32_t *ItemDest;  // [n*k]
  const float *SelW;        // [n][k+1]
  const float *Ysh;         // [n][H] shared expert's output (null: none)
  float *X;                 // [n][H]
  int32_t k, H;
  uint32_t slot_bytes;
};
// Launched with tokens x ceil(H / 256) blocks.
__global__ void __launch_bounds__(256) EpCombine(const EpCombineArgs a) {
  const int bpr = (a.H + 255) / 256;
  const int t = blockIdx.x / bpr;
  const int n = (blockIdx.x % bpr) * 256 + threadIdx.x;
  if (n >= a.H) return;
  float acc = 0.0f;
  for (int j = 0; j < a.k; ++j) {
    const int dp = a.ItemDest[t * a.k + j];
    const float y = reinterpret_cast<const float *>(a.Back + (size_t)(dp >> 16) * a.slot_bytes)[(size_t)(dp & 0xFFFF) * a.H + n];
    acc = acc + a.SelW[(size_t)t * (a.k + 1) + j] * y;
  }
  if (a.Ysh) acc = acc + a.SelW[(size_t)t * (a.k + 1) + a.k] * a.Ysh[(size_t)t * a.H + n];
  a.X[(size_t)t * a.H + n] = a.Res[(size_t)t * a.H + n] + acc;
}

#define F(f) AINFER_ARG(RouterLogitsRowsArgs, f)
AINFER_REGISTER(RouterLogitsRows, RouterLogitsRowsArgs, 256, 8, 0, nullptr, F(Wr), F(Wsg), F(Hn), F(Bias), F(Logits), F(E), F(H), F(rows),
                F(tokens_per_block));
#undef F
#define F(f) AINFER_ARG(RouterSelectRowsArgs, f)
AINFER_REGISTER(RouterSelectRows, RouterSelectRowsArgs, 256, 1, 0, nullptr, F(Logits), F(SelIdx), F(SelW), F(NearGap), F(E), F(k), F(has_shared));
#undef F
#define F(f) AINFER_ARG(EpPlanArgs, f)
AINFER_REGISTER(EpPlan, EpPlanArgs, 1024, 0, 0, nullptr, F(SelIdx), F(Send), F(ItemDest), F(n), F(k), F(experts_per_rank), F(world), F(cap),
                F(slot_bytes));
#undef F
#define F(f) AINFER_ARG(EpPackArgs, f)
AINFER_REGISTER(EpPack, EpPackArgs, 128, 1, 0, nullptr, F(Q8), F(SQ), F(ItemDest), F(Send), F(k), F(H), F(cap), F(slot_bytes));
#undef F
#define F(f) AINFER_ARG(EpGroupArgs, f)
AINFER_REGISTER(EpGroup, EpGroupArgs, 1024, 0, 0, nullptr, F(Recv), F(Experts), F(Sorted), F(GroupsGateUp), F(GroupsDown), F(GroupsGateUpL), F(GroupsDownL), F(Counts), F(world),
                F(rank), F(experts_per_rank), F(cap), F(I), F(slot_bytes), F(shared_row0), F(shared_rows), F(shared_expert), F(small_rows), F(max_rows));
#undef F
#define F(f) AINFER_ARG(EpGatherArgs, f)
AINFER_REGISTER(EpGather, EpGatherArgs, 128, 1, 0, nullptr, F(Recv), F(Sorted), F(Counts), F(XQ), F(SQ), F(H), F(cap), F(slot_bytes));
#undef F
#define F(f) AINFER_ARG(SiluQuantRowsArgs, f)
AINFER_REGISTER(SiluQuantRows, SiluQuantRowsArgs, 128, 1, 0, nullptr, F(GU), F(Counts), F(AQ), F(ASQ), F(I), F(always_from));
#undef F
#define F(f) AINFER_ARG(EpScatterArgs, f)
AINFER_REGISTER(EpScatter, EpScatterArgs, 128, 1, 0, nullptr, F(Y), F(Sorted), F(Counts), F(Ret), F(H), F(slot_bytes));
#undef F
#define F(f) AINFER_ARG(EpCombineArgs, f)
AINFER_REGISTER(EpCombine, EpCombineArgs, 256, 0, 0, nullptr, F(Res), F(Back), F(ItemDest), F(SelW), F(Ysh), F(X), F(k), F(H), F(slot_bytes));
#undef F

}  // namespace ainfer
