// The three weight-streaming stages of a decode layer on top of block_dot():
// multi-matrix GEMV with per-matrix epilogues, expert gate/up with SiLU-mul,
// expert down with the rank-ordered combine and residual. Rows are dealt to
// blocks in contiguous ranges (blk of nblk), so each block reads one contiguous
// span per matrix. Shared by the stand-alone kernels and the persistent step.
#pragma once
#include "block_dot.cuh"
#include "gemv_stage.cuh"
#include "moe_core.cuh"

namespace ainfer {


// Shared-memory working set of a block plus the thread's view of which of the
// two segment lists is current. `primed` says lists[cur] has already been built
// (and possibly prefetched into the ring) for the stage about to run.
struct BlockScratch {
  Ring *ring;      // shared
  SegList *lists;  // [2] shared
  float *T;        // [kTFloats] shared
  ExpertW *sew;    // [kMaxSegs] shared: weight pointers of the active expert slots (null if unused)
  int cur;
  bool primed;
};

// Copies the weight-pointer records of `slots` selected experts into shared
// memory, all at once (the list builders would otherwise chase them one by one
// through L2). Every thread calls; the caller synchronises before the use.
__device__ __forceinline__ void fetch_expert_rows(ExpertW *sew, const ExpertW *experts, const int32_t *sel,
                                                  int slots) {
  static_assert(sizeof(ExpertW) == 48, "ExpertW is three 16-byte words");
  const int t = threadIdx.x;
  if (t < slots * 3 && t < kMaxSegs * 3) {
    const uint4 *src = reinterpret_cast<const uint4 *>(experts + sel[t / 3]) + t % 3;
    reinterpret_cast<uint4 *>(sew + t / 3)[t % 3] = __ldg(src);
  }
}

// Rows [lo, hi) of `total` dealt to block blk of nblk, in multiples of 4 rows.
__device__ __forceinline__ void block_range(long total, int blk, int nblk, long &lo, long &hi) {
  const int per = (((int)total + nblk - 1) / nblk + 3) / 4 * 4;  // row counts fit 32 bits
  lo = (long)blk * per;
  hi = lo + per < total ? lo + per : total;
  if (lo > total) lo = total;
}

// One switch over the contraction widths, shared by every stage: the only
// K-specific code is block_dot itself.
template <bool kRegCursor>
__device__ __forceinline__ void block_dot_any(int K, Ring *ring, const SegList *cur, const SegList *next,
                                              const StagedAct4 &act, float *T) {
  switch (K) {
    case 128: block_dot<128, kRegCursor>(ring, cur, next, act, T); break;
    case 256: block_dot<256, kRegCursor>(ring, cur, next, act, T); break;
    case 512: block_dot<512, kRegCursor>(ring, cur, next, act, T); break;
    case 1024: block_dot<1024, kRegCursor>(ring, cur, next, act, T); break;
    case 2048: block_dot<2048, kRegCursor>(ring, cur, next, act, T); break;
    case 4096: block_dot<4096, kRegCursor>(ring, cur, next, act, T); break;
    case 8192: block_dot<8192, kRegCursor>(ring, cur, next, act, T); break;
    default: break;  // rejected on the host before launch
  }
}
// Sum of one row's group terms in ascending group order (G = K/128 at run time).
__device__ __forceinline__ float row_sum_rt(const float *T, int trow, int G) {
  const int TS = kTCap / G + 1;
  const float *t = T + trow;
  float acc = 0.0f;
#pragma unroll 4
  for (int g = 0; g < G; ++g) acc = acc + t[(size_t)g * TS];
  return acc;
}

// ---- GEMV over a table of matrices (global rows concatenated), M = 1 ----
__host__ __device__ constexpr int gemv_sub_rows(int K) { return kTCap / (K / 128) < 256 ? kTCap / (K / 128) : 256; }

// Segment list of global rows [sb, se). One thread.
__device__ __forceinline__ void gemv_list(SegList *l, const GemvMat *smats, int nmats, int K, int sb, int se) {
  const int G = K / 128;
  int n = 0;
  for (int i = 0; i < nmats; ++i) {
    int a = sb > smats[i].row_start ? sb : smats[i].row_start;
    int b = se < smats[i].row_start + smats[i].N ? se : smats[i].row_start + smats[i].N;
    if (a < b && n < kMaxSegs) {
      RowSeg &s = l->seg[n++];
      s.P = smats[i].P + (size_t)(a - smats[i].row_start) * (K / 2);
      s.S = smats[i].S + (size_t)(a - smats[i].row_start) * G;
      s.nrows = b - a;
      s.vec = 0;
      s.trow = a - sb;
    }
  }
  l->nseg = n;
  l->K = K;
  seglist_finalize(l);
}
// First list of a block's share, for prefetching ahead of the stage. One thread.
__device__ __forceinline__ void gemv_first_list(SegList *l, const GemvMat *smats, int nmats, int K,
                                                long total_rows, int blk, int nblk) {
  long lo, hi;
  block_range(total_rows, blk, nblk, lo, hi);
  const long se = lo + gemv_sub_rows(K) < hi ? lo + gemv_sub_rows(K) : hi;
  gemv_list(l, smats, nmats, K, (int)lo, (int)se);
}

template <bool kRegCursor>
__device__ __forceinline__ void gemv_block(int K, const GemvMat *smats, int nmats, long total_rows,
                                           const StagedAct4 &act, BlockScratch &bs, int blk, int nblk) {
  const int SB = gemv_sub_rows(K);  // rows per sub-block (one finishing thread per row)
  const int G = K / 128;
  long lo, hi;
  block_range(total_rows, blk, nblk, lo, hi);
  if (!bs.primed) {
    __syncthreads();  // the lists are no longer read by an earlier stage
    if (threadIdx.x == 0) gemv_list(&bs.lists[bs.cur], smats, nmats, K, (int)lo, (int)(lo + SB < hi ? lo + SB : hi));
  }
  bs.primed = false;
#pragma unroll 1
  for (long sb = lo; sb < hi; sb += SB) {
    const long se = sb + SB < hi ? sb + SB : hi;
    const bool more = se < hi;
    if (threadIdx.x == 0 && more)
      gemv_list(&bs.lists[bs.cur ^ 1], smats, nmats, K, (int)se, (int)(se + SB < hi ? se + SB : hi));
    __syncthreads();  // lists built; T of the previous sub-block is no longer read
    AINFER_STAMP(11);
    block_dot_any<kRegCursor>(K, bs.ring, &bs.lists[bs.cur], more ? &bs.lists[bs.cur ^ 1] : nullptr, act, bs.T);
    AINFER_STAMP(12);
    // one thread per row: ordered sum, then the matrix's epilogue
    const long r = sb + threadIdx.x;
    if (r < se) {
      int mi = 0;
      for (int i = 1; i < nmats; ++i)
        if (r >= smats[i].row_start) mi = i;
      gemv_epilogue(smats + mi, (int)(r - smats[mi].row_start), 0, row_sum_rt(bs.T, threadIdx.x, G));
    }
    AINFER_STAMP(13);
    bs.cur ^= 1;
  }
}

// ---- expert gate/up + SiLU-mul: "pair rows" (slot, n), n in [0, I) ----
__host__ __device__ constexpr int gateup_sub_rows(int K) {
  return kTCap / (2 * (K / 128)) < 256 ? kTCap / (2 * (K / 128)) : 256;
}
// Gate and up segments of pair rows [sb, se). One thread.
static __device__ __noinline__ void gateup_list(SegList *l, const ExpertGateUpArgs &a, const ExpertW *sew, int sb,
                                                int se) {
  const int K = a.H, G = K / 128, SB = gateup_sub_rows(K);
  int n = 0;
  if (sb < se)
    for (int s = sb / a.I; s <= (se - 1) / a.I && n + 2 <= kMaxSegs; ++s) {
      int aa = sb > s * a.I ? sb : s * a.I;
      int bb = se < (s + 1) * a.I ? se : (s + 1) * a.I;
      const ExpertW &ew = sew[s];
      size_t r0 = (size_t)(aa - s * a.I);
      RowSeg &g = l->seg[n++];
      g.P = ew.gP + r0 * (K / 2); g.S = ew.gS + r0 * G; g.nrows = bb - aa; g.vec = 0;
      g.trow = aa - sb;
      RowSeg &u = l->seg[n++];
      u.P = ew.uP + r0 * (K / 2); u.S = ew.uS + r0 * G; u.nrows = bb - aa; u.vec = 0;
      u.trow = SB + (aa - sb);
    }
  l->nseg = n;
  l->K = K;
  seglist_finalize(l);
}

template <bool kRegCursor>
__device__ __forceinline__ void gateup_block_dispatch(const ExpertGateUpArgs &a, const StagedAct4 &act,
                                                      BlockScratch &bs, int blk, int nblk) {
  const int K = a.H, G = K / 128;
  const int SB = gateup_sub_rows(K);  // pair rows per sub-block
  long lo, hi;
  block_range((long)a.slots * a.I, blk, nblk, lo, hi);
  if (!bs.primed) {
    __syncthreads();
    if (threadIdx.x == 0) gateup_list(&bs.lists[bs.cur], a, bs.sew, (int)lo, (int)(lo + SB < hi ? lo + SB : hi));
  }
  bs.primed = false;
#pragma unroll 1
  for (long sb = lo; sb < hi; sb += SB) {
    const long se = sb + SB < hi ? sb + SB : hi;
    const bool more = se < hi;
    if (threadIdx.x == 0 && more)
      gateup_list(&bs.lists[bs.cur ^ 1], a, bs.sew, (int)se, (int)(se + SB < hi ? se + SB : hi));
    __syncthreads();
    AINFER_STAMP(21);
    block_dot_any<kRegCursor>(K, bs.ring, &bs.lists[bs.cur], more ? &bs.lists[bs.cur ^ 1] : nullptr, act, bs.T);
    AINFER_STAMP(22);
    const long r = sb + threadIdx.x;
    if (r < se) {
      float g = row_sum_rt(bs.T, threadIdx.x, G), u = row_sum_rt(bs.T, SB + threadIdx.x, G);
      a.Act[(size_t)a.slot_begin * a.I + r] = silu_mul(g, u);
    }
    bs.cur ^= 1;
  }
}

// ---- expert down + combine + residual: output rows n in [0, H), all slots ----
__device__ __forceinline__ int down_sub_rows(int K, int slots) {
  const int per = kTCap / ((K / 128) * (slots > 0 ? slots : 1));
  return per < 256 ? per : 256;
}
// One segment per slot over output rows [sb, se). One thread.
static __device__ __noinline__ void down_list(SegList *l, const ExpertDownCombineArgs &a, const ExpertW *sew, int sb,
                                              int se) {
  const int K = a.I, G = K / 128, nr = se - sb;
  int n = 0;
  if (nr > 0)
    for (int s = 0; s < a.slots && n < kMaxSegs; ++s) {
      const ExpertW &ew = sew[s];
      RowSeg &d = l->seg[n++];
      d.P = ew.dP + (size_t)sb * (K / 2); d.S = ew.dS + (size_t)sb * G; d.nrows = nr; d.vec = s; d.trow = s * nr;
    }
  l->nseg = n;
  l->K = K;
  seglist_finalize(l);
}

template <bool kRegCursor>
__device__ __forceinline__ void down_block_dispatch(const ExpertDownCombineArgs &a, const StagedAct4 &act,
                                                    BlockScratch &bs, int blk, int nblk) {
  const int K = a.I, G = K / 128;
  long lo, hi;
  block_range(a.H, blk, nblk, lo, hi);
  const int SB = down_sub_rows(K, a.slots);
  if (!bs.primed) {
    __syncthreads();
    if (threadIdx.x == 0) down_list(&bs.lists[bs.cur], a, bs.sew, (int)lo, (int)(lo + SB < hi ? lo + SB : hi));
  }
  bs.primed = false;
#pragma unroll 1
  for (long sb = lo; sb < hi; sb += SB) {
    const long se = sb + SB < hi ? sb + SB : hi;
    const int nr = (int)(se - sb);
    const bool more = se < hi;
    if (threadIdx.x == 0 && more)
      down_list(&bs.lists[bs.cur ^ 1], a, bs.sew, (int)se, (int)(se + SB < hi ? se + SB : hi));
    __syncthreads();
    AINFER_STAMP(31);
    block_dot_any<kRegCursor>(K, bs.ring, &bs.lists[bs.cur], more ? &bs.lists[bs.cur ^ 1] : nullptr, act, bs.T);
    AINFER_STAMP(32);
    const long n = sb + threadIdx.x;
    if (n < se) {
      float acc = 0.0f;
      for (int s = 0; s < a.slots; ++s) acc = acc + a.SelW[s] * row_sum_rt(bs.T, s * nr + threadIdx.x, G);
      if (a.Moe) a.Moe[n] = acc;
      a.X[n] = __ldcg(a.Res + n) + acc;
    }
    bs.cur ^= 1;
  }
}

// ---- the same three drivers with K fixed at compile time (stand-alone streaming kernels) ----
template <int K>
__device__ __forceinline__ void gemv_block_t(const GemvMat *smats, int nmats, long total_rows,
                                           const StagedAct4 &act, BlockScratch &bs, int blk, int nblk, int m) {
  constexpr int SB = gemv_sub_rows(K);  // rows per sub-block (one finishing thread per row)
  long lo, hi;
  block_range(total_rows, blk, nblk, lo, hi);
  if (!bs.primed) {
    __syncthreads();  // the lists are no longer read by an earlier stage
    if (threadIdx.x == 0) gemv_list(&bs.lists[bs.cur], smats, nmats, K, (int)lo, (int)( lo + SB < hi ? lo + SB : hi));
  }
  bs.primed = false;
#pragma unroll 1
  for (long sb = lo; sb < hi; sb += SB) {
    const long se = sb + SB < hi ? sb + SB : hi;
    const bool more = se < hi;
    if (threadIdx.x == 0 && more) gemv_list(&bs.lists[bs.cur ^ 1], smats, nmats, K, (int)se, (int)( se + SB < hi ? se + SB : hi));
    // one thread per row: its epilogue's operands are fetched now, under the dot
    const long r = sb + threadIdx.x;
    int mi = 0;
    EpiOperands eo;
    if (r < se) {
      for (int i = 1; i < nmats; ++i)
        if (r >= smats[i].row_start) mi = i;
      gemv_epilogue_fetch(smats + mi, (int)(r - smats[mi].row_start), m, eo);
    }
    __syncthreads();  // lists built; T of the previous sub-block is no longer read
    block_dot<K, true>(bs.ring, &bs.lists[bs.cur], more ? &bs.lists[bs.cur ^ 1] : nullptr, act, bs.T);
    // ordered sum, then the matrix's epilogue
    if (r < se) gemv_epilogue_with(smats + mi, (int)(r - smats[mi].row_start), m, row_sum<K>(bs.T, threadIdx.x), eo);
    bs.cur ^= 1;
  }
}

template <int K>
__device__ __forceinline__ void gateup_block_t(const ExpertGateUpArgs &a, const StagedAct4 &act,
                                             BlockScratch &bs, int blk, int nblk) {
  constexpr int SB = gateup_sub_rows(K);  // pair rows per sub-block
  long lo, hi;
  block_range((long)a.slots * a.I, blk, nblk, lo, hi);
  if (!bs.primed) {
    __syncthreads();
    if (threadIdx.x == 0) gateup_list(&bs.lists[bs.cur], a, bs.sew, (int)lo, (int)( lo + SB < hi ? lo + SB : hi));
  }
  bs.primed = false;
#pragma unroll 1
  for (long sb = lo; sb < hi; sb += SB) {
    const long se = sb + SB < hi ? sb + SB : hi;
    const bool more = se < hi;
    if (threadIdx.x == 0 && more) gateup_list(&bs.lists[bs.cur ^ 1], a, bs.sew, (int)se, (int)( se + SB < hi ? se + SB : hi));
    __syncthreads();
    block_dot<K, true>(bs.ring, &bs.lists[bs.cur], more ? &bs.lists[bs.cur ^ 1] : nullptr, act, bs.T);
    const long r = sb + threadIdx.x;
    if (r < se) {
      float g = row_sum<K>(bs.T, threadIdx.x), u = row_sum<K>(bs.T, SB + threadIdx.x);
      a.Act[(size_t)a.slot_begin * a.I + r] = silu_mul(g, u);
    }
    bs.cur ^= 1;
  }
}
template <int K>
__device__ __forceinline__ void down_block_t(const ExpertDownCombineArgs &a, const StagedAct4 &act,
                                           BlockScratch &bs, int blk, int nblk) {
  long lo, hi;
  block_range(a.H, blk, nblk, lo, hi);
  const int SB = down_sub_rows(K, a.slots);
  if (!bs.primed) {
    __syncthreads();
    if (threadIdx.x == 0) down_list(&bs.lists[bs.cur], a, bs.sew, (int)lo, (int)( lo + SB < hi ? lo + SB : hi));
  }
  bs.primed = false;
#pragma unroll 1
  for (long sb = lo; sb < hi; sb += SB) {
    const long se = sb + SB < hi ? sb + SB : hi;
    const int nr = (int)(se - sb);
    const bool more = se < hi;
    if (threadIdx.x == 0 && more) down_list(&bs.lists[bs.cur ^ 1], a, bs.sew, (int)se, (int)( se + SB < hi ? se + SB : hi));
    __syncthreads();
    block_dot<K, true>(bs.ring, &bs.lists[bs.cur], more ? &bs.lists[bs.cur ^ 1] : nullptr, act, bs.T);
    const long n = sb + threadIdx.x;
    if (n < se) {
      float acc = 0.0f;
      for (int s = 0; s < a.slots; ++s) acc = acc + a.SelW[s] * row_sum<K>(bs.T, s * nr + threadIdx.x);
      if (a.Moe) a.Moe[n] = acc;
      a.X[n] = __ldcg(a.Res + n) + acc;
    }
    bs.cur ^= 1;
  }
}

__device__ __forceinline__ void gemv_block_dispatch(int K, const GemvMat *smats, int nmats, long total_rows,
                                                    const StagedAct4 &act, BlockScratch &bs, int blk,
                                                    int nblk, int m = 0) {
  switch (K) {
    case 128: gemv_block_t<128>(smats, nmats, total_rows, act, bs, blk, nblk, m); break;
    case 256: gemv_block_t<256>(smats, nmats, total_rows, act, bs, blk, nblk, m); break;
    case 512: gemv_block_t<512>(smats, nmats, total_rows, act, bs, blk, nblk, m); break;
    case 1024: gemv_block_t<1024>(smats, nmats, total_rows, act, bs, blk, nblk, m); break;
    case 2048: gemv_block_t<2048>(smats, nmats, total_rows, act, bs, blk, nblk, m); break;
    case 4096: gemv_block_t<4096>(smats, nmats, total_rows, act, bs, blk, nblk, m); break;
    case 8192: gemv_block_t<8192>(smats, nmats, total_rows, act, bs, blk, nblk, m); break;
    default: break;  // rejected on the host before launch
  }
}
__device__ __forceinline__ void gateup_block_dispatch_t(const ExpertGateUpArgs &a, const StagedAct4 &act,
                                                        BlockScratch &bs, int blk, int nblk) {
  switch (a.H) {
    case 256: gateup_block_t<256>(a, act, bs, blk, nblk); break;
    case 512: gateup_block_t<512>(a, act, bs, blk, nblk); break;
    case 1024: gateup_block_t<1024>(a, act, bs, blk, nblk); break;
    case 2048: gateup_block_t<2048>(a, act, bs, blk, nblk); break;
    case 4096: gateup_block_t<4096>(a, act, bs, blk, nblk); break;
    default: break;
  }
}
__device__ __forceinline__ void down_block_dispatch_t(const ExpertDownCombineArgs &a, const StagedAct4 &act,
                                                      BlockScratch &bs, int blk, int nblk) {
  switch (a.I) {
    case 128: down_block_t<128>(a, act, bs, blk, nblk); break;
    case 256: down_block_t<256>(a, act, bs, blk, nblk); break;
    case 512: down_block_t<512>(a, act, bs, blk, nblk); break;
    case 1024: down_block_t<1024>(a, act, bs, blk, nblk); break;
    default: break;
  }
}

}  // namespace ainfer
