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

constexpr int kTCap = 4096;  // floats of t[][] scratch a block needs (16 KB)

struct BlockScratch {
  RowSeg *segs;   // [kMaxSegs] shared
  float *T;       // [kTCap] shared
  int *ibox;      // [4] shared ints for block-uniform values
};

// Rows [lo, hi) of `total` dealt to block blk of nblk, in multiples of 4 rows.
__device__ __forceinline__ void block_range(long total, int blk, int nblk, long &lo, long &hi) {
  long per = ((total + nblk - 1) / nblk + 3) / 4 * 4;
  lo = (long)blk * per;
  hi = lo + per < total ? lo + per : total;
  if (lo > total) lo = total;
}

// ---- GEMV over a table of matrices (global rows concatenated), M = 1 ----
template <int K>
__device__ __forceinline__ void gemv_block(const GemvMat *smats, int nmats, long total_rows,
                                           const StagedAct4 &act, const BlockScratch &bs, int blk, int nblk) {
  constexpr int G = K / 128;
  constexpr int SB = kTCap / G < 256 ? kTCap / G : 256;  // rows per sub-block (one finishing thread per row)
  long lo, hi;
  block_range(total_rows, blk, nblk, lo, hi);
#pragma unroll 1
  for (long sb = lo; sb < hi; sb += SB) {
    const long se = sb + SB < hi ? sb + SB : hi;
    __syncthreads();  // segs / T of the previous sub-block are no longer read
    if (threadIdx.x == 0) {
      int n = 0;
      for (int i = 0; i < nmats; ++i) {
        long a = sb > smats[i].row_start ? sb : smats[i].row_start;
        long b = se < smats[i].row_start + smats[i].N ? se : smats[i].row_start + smats[i].N;
        if (a < b) {
          RowSeg &s = bs.segs[n++];
          s.P = smats[i].P + (a - smats[i].row_start) * (K / 2);
          s.S = smats[i].S + (a - smats[i].row_start) * G;
          s.nrows = (int)(b - a);
          s.vec = 0;
          s.trow = (int)(a - sb);
        }
      }
      bs.ibox[0] = n;
      bs.ibox[1] = seg_finalize(bs.segs, n);
    }
    __syncthreads();
    block_dot<K>(bs.segs, bs.ibox[0], bs.ibox[1], act, bs.T);
    // one thread per row: ordered sum, then the matrix's epilogue
    const long r = sb + threadIdx.x;
    if (r < se) {
      int mi = 0;
      for (int i = 1; i < nmats; ++i)
        if (r >= smats[i].row_start) mi = i;
      gemv_epilogue(smats + mi, (int)(r - smats[mi].row_start), 0, row_sum<K>(bs.T, threadIdx.x));
    }
  }
}

__device__ __forceinline__ void gemv_block_dispatch(int K, const GemvMat *smats, int nmats, long total_rows,
                                                    const StagedAct4 &act, const BlockScratch &bs, int blk,
                                                    int nblk) {
  switch (K) {
    case 128: gemv_block<128>(smats, nmats, total_rows, act, bs, blk, nblk); break;
    case 256: gemv_block<256>(smats, nmats, total_rows, act, bs, blk, nblk); break;
    case 512: gemv_block<512>(smats, nmats, total_rows, act, bs, blk, nblk); break;
    case 1024: gemv_block<1024>(smats, nmats, total_rows, act, bs, blk, nblk); break;
    case 2048: gemv_block<2048>(smats, nmats, total_rows, act, bs, blk, nblk); break;
    case 4096: gemv_block<4096>(smats, nmats, total_rows, act, bs, blk, nblk); break;
    case 8192: gemv_block<8192>(smats, nmats, total_rows, act, bs, blk, nblk); break;
    default: break;  // rejected on the host before launch
  }
}

// ---- expert gate/up + SiLU-mul: "pair rows" (slot, n), n in [0, I) ----
template <int K>
__device__ __forceinline__ void gateup_block(const ExpertGateUpArgs &a, const StagedAct4 &act,
                                             const BlockScratch &bs, int blk, int nblk) {
  constexpr int G = K / 128;
  constexpr int SB = kTCap / (2 * G) < 256 ? kTCap / (2 * G) : 256;  // pair rows per sub-block
  long lo, hi;
  block_range((long)a.slots * a.I, blk, nblk, lo, hi);
#pragma unroll 1
  for (long sb = lo; sb < hi; sb += SB) {
    const long se = sb + SB < hi ? sb + SB : hi;
    __syncthreads();
    if (threadIdx.x == 0) {
      int n = 0;
      for (int s = (int)(sb / a.I); s <= (int)((se - 1) / a.I) && n + 2 <= kMaxSegs; ++s) {
        long aa = sb > (long)s * a.I ? sb : (long)s * a.I;
        long bb = se < (long)(s + 1) * a.I ? se : (long)(s + 1) * a.I;
        const ExpertW &ew = a.Experts[a.SelIdx[a.slot_begin + s]];
        long r0 = aa - (long)s * a.I;
        RowSeg &g = bs.segs[n++];
        g.P = ew.gP + r0 * (K / 2); g.S = ew.gS + r0 * G; g.nrows = (int)(bb - aa); g.vec = 0;
        g.trow = (int)(aa - sb);
        RowSeg &u = bs.segs[n++];
        u.P = ew.uP + r0 * (K / 2); u.S = ew.uS + r0 * G; u.nrows = (int)(bb - aa); u.vec = 0;
        u.trow = SB + (int)(aa - sb);
      }
      bs.ibox[0] = n;
      bs.ibox[1] = seg_finalize(bs.segs, n);
    }
    __syncthreads();
    block_dot<K>(bs.segs, bs.ibox[0], bs.ibox[1], act, bs.T);
    const long r = sb + threadIdx.x;
    if (r < se) {
      float g = row_sum<K>(bs.T, threadIdx.x), u = row_sum<K>(bs.T, SB + threadIdx.x);
      a.Act[(size_t)a.slot_begin * a.I + r] = silu_mul(g, u);
    }
  }
}
__device__ __forceinline__ void gateup_block_dispatch(const ExpertGateUpArgs &a, const StagedAct4 &act,
                                                      const BlockScratch &bs, int blk, int nblk) {
  switch (a.H) {
    case 256: gateup_block<256>(a, act, bs, blk, nblk); break;
    case 512: gateup_block<512>(a, act, bs, blk, nblk); break;
    case 1024: gateup_block<1024>(a, act, bs, blk, nblk); break;
    case 2048: gateup_block<2048>(a, act, bs, blk, nblk); break;
    case 4096: gateup_block<4096>(a, act, bs, blk, nblk); break;
    default: break;
  }
}

// ---- expert down + combine + residual: output rows n in [0, H), all slots ----
template <int K>
__device__ __forceinline__ void down_block(const ExpertDownCombineArgs &a, const StagedAct4 &act,
                                           const BlockScratch &bs, int blk, int nblk) {
  constexpr int G = K / 128;
  long lo, hi;
  block_range(a.H, blk, nblk, lo, hi);
  const int sb_rows = kTCap / (G * (a.slots > 0 ? a.slots : 1)) < 256 ? kTCap / (G * (a.slots > 0 ? a.slots : 1)) : 256;
#pragma unroll 1
  for (long sb = lo; sb < hi; sb += sb_rows) {
    const long se = sb + sb_rows < hi ? sb + sb_rows : hi;
    const int nr = (int)(se - sb);
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int s = 0; s < a.slots; ++s) {
        const ExpertW &ew = a.Experts[a.SelIdx[s]];
        RowSeg &d = bs.segs[s];
        d.P = ew.dP + sb * (K / 2); d.S = ew.dS + sb * G; d.nrows = nr; d.vec = s; d.trow = s * nr;
      }
      bs.ibox[0] = a.slots;
      bs.ibox[1] = seg_finalize(bs.segs, a.slots);
    }
    __syncthreads();
    block_dot<K>(bs.segs, bs.ibox[0], bs.ibox[1], act, bs.T);
    const long n = sb + threadIdx.x;
    if (n < se) {
      float acc = 0.0f;
      for (int s = 0; s < a.slots; ++s) acc = acc + a.SelW[s] * row_sum<K>(bs.T, s * nr + threadIdx.x);
      if (a.Moe) a.Moe[n] = acc;
      a.X[n] = __ldcg(a.Res + n) + acc;
    }
  }
}
__device__ __forceinline__ void down_block_dispatch(const ExpertDownCombineArgs &a, const StagedAct4 &act,
                                                    const BlockScratch &bs, int blk, int nblk) {
  switch (a.I) {
    case 128: down_block<128>(a, act, bs, blk, nblk); break;
    case 256: down_block<256>(a, act, bs, blk, nblk); break;
    case 512: down_block<512>(a, act, bs, blk, nblk); break;
    case 1024: down_block<1024>(a, act, bs, blk, nblk); break;
    default: break;
  }
}

}  // namespace ainfer
