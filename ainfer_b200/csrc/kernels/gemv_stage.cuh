// Int4GemvA8: the weight-streaming GEMV of the decode loop (batch <= 8).
// Replaces the reference's Int4Gemv (tools/cmdlist/kernels.cpp:148-193) and,
// through per-matrix epilogues, the single-purpose kernels that follow it in
// the recorded layer lists (tools/decode/decode_l0.cpp:611-621,630-638,663):
// ResAddF, SsmConv, BetaG. One launch covers several matrices that share the
// same quantised activation (e.g. in_proj_qkv, in_proj_z, in_proj_b, in_proj_a).
#pragma once
#include "../common/tables.h"
#include "gemv_core.cuh"

namespace ainfer {

struct Int4GemvA8Args {
  const GemvMat *mats;
  int32_t nmats;
  int32_t total_rows;
  const int8_t *XQ;   // [M][K] natural order
  const float *SQ;    // [M][K/128]
  int32_t K;
  int32_t M;
};

__device__ __forceinline__ void gemv_epilogue(const GemvMat &mt, int n, int m, float acc) {
  switch (mt.epi) {
    case EPI_STORE:
      mt.Y[(size_t)m * mt.ldy + n] = acc;
      break;
    case EPI_RESADD:
      mt.Y[(size_t)m * mt.ldy + n] = __ldcg(mt.e0 + (size_t)m * mt.ldy + n) + acc;
      break;
    case EPI_CONV_SILU: {
      float *cs = mt.e1 + (size_t)n * 3;
      const float *cw = mt.e0 + (size_t)n * 4;
      float h0 = __ldcg(cs), h1 = __ldcg(cs + 1), h2 = __ldcg(cs + 2);
      float a = h0 * cw[0];
      a = a + h1 * cw[1];
      a = a + h2 * cw[2];
      a = a + acc * cw[3];
      mt.Y[n] = a / (1.0f + det_expf(-a));
      cs[0] = h1;
      cs[1] = h2;
      cs[2] = acc;
      break;
    }
    case EPI_BETA:
      mt.Y[n] = 1.0f / (1.0f + det_expf(-acc));
      break;
    case EPI_GDECAY: {
      float sa = acc + mt.e2[n];
      float soft = sa > 20.0f ? sa : det_logf(1.0f + det_expf(sa));
      mt.Y[n] = (-det_expf(mt.e0[n])) * soft;
      break;
    }
  }
}

template <int K, int M, int RT>
__device__ __forceinline__ void gemv_rows(const Int4GemvA8Args &a, const StagedAct &act,
                                          const GemvMat *smats, int blk, int nblk) {
  using Gm = RowGeom<K>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  constexpr int ROWS_PER_WARP = RT * Gm::RPW;
  const long tile_rows = (long)warps * ROWS_PER_WARP;
  for (long base = (long)blk * tile_rows; base < a.total_rows; base += (long)nblk * tile_rows) {
    long row0 = base + (long)warp * ROWS_PER_WARP;
    if (row0 >= a.total_rows) continue;
    // Per-lane row -> matrix lookup (rows are global over the table, nmats <= 8;
    // lanes of one warp may fall into different matrices).
    float acc[RT][M];
    LaneRows<RT> rows;
    int mi[RT];
    long lrow[RT];
#pragma unroll
    for (int p = 0; p < RT; ++p) {
      long r = row0 + (long)p * Gm::RPW + lane / Gm::LPR;
      int idx = 0;
      for (int i = 1; i < a.nmats; ++i)
        if (r >= smats[i].row_start) idx = i;
      mi[p] = idx;
      lrow[p] = r - smats[idx].row_start;
      rows.ok[p] = r < a.total_rows;
      long lr = rows.ok[p] ? lrow[p] : 0;
      rows.P[p] = smats[idx].P + lr * (K / 2);
      rows.S[p] = smats[idx].S + lr * Gm::G;
    }
    warp_rows_dot<K, M, RT>(rows, act, acc);
#pragma unroll
    for (int p = 0; p < RT; ++p) {
      long r = row0 + (long)p * Gm::RPW + lane / Gm::LPR;
      if (r < a.total_rows && (lane % Gm::LPR) == 0) {
        const GemvMat &mt = smats[mi[p]];
#pragma unroll
        for (int m = 0; m < M; ++m) gemv_epilogue(mt, (int)lrow[p], m, acc[p][m]);
      }
    }
  }
}

// Rows of one launch for this block: act holds the staged activations, smats
// the launch's matrix table (shared memory).
template <int M>
__device__ __forceinline__ void gemv_dispatch_k(const Int4GemvA8Args &a, const StagedAct &act,
                                                const GemvMat *smats, int blk, int nblk) {
  switch (a.K) {
    case 128: gemv_rows<128, M, 4>(a, act, smats, blk, nblk); break;
    case 256: gemv_rows<256, M, 4>(a, act, smats, blk, nblk); break;
    case 512: gemv_rows<512, M, 4>(a, act, smats, blk, nblk); break;
    case 1024: gemv_rows<1024, M, 4>(a, act, smats, blk, nblk); break;
    case 2048: gemv_rows<2048, M, 2>(a, act, smats, blk, nblk); break;
    case 4096: gemv_rows<4096, M, 1>(a, act, smats, blk, nblk); break;
    case 8192: gemv_rows<8192, M, 1>(a, act, smats, blk, nblk); break;
    default: break;  // rejected on the host before launch
  }
}
// Rows one block tile covers (8 warps), by K; the host mirrors this to size grids.
__host__ __device__ inline int gemv_tile_rows(int K) {
  int cpr = K / 32, lpr = cpr < 32 ? cpr : 32, rpw = 32 / lpr;
  int rt = K <= 1024 ? 4 : (K == 2048 ? 2 : 1);
  return 8 * rt * rpw;
}

}  // namespace ainfer
