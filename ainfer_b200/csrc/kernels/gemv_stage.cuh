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

// Not inlined: called by one lane per finished row, and kept out of the row loop's code.
static __device__ __noinline__ void gemv_epilogue(const GemvMat *pmt, int n, int m, float acc) {
  const GemvMat &mt = *pmt;
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

// Rows of one launch for this block. Each warp walks passes of RPW rows (grid
// stride over blocks), keeps the next pass' loads in flight while it computes
// the current one, and hands each finished row to the matrix's epilogue.
template <int K, int M>
__device__ __forceinline__ void gemv_rows(const Int4GemvA8Args &a, const StagedAct &act,
                                          const GemvMat *smats, int blk, int nblk) {
  using Gm = RowGeom<K>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const long total = a.total_rows;
  const long stride = (long)nblk * warps * Gm::RPW;
  long wrow = ((long)blk * warps + warp) * Gm::RPW;  // first row of this warp's pass
  if (wrow >= total) return;
  const int rs = lane / Gm::LPR;
  // row -> (matrix, local row); rows are global over the launch's table (nmats <= 8)
  auto locate = [&](long r, int &mi, long &lr, bool &ok) {
    int idx = 0;
    for (int i = 1; i < a.nmats; ++i)
      if (r >= smats[i].row_start) idx = i;
    ok = r < total;
    mi = idx;
    lr = ok ? r - smats[idx].row_start : 0;
  };
  PassRegs<K> cur, nxt;
  int mi_c, mi_n = 0;
  long lr_c, lr_n = 0;
  bool ok_c, ok_n = false;
  locate(wrow + rs, mi_c, lr_c, ok_c);
  pass_load<K>(cur, smats[mi_c].P + lr_c * (K / 2), smats[mi_c].S + lr_c * Gm::G, ok_c);
#pragma unroll 1
  for (; wrow < total; wrow += stride) {
    const bool more = wrow + stride < total;  // warp-uniform
    if (more) {
      locate(wrow + stride + rs, mi_n, lr_n, ok_n);
      pass_load<K>(nxt, smats[mi_n].P + lr_n * (K / 2), smats[mi_n].S + lr_n * Gm::G, ok_n);
    }
    float acc[M];
    pass_dot<K, M>(cur, act, 0, acc);
    if (ok_c && (lane % Gm::LPR) == 0) {
#pragma unroll
      for (int m = 0; m < M; ++m) gemv_epilogue(smats + mi_c, (int)lr_c, m, acc[m]);
    }
    cur = nxt;
    mi_c = mi_n; lr_c = lr_n; ok_c = ok_n;
  }
}

// act holds the staged activations, smats the launch's matrix table (shared memory).
template <int M>
__device__ __forceinline__ void gemv_dispatch_k(const Int4GemvA8Args &a, const StagedAct &act,
                                                const GemvMat *smats, int blk, int nblk) {
  switch (a.K) {
    case 128: gemv_rows<128, M>(a, act, smats, blk, nblk); break;
    case 256: gemv_rows<256, M>(a, act, smats, blk, nblk); break;
    case 512: gemv_rows<512, M>(a, act, smats, blk, nblk); break;
    case 1024: gemv_rows<1024, M>(a, act, smats, blk, nblk); break;
    case 2048: gemv_rows<2048, M>(a, act, smats, blk, nblk); break;
    case 4096: gemv_rows<4096, M>(a, act, smats, blk, nblk); break;
    case 8192: gemv_rows<8192, M>(a, act, smats, blk, nblk); break;
    default: break;  // rejected on the host before launch
  }
}
// Rows one pass of a block (8 warps) covers, by K; the host mirrors this to size grids.
__host__ __device__ inline int gemv_tile_rows(int K) {
  int cpr = K / 32, lpr = cpr < 32 ? cpr : 32;
  return 8 * (32 / lpr);
}

}  // namespace ainfer
