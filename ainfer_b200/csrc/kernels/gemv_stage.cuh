// Int4GemvA8: the weight-streaming GEMV of the decode loop (batch <= 8).
// Replaces the reference's Int4Gemv (tools/cmdlist/kernels.cpp:148-193) and,
// through per-matrix epilogues, the single-purpose kernels that follow it in
// the recorded layer lists (tools/decode/decode_l0.cpp:611-621,630-638,663):
// ResAddF, SsmConv, BetaG. One launch covers several matrices that share the
// same quantised activation (e.g. in_proj_qkv, in_proj_z, in_proj_b, in_proj_a).
#pragma once
#include "../common/tables.h"
#include "common.cuh"

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

// Operands of a row's epilogue that do not depend on the row's dot product, fetched before
// the dot so that their round trip to memory overlaps it (gemv_epilogue would otherwise start
// these loads only after the last tile has been consumed).
struct EpiOperands {
  float v[7];
};
__device__ __forceinline__ void gemv_epilogue_fetch(const GemvMat *pmt, int n, int m, EpiOperands &o) {
  const GemvMat &mt = *pmt;
  switch (mt.epi) {
    case EPI_RESADD:
      o.v[0] = __ldcg(mt.e0 + (size_t)m * mt.ldy + n);
      break;
    case EPI_CONV_SILU: {
      const float *cs = mt.e1 + (size_t)n * 3;
      const float4 cw = __ldg(reinterpret_cast<const float4 *>(mt.e0) + n);
      o.v[0] = __ldcg(cs); o.v[1] = __ldcg(cs + 1); o.v[2] = __ldcg(cs + 2);
      o.v[3] = cw.x; o.v[4] = cw.y; o.v[5] = cw.z; o.v[6] = cw.w;
      break;
    }
    case EPI_GDECAY:
      o.v[0] = __ldg(mt.e2 + n);
      o.v[1] = __ldg(mt.e0 + n);
      break;
    default:
      break;
  }
}
// gemv_epilogue with the operands already in registers (same arithmetic).
static __device__ __noinline__ void gemv_epilogue_with(const GemvMat *pmt, int n, int m, float acc,
                                                       const EpiOperands &o) {
  const GemvMat &mt = *pmt;
  switch (mt.epi) {
    case EPI_STORE:
      mt.Y[(size_t)m * mt.ldy + n] = acc;
      break;
    case EPI_RESADD:
      mt.Y[(size_t)m * mt.ldy + n] = o.v[0] + acc;
      break;
    case EPI_CONV_SILU: {
      float *cs = mt.e1 + (size_t)n * 3;
      float a = o.v[0] * o.v[3];
      a = a + o.v[1] * o.v[4];
      a = a + o.v[2] * o.v[5];
      a = a + acc * o.v[6];
      mt.Y[n] = a / (1.0f + det_expf(-a));
      cs[0] = o.v[1];
      cs[1] = o.v[2];
      cs[2] = acc;
      break;
    }
    case EPI_BETA:
      mt.Y[n] = 1.0f / (1.0f + det_expf(-acc));
      break;
    case EPI_GDECAY: {
      float sa = acc + o.v[0];
      float soft = sa > 20.0f ? sa : det_logf(1.0f + det_expf(sa));
      mt.Y[n] = (-det_expf(o.v[1])) * soft;
      break;
    }
  }
}

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
}  // namespace ainfer
