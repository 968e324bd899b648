// Chunk path of the Gated DeltaNet layer: M consecutive tokens per launch, with the conv history
// and the recurrent state carried from row to row on the chip and across launches in memory.
// Replaces ChunkSsmConv and ChunkSsmRecur of the reference (tools/cmdlist/kernels.cpp:896-917,
// 919-999; host mirror tools/cmdlist/chunkssm_replay.cpp:220-255). Like the reference's, the
// chunk kernels run the sequential recurrence (row m + 1 sees the state row m left), so a chunk
// of M rows is bit-identical to M decode steps; what changes is where the state lives: a block
// owns 32 columns of one head's 128x128 state in registers for the whole chunk, reads it once
// and writes it once, instead of once per token.
#include "deltanet_core.cuh"

namespace ainfer {

// ---- ChunkConvSilu: depthwise conv (k = 4) + SiLU over M rows, history chained through the chunk ----
struct ChunkConvSiluArgs {
  float *Mx;          // [M][C] conv outputs (SiLU applied)
  const float *QKV;   // [M][C] projections
  float *CS;          // [C][3] history, updated
  const float *CW;    // [C][4] taps
  int32_t C, M;
  float *Snap;        // optional: the history [C][3] after row m at Snap + m * snap_stride (to roll a speculative chunk back); null: none
  int64_t snap_stride;
};
__global__ void __launch_bounds__(256) ChunkConvSilu(const ChunkConvSiluArgs a) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= a.C) return;
  float h0 = a.CS[c * 3 + 0], h1 = a.CS[c * 3 + 1], h2 = a.CS[c * 3 + 2];
  const float4 w = __ldg(reinterpret_cast<const float4 *>(a.CW) + c);
  for (int m = 0; m < a.M; ++m) {
    const float x = a.QKV[(size_t)m * a.C + c];
    float acc = h0 * w.x;
    acc = acc + h1 * w.y;
    acc = acc + h2 * w.z;
    acc = acc + x * w.w;
    a.Mx[(size_t)m * a.C + c] = acc / (1.0f + det_expf(-acc));
    h0 = h1; h1 = h2; h2 = x;
    if (a.Snap) {
      float *sn = a.Snap + (size_t)m * a.snap_stride + (size_t)c * 3;
      sn[0] = h0; sn[1] = h1; sn[2] = h2;
    }
  }
  a.CS[c * 3 + 0] = h0; a.CS[c * 3 + 1] = h1; a.CS[c * 3 + 2] = h2;
}

// ---- ChunkBetaDecay: beta = sigmoid(b), g = -exp(A_log) * softplus(a + dt_bias) for M rows ----
// (BetaG, tools/cmdlist/kernels.cpp:606-617; the arithmetic of the decode GEMV's epilogues.)
struct ChunkBetaDecayArgs {
  const float *B;        // [M][nV] in_proj_b outputs
  const float *A;        // [M][nV] in_proj_a outputs
  const float *ALog;     // [nV]
  const float *DtBias;   // [nV]
  float *Bt;             // [M][nV]
  float *Gt;             // [M][nV]
  int32_t nV, count;     // count = M * nV
};
__global__ void __launch_bounds__(256) ChunkBetaDecay(const ChunkBetaDecayArgs a) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= a.count) return;
  const int h = i % a.nV;
  a.Bt[i] = 1.0f / (1.0f + det_expf(-a.B[i]));
  const float sa = a.A[i] + a.DtBias[h];
  const float soft = sa > 20.0f ? sa : det_logf(1.0f + det_expf(sa));
  a.Gt[i] = (-det_expf(a.ALog[h])) * soft;
}

// ---- ChunkDeltaNet: the gated delta rule over M rows ----
struct ChunkDeltaNetArgs {
  float *Out;        // [M][nV][128] head outputs
  const float *Mx;   // [M][C] conv outputs, a row = [q: nK*128 | k: nK*128 | v: nV*128]
  float *S;          // [nV][128][128] state, row-major [k][v], updated
  const float *Bt;   // [M][nV] beta
  const float *Gt;   // [M][nV] log decay
  int32_t nK, nV, M;
  float *Snap;       // optional: the state [nV][128][128] after row m at Snap + m * snap_stride (to roll a speculative chunk back); null: none
  int64_t snap_stride;
};
constexpr int kChunkRows = 64;   // rows whose normalised q / k are staged at a time

extern __shared__ __align__(16) float chunk_smem[];

// One block of 256 threads per (head, 32-column slice); grid = nV * 4. Per row the arithmetic of
// deltanet_step_body: S *= exp(g); kv = tree8 of 16-row fma chains; d = (v - kv) * beta;
// S += k d; o = tree8 of fma chains with q.
__global__ void __launch_bounds__(256) ChunkDeltaNet(const ChunkDeltaNetArgs a) {
  constexpr int D = 128, SEG = kDnSeg;
  float *qs = chunk_smem;                       // [kChunkRows][128] normalised, scaled q
  float *ks = qs + kChunkRows * D;              // [kChunkRows][128] normalised k
  __shared__ float part[2][8][32];
  __shared__ float s_beta[kChunkRows], s_gt[kChunkRows];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x / kDnSlices, slice = blockIdx.x % kDnSlices;
  if (h >= a.nV) return;
  const int kh = h / (a.nV / a.nK);
  const int col = slice * 32 + lane;
  const int C = 2 * a.nK * D + a.nV * D;
  float *Sh = a.S + (size_t)h * D * D;
  float s[SEG];
#pragma unroll
  for (int r = 0; r < SEG; ++r) s[r] = Sh[(size_t)(warp * SEG + r) * D + col];
  for (int m0 = 0; m0 < a.M; m0 += kChunkRows) {
    const int rows = a.M - m0 < kChunkRows ? a.M - m0 : kChunkRows;
    __syncthreads();   // the previous rows' q / k are no longer read
    // l2norm of the rows' q and k (a warp per (row, which)), beta and decay of the rows
    for (int t = warp; t < rows * 2; t += 8) {
      const int m = t >> 1, which = t & 1;
      const float *src = a.Mx + (size_t)(m0 + m) * C + (which == 0 ? (size_t)kh * D : (size_t)a.nK * D + (size_t)kh * D);
      float x[4];
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[i] = src[lane + 32 * i];
        ss = fmaf(x[i], x[i], ss);
      }
      ss = warp_tree_sum(ss);
      const float inv = 1.0f / sqrtf(ss + 1e-6f);
      const float f = inv * (which == 0 ? 0.0883883476483184405f : 1.0f);  // 128^-1/2 for q
      float *dst = (which == 0 ? qs : ks) + m * D;
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = x[i] * f;
    }
    for (int m = threadIdx.x; m < rows; m += 256) {
      s_beta[m] = a.Bt[(size_t)(m0 + m) * a.nV + h];
      s_gt[m] = det_expf(a.Gt[(size_t)(m0 + m) * a.nV + h]);
    }
    __syncthreads();
    float val = a.Mx[(size_t)m0 * C + (size_t)2 * a.nK * D + (size_t)h * D + col];
    for (int m = 0; m < rows; ++m) {
      const float *kr = ks + m * D + warp * SEG, *qr = qs + m * D + warp * SEG;
      const float gt = s_gt[m], beta = s_beta[m];
      const float val_next = m + 1 < rows ? a.Mx[(size_t)(m0 + m + 1) * C + (size_t)2 * a.nK * D + (size_t)h * D + col] : 0.0f;
      float acc = 0.0f;
#pragma unroll
      for (int r = 0; r < SEG; ++r) {
        s[r] = s[r] * gt;
        acc = fmaf(s[r], kr[r], acc);
      }
      part[0][warp][lane] = acc;
      __syncthreads();
      const float kv = ((part[0][0][lane] + part[0][1][lane]) + (part[0][2][lane] + part[0][3][lane])) +
                       ((part[0][4][lane] + part[0][5][lane]) + (part[0][6][lane] + part[0][7][lane]));
      const float dl = (val - kv) * beta;
      acc = 0.0f;
#pragma unroll
      for (int r = 0; r < SEG; ++r) {
        s[r] = fmaf(kr[r], dl, s[r]);
        acc = fmaf(s[r], qr[r], acc);
      }
      part[1][warp][lane] = acc;
      __syncthreads();   // also: every thread has read part[0] of this row
      if (warp == 0) {
        const float o = ((part[1][0][lane] + part[1][1][lane]) + (part[1][2][lane] + part[1][3][lane])) +
                        ((part[1][4][lane] + part[1][5][lane]) + (part[1][6][lane] + part[1][7][lane]));
        a.Out[((size_t)(m0 + m) * a.nV + h) * D + col] = o;
      }
      if (a.Snap) {
        float *sn = a.Snap + (size_t)(m0 + m) * a.snap_stride + (size_t)h * D * D;
#pragma unroll
        for (int r = 0; r < SEG; ++r) sn[(size_t)(warp * SEG + r) * D + col] = s[r];
      }
      val = val_next;
      // part[1] of this row is read by warp 0 only, before it writes part[1] of the next row
      // (it passes the next row's first barrier in between, as every writer of part[1] does)
    }
  }
#pragma unroll
  for (int r = 0; r < SEG; ++r) Sh[(size_t)(warp * SEG + r) * D + col] = s[r];
}

static uint32_t chunk_dn_smem_fn(const void *) { return 2u * kChunkRows * 128u * 4u; }

#define F(f) AINFER_ARG(ChunkConvSiluArgs, f)
AINFER_REGISTER(ChunkConvSilu, ChunkConvSiluArgs, 256, 256, 0, nullptr, F(Mx), F(QKV), F(CS), F(CW), F(C), F(M), F(Snap), F(snap_stride));
#undef F
#define F(f) AINFER_ARG(ChunkBetaDecayArgs, f)
AINFER_REGISTER(ChunkBetaDecay, ChunkBetaDecayArgs, 256, 256, 0, nullptr, F(B), F(A), F(ALog), F(DtBias), F(Bt), F(Gt), F(nV), F(count));
#undef F
#define F(f) AINFER_ARG(ChunkDeltaNetArgs, f)
AINFER_REGISTER(ChunkDeltaNet, ChunkDeltaNetArgs, 256, 1, 0, chunk_dn_smem_fn, F(Out), F(Mx), F(S), F(Bt), F(Gt), F(nK), F(nV), F(M), F(Snap), F(snap_stride));
#undef F

}  // namespace ainfer
