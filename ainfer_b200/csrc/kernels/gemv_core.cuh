// Warp-level INT4 (group 128) x INT8 row dot used by every weight-streaming
// kernel of the decode path.
//
// Arithmetic (tools/cmdlist/kernels.cpp:157-191 of the reference): per row and
// per group of 128 weights an exact int32 sum of nibble*activation, then
//   acc = acc + ((float)gs * weight_scale) * act_scale[g]
// in ascending group order, fp32, no fused multiply-add. Integer sums are
// associative, so the 128 products of a group may be split over four lanes;
// the fp32 accumulation is replayed in group order, so the result equals the
// reference's one-work-item-per-row loop bit for bit.
//
// Memory: a row is K/2 contiguous bytes; lanes read consecutive 16-byte chunks
// (128-bit coalesced loads, kept out of L1), unpack nibbles in registers with
// two logic ops per 8 weights and feed dp4a.
//
// Code shape: row loops are rolled (one pass of the warp per iteration, the
// next pass' loads issued before the current pass' math) and the slow scalar
// helpers are not inlined, so that the instructions a layer executes stay
// resident in the instruction caches. A first version unrolled whole tiles
// (34 KB of straight-line code per shape) and was bound by instruction fetch.
#pragma once
#include "common.cuh"

namespace ainfer {

// Shared-memory view of the staged activations for one GEMV launch.
struct StagedAct {
  const uint4 *x;    // [M][K/16] de-interleaved activation words
  const int *gsum;   // [M][K/128] sum of INT8 activations per group
  const float *sq;   // [M][K/128] activation scales
};

template <int K>
struct RowGeom {
  static constexpr int CPR = K / 32;                   // 16-byte chunks per row
  static constexpr int LPR = CPR < 32 ? CPR : 32;      // lanes that share a row
  static constexpr int RPW = 32 / LPR;                 // rows per warp pass
  static constexpr int ITERS = (CPR + LPR - 1) / LPR;  // chunks per lane per row
  static constexpr int G = K / 128;
  static constexpr int GPI = LPR / 4;                  // groups finished per iteration
};

// Registers of one pass: the lane's 16-byte chunks of its row (ITERS of them)
// and, on the first lane of each quad, the group's weight scale.
template <int K>
struct PassRegs {
  uint4 w[RowGeom<K>::ITERS];
  float sc[RowGeom<K>::ITERS];
};

// Issues the loads of one pass. P/S point at the lane's row; ok = the row exists.
template <int K>
__device__ __forceinline__ void pass_load(PassRegs<K> &r, const uint8_t *P, const uint16_t *S, bool ok) {
  using Gm = RowGeom<K>;
  const int cl = (threadIdx.x & 31) % Gm::LPR;
#pragma unroll
  for (int it = 0; it < Gm::ITERS; ++it) {
    int c = cl + Gm::LPR * it;
    if (ok && c < Gm::CPR) {
      r.w[it] = ldg_stream16(P + (long)c * 16);
      r.sc[it] = (cl & 3) == 0 ? bf16_to_f32(__ldg(S + (c >> 2))) : 0.0f;
    } else {
      r.w[it] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
      r.sc[it] = 0.0f;
    }
  }
}

// Dot of one pass with M activation vectors starting at vector v0: exact int32
// group sums (four lanes per group), then the fp32 accumulation replayed in
// ascending group order.
template <int K, int M>
__device__ __forceinline__ void pass_dot(const PassRegs<K> &r, const StagedAct &a, int v0, float (&acc)[M]) {
  using Gm = RowGeom<K>;
  const int lane = threadIdx.x & 31;
  const int cl = lane % Gm::LPR;
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.0f;
#pragma unroll
  for (int it = 0; it < Gm::ITERS; ++it) {
    int c = cl + Gm::LPR * it;
    int cc = c < Gm::CPR ? c : 0;
    int g = cc >> 2;
    float t[M];
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint4 *xm = a.x + (size_t)(v0 + m) * (K / 16);
      int s = dot_chunk_biased(r.w[it], xm[2 * cc], xm[2 * cc + 1], 0);
      s += __shfl_xor_sync(kFull, s, 1);
      s += __shfl_xor_sync(kFull, s, 2);
      int gs = s - 8 * a.gsum[(v0 + m) * Gm::G + g];
      float v = (float)gs * r.sc[it];
      t[m] = v * a.sq[(v0 + m) * Gm::G + g];
    }
#pragma unroll
    for (int j = 0; j < Gm::GPI; ++j) {
      if (Gm::GPI * it + j < Gm::G) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          float tj = __shfl_sync(kFull, t[m], (lane & ~(Gm::LPR - 1)) + 4 * j);
          acc[m] = acc[m] + tj;
        }
      }
    }
  }
}

// Quantises M fp32 vectors of K elements (per-128 activation quantiser,
// tools/cmdlist/kernels.cpp:551-579) straight into the staged shared-memory
// form. One warp per group; same smem layout as stage_act.
template <bool kGlobalSrc = true>
__device__ __forceinline__ StagedAct stage_act_from_f32(unsigned char *smem, const float *x, int K,
                                                        int M, long x_stride) {
  uint32_t *xw = reinterpret_cast<uint32_t *>(smem);
  const int G = K / 128;
  int *gs = reinterpret_cast<int *>(smem + (size_t)M * K);
  float *sqs = reinterpret_cast<float *>(smem + (size_t)M * K + (size_t)M * G * 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int i = warp; i < M * G; i += warps) {
    int m = i / G, g = i % G;
    const float4 *src = reinterpret_cast<const float4 *>(x + m * x_stride + (long)g * 128 + lane * 4);
    float4 v = kGlobalSrc ? __ldcg(src) : *src;  // shared-memory sources take the plain load
    float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    mx = warp_max(mx);
    float s = mx / 127.0f;
    if (s == 0.0f) s = 1.0f;
    int q0 = quant_round(v.x, s), q1 = quant_round(v.y, s), q2 = quant_round(v.z, s),
        q3 = quant_round(v.w, s);
    uint32_t own = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) |
                   ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
    uint32_t other = __shfl_xor_sync(kFull, own, 1);
    int piece = (m * (K / 8)) + g * 16 + (lane >> 1);
    if (lane & 1) xw[2 * piece + 1] = __byte_perm(other, own, 0x7531);
    else xw[2 * piece] = __byte_perm(own, other, 0x6420);
    int sum = warp_sum_int(q0 + q1 + q2 + q3);
    if (lane == 0) {
      gs[i] = sum;
      sqs[i] = s;
    }
  }
  __syncthreads();
  StagedAct a;
  a.x = reinterpret_cast<const uint4 *>(smem);
  a.gsum = gs;
  a.sq = sqs;
  return a;
}

// Stages M activation vectors (natural-order INT8, fp32 group scales) for
// warp_rows_dot. smem layout: [M*K bytes x][M*G ints gsum][M*G floats sq].
__device__ __forceinline__ StagedAct stage_act(unsigned char *smem, const int8_t *__restrict__ xq,
                                               const float *__restrict__ sq, int K, int M,
                                               long xq_stride, long sq_stride) {
  uint32_t *xw = reinterpret_cast<uint32_t *>(smem);
  int G = K / 128;
  int *gs = reinterpret_cast<int *>(smem + (size_t)M * K);
  float *sqs = reinterpret_cast<float *>(smem + (size_t)M * K + (size_t)M * G * 4);
  for (int i = threadIdx.x; i < M * (K / 8); i += blockDim.x) {
    int m = i / (K / 8), j = i % (K / 8);
    uint2 v = __ldcg(reinterpret_cast<const uint2 *>(xq + m * xq_stride + (long)j * 8));
    xw[2 * i] = __byte_perm(v.x, v.y, 0x6420);
    xw[2 * i + 1] = __byte_perm(v.x, v.y, 0x7531);
  }
  for (int i = threadIdx.x; i < M * G; i += blockDim.x) sqs[i] = __ldcg(sq + (i / G) * sq_stride + (i % G));
  __syncthreads();
  for (int i = threadIdx.x; i < M * G; i += blockDim.x) {
    int s = 0;
#pragma unroll 8
    for (int k = 0; k < 32; ++k) s = __dp4a((int)xw[i * 32 + k], 0x01010101, s);
    gs[i] = s;
  }
  __syncthreads();
  StagedAct a;
  a.x = reinterpret_cast<const uint4 *>(smem);
  a.gsum = gs;
  a.sq = sqs;
  return a;
}
__host__ __device__ inline uint32_t staged_act_bytes(int K, int M) {
  return (uint32_t)((size_t)M * K + (size_t)M * (K / 128) * 8);
}

}  // namespace ainfer
