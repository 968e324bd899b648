// Int4GemmA16: INT4 g128 weights x BF16 activations, 1 <= M <= 64 rows of
// activations (the "float-activation" policy of the operator sweep,
// tools/kernels/gemv.cpp:480-501: y[m][n] = sum_k nib * scale * x[m][k]).
// Unlike the decode path (W4A8, integer dots, bit-exact) this operator is
// floating point: products run on the tensor cores (mma.sync m16n8k16, bf16
// inputs, fp32 accumulate) with the weights as the 16-row operand, so one mma
// covers 16 weight rows x 8 activation rows x 16 k. Nibbles become exact bf16
// integers in registers; a group's 128 k are accumulated unscaled in fp32 and
// the group's scale is applied once per group. Tolerance against the double
// precision host form: rel 2e-2 / abs 1e-2 (the reference's bar,
// tools/kernels/gemv.cpp:586-593); measured error is ~1e-6 relative.
//
// Block = 256 threads = 8 warps = 128 weight rows; a warp owns 16 rows and all
// M columns. Weights go straight from global memory to registers (each lane
// reads 16 contiguous bytes of two rows per group, prefetched one group ahead);
// the activations of a group ([M][128] bf16) are staged in shared memory by
// the whole block, double buffered.
#include <cuda_bf16.h>

#include "../common/tables.h"
#include "common.cuh"
#include "registry.h"

namespace ainfer {

struct Int4GemmA16Args {
  const uint8_t *P;    // [N][K/2]
  const uint16_t *S;   // [N][K/128] bf16
  const uint16_t *X;   // [M][K] bf16 activations
  float *Y;            // [M][N]
  int32_t N, K, M;
};

constexpr int kA16RowStride = 136;  // bf16 elements per staged activation row (128 + 8 of padding)

// Two nibbles of a byte (low = even k, high = odd k, two's complement) as bf16x2 {v_even, v_odd}.
__device__ __forceinline__ uint32_t nib2_to_bf16x2(uint32_t byte) {
  // 0x4300 | u is the bf16 128 + u for u in 0..15; with u = n ^ 8 = v + 8 that is v + 136
  uint32_t t = (((byte & 0x0Fu) | ((byte & 0xF0u) << 12)) ^ 0x00080008u) | 0x43004300u;
  __nv_bfloat162 r = *reinterpret_cast<__nv_bfloat162 *>(&t);
  r = __hsub2(r, __float2bfloat162_rn(136.0f));
  return *reinterpret_cast<uint32_t *>(&r);
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(256) Int4GemmA16(const Int4GemmA16Args a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ __align__(16) uint16_t xs[2][64 * kA16RowStride];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g4 = lane >> 2, c = lane & 3;
  const int G = a.K / 128;
  const int MT = (a.M + 7) / 8;  // 8-column tiles of activation rows
  const long row_lo = (long)blockIdx.x * 128 + warp * 16;
  // rows this lane feeds into the mma: row_lo + g4 and row_lo + g4 + 8 (clamped; results of rows >= N are dropped)
  const long r0 = row_lo + g4 < a.N ? row_lo + g4 : a.N - 1;
  const long r1 = row_lo + g4 + 8 < a.N ? row_lo + g4 + 8 : a.N - 1;
  const uint8_t *p0 = a.P + r0 * (a.K / 2) + c * 16, *p1 = a.P + r1 * (a.K / 2) + c * 16;
  const uint16_t *s0 = a.S + r0 * G, *s1 = a.S + r1 * G;

  float tot[8][4];
#pragma unroll
  for (int t = 0; t < 8; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) tot[t][i] = 0.0f;

  // stage the activations of group g into buffer b: [M][128] bf16, zero rows beyond M
  auto stage_x = [&](int g, int b) {
    for (int i = tid; i < MT * 8 * 16; i += 256) {  // 16-byte pieces: 16 per row
      const int m = i >> 4, piece = i & 15;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < a.M) v = __ldg(reinterpret_cast<const uint4 *>(a.X + (size_t)m * a.K + (size_t)g * 128) + piece);
      *reinterpret_cast<uint4 *>(&xs[b][m * kA16RowStride + piece * 8]) = v;
    }
  };

  uint4 w0 = __ldg(reinterpret_cast<const uint4 *>(p0)), w1 = __ldg(reinterpret_cast<const uint4 *>(p1));
  uint32_t sc0 = __ldg(s0), sc1 = __ldg(s1);
  stage_x(0, 0);
  __syncthreads();
#pragma unroll 1
  for (int g = 0; g < G; ++g) {
    const int b = g & 1;
    // prefetch the next group's weights and activations
    uint4 nw0 = w0, nw1 = w1;
    uint32_t nsc0 = sc0, nsc1 = sc1;
    if (g + 1 < G) {
      nw0 = __ldg(reinterpret_cast<const uint4 *>(p0 + (size_t)(g + 1) * 64));
      nw1 = __ldg(reinterpret_cast<const uint4 *>(p1 + (size_t)(g + 1) * 64));
      nsc0 = __ldg(s0 + g + 1);
      nsc1 = __ldg(s1 + g + 1);
      stage_x(g + 1, b ^ 1);
    }
    float acc[8][4];
#pragma unroll
    for (int t = 0; t < 8; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][i] = 0.0f;
    const uint32_t wa[4] = {w0.x, w0.y, w0.z, w0.w}, wb[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      // this lane's bytes 2kk and 2kk+1 of its 16-byte chunk: k = 32c + 4kk + {0,1} and + {2,3}
      const uint32_t wwa = wa[kk >> 1], wwb = wb[kk >> 1];
      const int sh = (kk & 1) * 16;
      uint32_t af[4];
      af[0] = nib2_to_bf16x2((wwa >> sh) & 0xFFu);
      af[1] = nib2_to_bf16x2((wwb >> sh) & 0xFFu);
      af[2] = nib2_to_bf16x2((wwa >> (sh + 8)) & 0xFFu);
      af[3] = nib2_to_bf16x2((wwb >> (sh + 8)) & 0xFFu);
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        if (t < MT) {
          // column t*8 + g4 of the activation tile, k = 32c + 4kk .. +3 (four consecutive bf16)
          const uint2 xv = *reinterpret_cast<const uint2 *>(&xs[b][(t * 8 + g4) * kA16RowStride + 32 * c + 4 * kk]);
          mma_bf16_16816(acc[t], af, xv.x, xv.y);
        }
      }
    }
    const float f0 = __uint_as_float(sc0 << 16), f1 = __uint_as_float(sc1 << 16);
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      if (t < MT) {
        tot[t][0] = tot[t][0] + acc[t][0] * f0;
        tot[t][1] = tot[t][1] + acc[t][1] * f0;
        tot[t][2] = tot[t][2] + acc[t][2] * f1;
        tot[t][3] = tot[t][3] + acc[t][3] * f1;
      }
    }
    w0 = nw0; w1 = nw1; sc0 = nsc0; sc1 = nsc1;
    __syncthreads();  // the next buffer is complete; this one is free for group g + 2
  }
  // d0,d1: row g4, columns 2c, 2c+1 of the tile; d2,d3: row g4 + 8
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    if (t < MT) {
      const int m0 = t * 8 + 2 * c;
      const long ra = row_lo + g4, rb = row_lo + g4 + 8;
      if (ra < a.N) {
        if (m0 < a.M) a.Y[(size_t)m0 * a.N + ra] = tot[t][0];
        if (m0 + 1 < a.M) a.Y[(size_t)(m0 + 1) * a.N + ra] = tot[t][1];
      }
      if (rb < a.N) {
        if (m0 < a.M) a.Y[(size_t)m0 * a.N + rb] = tot[t][2];
        if (m0 + 1 < a.M) a.Y[(size_t)(m0 + 1) * a.N + rb] = tot[t][3];
      }
    }
  }
}

#define F(f) AINFER_ARG(Int4GemmA16Args, f)
AINFER_REGISTER(Int4GemmA16, Int4GemmA16Args, 256, 128, 0, nullptr, F(P), F(S), F(X), F(Y), F(N), F(K), F(M));
#undef F
AINFER_EARLY_LAUNCH(Int4GemmA16);

}  // namespace ainfer
