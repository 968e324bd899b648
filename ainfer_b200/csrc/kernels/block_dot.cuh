// Block-level INT4 (group 128) x INT8 dot over a set of row segments.
//
// The kernel is bound by instruction issue, not by HBM, unless the inner loop
// is lean: at 6.5 TB/s an SM receives 16 bytes of weights every 0.7 cycles,
// which leaves about 90 thread instructions per 16 bytes at perfect issue. A
// first version spent 88 (two shuffles per 16 bytes, a 16-step shuffle replay
// per row, shared-memory reads and address arithmetic per chunk) and reached
// 51 % of the HBM roofline. This version spends about 24:
//   * a lane owns HALF a group: 32 contiguous bytes = 64 weights, fetched with
//     one 256-bit load; a warp instruction reads 1 KB contiguous;
//   * nibbles are never shifted: low nibbles are masked in place, high nibbles
//     are masked in place as 16*n and their dot is divided by 16 at the end
//     (exact: it is a multiple of 16); both are biased by xor 8 to unsigned so
//     that one LOP3 prepares each dp4a operand, and 8*sum(x) is subtracted per
//     group;
//   * one shuffle joins the two halves of a group; the even lane stores
//       t[row][g] = ((float)group_sum * weight_scale) * act_scale[g];
//   * after one __syncthreads a single thread per row adds t[row][0..G) in
//     ascending group order (the reference's accumulation order,
//     tools/cmdlist/kernels.cpp:157-191) and runs the row's epilogue.
// Integer sums are associative and the fp32 sum keeps the reference order, so
// results are bit-identical to the one-work-item-per-row loop.
//
// A block owns contiguous rows (possibly of several matrices: "segments");
// rows are dealt to threads as row = tid / HPR + j * (threads / HPR) with the
// half-group column hc = tid % HPR fixed per thread (HPR = K/64 divides 256).
#pragma once
#include "common.cuh"

namespace ainfer {

// Contiguous rows of one matrix, dotted with one staged activation vector.
struct RowSeg {
  const uint8_t *P;   // packed nibbles of the segment's first row
  const uint16_t *S;  // bf16 scales of the segment's first row
  int32_t nrows;
  int32_t vec;        // staged activation vector this segment is dotted with
  int32_t trow;       // first row of this segment in the t[][] scratch
  int32_t row0;       // first flat row index of this segment (filled by seg_finalize)
};

constexpr int kMaxSegs = 16;
constexpr int kDotLD = 6;  // rows (32-byte loads) in flight per thread

// Staged activations, half-group layout: for vector v, half-group hc and j in
// 0..3 the uint4 x[(v*4 + j) * HPR + hc] holds the de-interleaved INT8 bytes of
// weights hc*64 + 16j .. +15: {even(0..7), odd(0..7), even(8..15), odd(8..15)}
// where even = bytes (x0,x2,x4,x6), odd = (x1,x3,x5,x7) of an 8-weight word.
struct StagedAct4 {
  const uint4 *x;
  const int *gsum;   // [M][K/128] sum of INT8 activations per group
  const float *sq;   // [M][K/128] activation scales
};
__host__ __device__ inline uint32_t staged4_bytes(int K, int M) {
  return (uint32_t)((size_t)M * K + (size_t)M * (K / 128) * 8);
}
// word index (in 32-bit words) of 8-weight piece pc of vector v, parity 0 even / 1 odd
__device__ __forceinline__ int staged4_word(int K, int v, int pc, int parity) {
  const int HPR = K / 64;
  int hc = pc >> 3, j = (pc >> 1) & 3;
  return (((v * 4 + j) * HPR + hc) << 2) + ((pc & 1) << 1) + parity;
}

// Stages M natural-order INT8 vectors (global memory) with their fp32 group scales.
__device__ __forceinline__ StagedAct4 stage4(unsigned char *smem, const int8_t *xq, const float *sq, int K,
                                             int M, long xq_stride, long sq_stride) {
  uint32_t *xw = reinterpret_cast<uint32_t *>(smem);
  const int G = K / 128;
  int *gs = reinterpret_cast<int *>(smem + (size_t)M * K);
  float *sqs = reinterpret_cast<float *>(smem + (size_t)M * K + (size_t)M * G * 4);
  for (int i = threadIdx.x; i < M * (K / 8); i += blockDim.x) {
    int m = i / (K / 8), pc = i % (K / 8);
    uint2 v = __ldcg(reinterpret_cast<const uint2 *>(xq + m * xq_stride + (long)pc * 8));
    xw[staged4_word(K, m, pc, 0)] = __byte_perm(v.x, v.y, 0x6420);
    xw[staged4_word(K, m, pc, 1)] = __byte_perm(v.x, v.y, 0x7531);
  }
  for (int i = threadIdx.x; i < M * G; i += blockDim.x) {
    int m = i / G, g = i % G;
    sqs[i] = __ldcg(sq + m * sq_stride + g);
    const uint4 *grp = reinterpret_cast<const uint4 *>(xq + m * xq_stride + (long)g * 128);
    int s = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      uint4 u = __ldcg(grp + q);
      s = __dp4a((int)u.x, 0x01010101, s);
      s = __dp4a((int)u.y, 0x01010101, s);
      s = __dp4a((int)u.z, 0x01010101, s);
      s = __dp4a((int)u.w, 0x01010101, s);
    }
    gs[i] = s;
  }
  __syncthreads();
  return StagedAct4{reinterpret_cast<const uint4 *>(smem), gs, sqs};
}

// Quantises M fp32 vectors (per-128 activation quantiser, tools/cmdlist/
// kernels.cpp:551-579) straight into the staged form. One warp per group.
template <bool kGlobalSrc>
__device__ __forceinline__ StagedAct4 stage4_from_f32(unsigned char *smem, const float *x, int K, int M,
                                                      long x_stride) {
  uint32_t *xw = reinterpret_cast<uint32_t *>(smem);
  const int G = K / 128;
  int *gs = reinterpret_cast<int *>(smem + (size_t)M * K);
  float *sqs = reinterpret_cast<float *>(smem + (size_t)M * K + (size_t)M * G * 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int i = warp; i < M * G; i += warps) {
    int m = i / G, g = i % G;
    const float4 *src = reinterpret_cast<const float4 *>(x + m * x_stride + (long)g * 128 + lane * 4);
    float4 v = kGlobalSrc ? __ldcg(src) : *src;
    float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    mx = warp_max(mx);
    float s = mx / 127.0f;
    if (s == 0.0f) s = 1.0f;
    int q0 = quant_round(v.x, s), q1 = quant_round(v.y, s), q2 = quant_round(v.z, s),
        q3 = quant_round(v.w, s);
    uint32_t own = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) |
                   ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
    uint32_t other = __shfl_xor_sync(kFull, own, 1);
    int pc = g * 16 + (lane >> 1);  // 8-weight piece: two lanes of 4 weights each
    if (lane & 1) xw[staged4_word(K, m, pc, 1)] = __byte_perm(other, own, 0x7531);
    else xw[staged4_word(K, m, pc, 0)] = __byte_perm(own, other, 0x6420);
    int sum = warp_sum_int(q0 + q1 + q2 + q3);
    if (lane == 0) {
      gs[i] = sum;
      sqs[i] = s;
    }
  }
  __syncthreads();
  return StagedAct4{reinterpret_cast<const uint4 *>(smem), gs, sqs};
}

// Fills row0 (prefix sums); returns the total number of rows. One thread.
__device__ __forceinline__ int seg_finalize(RowSeg *segs, int nseg) {
  int r = 0;
  for (int i = 0; i < nseg; ++i) {
    segs[i].row0 = r;
    r += segs[i].nrows;
  }
  return r;
}

// 256-bit streaming load of a lane's 32 bytes (64 weights).
__device__ __forceinline__ void ldg_stream32(const void *p, uint32_t (&w)[8]) {
  asm("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
      : "l"(p));
}

// sum over 64 weights of (nibble ^ 8) * x: low nibbles exactly, high nibbles as 16*(n^8).
__device__ __forceinline__ void dot64_biased(const uint32_t (&w)[8], const uint4 &x0, const uint4 &x1,
                                             const uint4 &x2, const uint4 &x3, int &lo, int &hi) {
  const uint32_t xe[8] = {x0.x, x0.z, x1.x, x1.z, x2.x, x2.z, x3.x, x3.z};
  const uint32_t xo[8] = {x0.y, x0.w, x1.y, x1.w, x2.y, x2.w, x3.y, x3.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint32_t l = (w[i] & 0x0F0F0F0Fu) ^ 0x08080808u;
    uint32_t h = (w[i] & 0xF0F0F0F0u) ^ 0x80808080u;
    int lo2, hi2;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(lo2) : "r"(l), "r"(xe[i]), "r"(lo));
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(hi2) : "r"(h), "r"(xo[i]), "r"(hi));
    lo = lo2;
    hi = hi2;
  }
}

// t[(trow + local_row) * G + g] for every (row, group) of the segments.
// segs/T live in shared memory; total_rows = seg_finalize(). Ends with a
// __syncthreads, after which T is complete. One instance per K, shared by every
// stage (not inlined: the code a layer executes has to stay resident in the
// instruction cache).
// (nvcc 12.9 crashes on the non-inlined template with -lineinfo in one translation
// unit; that unit defines AINFER_BLOCK_DOT_INLINE.)
#ifdef AINFER_BLOCK_DOT_INLINE
#define AINFER_BLOCK_DOT_LINKAGE __device__ __forceinline__
#else
#define AINFER_BLOCK_DOT_LINKAGE static __device__ __noinline__
#endif
template <int K>
AINFER_BLOCK_DOT_LINKAGE void block_dot(const RowSeg *segs, int nseg, int total_rows,
                                              const StagedAct4 &act, float *T) {
  constexpr int HPR = K / 64, G = K / 128;
  constexpr int NTHR = 256, RPI = NTHR / HPR;  // rows per block iteration
  static_assert(NTHR % HPR == 0, "K/64 must divide the block size");
  const int hc = threadIdx.x % HPR, rt = threadIdx.x / HPR;
#pragma unroll 1
  for (int base = 0; base < total_rows; base += RPI * kDotLD) {
    uint32_t w[kDotLD][8];
    float sc[kDotLD];
    int meta[kDotLD];  // (t index << 4) | vector, or -1
    int s = 0;
    // ---- issue every load of this batch ----
#pragma unroll
    for (int j = 0; j < kDotLD; ++j) {
      const int r = base + j * RPI + rt;
      if (r < total_rows) {
        while (s + 1 < nseg && r >= segs[s + 1].row0) ++s;
        const int lr = r - segs[s].row0;
        ldg_stream32(segs[s].P + ((size_t)lr * HPR + hc) * 32, w[j]);
        sc[j] = (hc & 1) == 0 ? bf16_to_f32(__ldg(segs[s].S + (size_t)lr * G + (hc >> 1))) : 0.0f;
        meta[j] = (((segs[s].trow + lr) * G + (hc >> 1)) << 4) | segs[s].vec;
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) w[j][q] = 0x88888888u;
        sc[j] = 0.0f;
        meta[j] = -1;
      }
    }
    // ---- group sums: two lanes (hc even/odd) hold one group ----
#pragma unroll
    for (int j = 0; j < kDotLD; ++j) {
      const int vec = meta[j] < 0 ? 0 : (meta[j] & 15);
      const uint4 *xv = act.x + (size_t)vec * 4 * HPR + hc;
      int lo = 0, hi = 0;
      dot64_biased(w[j], xv[0], xv[HPR], xv[2 * HPR], xv[3 * HPR], lo, hi);
      int d = lo + (hi >> 4);
      d += __shfl_xor_sync(kFull, d, 1);
      if ((hc & 1) == 0 && meta[j] >= 0) {
        const int gi = vec * G + (hc >> 1);
        float v = (float)(d - 8 * act.gsum[gi]) * sc[j];
        T[meta[j] >> 4] = v * act.sq[gi];
      }
    }
  }
  __syncthreads();
}

// Sum of one row's group terms in ascending group order.
template <int K>
__device__ __forceinline__ float row_sum(const float *T, int trow) {
  constexpr int G = K / 128;
  const float *t = T + (size_t)trow * G;
  float acc = 0.0f;
#pragma unroll
  for (int g = 0; g < G; ++g) acc = acc + t[g];
  return acc;
}

}  // namespace ainfer
