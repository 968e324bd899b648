// Block-level INT4 (group 128) x INT8 dot over a list of row segments, fed by
// the weight ring (weight_ring.cuh).
//
// Unless its inner loop is lean the kernel is bound by instruction issue, not
// by HBM: at 6.5 TB/s an SM receives 16 bytes of weights every 0.7 cycles,
// which leaves about 90 thread instructions per 16 bytes at perfect issue.
//   * a lane owns HALF a group: 32 contiguous bytes = 64 weights of a tile that
//     a bulk copy has put in shared memory; it moves them into registers and
//     releases the stage at once;
//   * the lane's 64 activations, the group's activation sum and scale stay in
//     registers for as long as consecutive tiles use the same staged vector;
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
// Lane tid of the block holds bytes [32*tid, 32*tid+32) of a tile: row
// tid / HPR of the tile, half-group hc = tid % HPR (HPR = K/64 divides 256).
#pragma once
#include "common.cuh"
#include "weight_ring.cuh"

namespace ainfer {

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

// sum over 64 weights of (nibble ^ 8) * x: low nibbles exactly, high nibbles as 16*(n^8).
__device__ __forceinline__ void dot64_biased(const uint4 &wa, const uint4 &wb, const uint4 (&x)[4], int &lo,
                                             int &hi) {
  const uint32_t w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
  const uint32_t xe[8] = {x[0].x, x[0].z, x[1].x, x[1].z, x[2].x, x[2].z, x[3].x, x[3].z};
  const uint32_t xo[8] = {x[0].y, x[0].w, x[1].y, x[1].w, x[2].y, x[2].w, x[3].y, x[3].w};
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

// t[(trow + local_row) * G + g] for every (row, group) of the list `cur`.
// cur/next/ring/T live in shared memory and cur->ntiles is final. While it
// consumes, the issuing thread keeps the ring full, running on into `next`
// (the list of the following call, any K; may be null) once `cur` is fully
// issued. Ends with a __syncthreads, after which T is complete and every tile
// of `cur` has been consumed. One instance per K, shared by every stage (not
// inlined: the code a layer executes has to stay resident in the instruction
// cache).
// (nvcc 12.9 crashes on the non-inlined template with -lineinfo in one translation
// unit; that unit defines AINFER_BLOCK_DOT_INLINE.)
#ifdef AINFER_BLOCK_DOT_INLINE
#define AINFER_BLOCK_DOT_LINKAGE __device__ __forceinline__
#else
#define AINFER_BLOCK_DOT_LINKAGE static __device__ __noinline__
#endif
template <int K>
AINFER_BLOCK_DOT_LINKAGE void block_dot(Ring *ring, const SegList *cur, const SegList *next,
                                        const StagedAct4 &act, float *T) {
  constexpr int HPR = K / 64, G = K / 128;
  constexpr int NTHR = 256, RPI = NTHR / HPR;  // rows per tile
  static_assert(NTHR % HPR == 0, "K/64 must divide the block size");
  const int tid = threadIdx.x, hc = tid % HPR, rt = tid / HPR;
  const uint32_t nst = ring->nst;
  unsigned char *const data = ring->data;
  uint32_t cs = ring->c_stage, cph = ring->c_phase;
  const int ntiles = cur->ntiles;
  const bool even = (hc & 1) == 0;

  // ---- issuing thread: fill the ring ----
  Producer pr;
  uint32_t issued = 0;  // tiles issued, counted from tile 0 of cur (runs on into next)
  uint32_t ntot = (uint32_t)ntiles;
  bool in_next = false;
  if (tid == 0) {
    if (next) ntot += (uint32_t)next->ntiles;
    pr.stage = cs;
    pr.phase = cph;
    if (ntiles > 0) pr.open(cur);
    else if (next) { pr.open(next); in_next = true; }
    for (; issued < ring->pre; ++issued) {
      pr.skip();
      pr.next_stage(nst);
    }
    const uint32_t cap = ntot < nst ? ntot : nst;
    const uint32_t first = issued;
    for (; issued < cap; ++issued) {
      if (!in_next && issued == (uint32_t)ntiles) { pr.open(next); in_next = true; }
      pr.issue(ring, data, nst);
    }
    ring->issued += issued - first;
  }

  // ---- consume ----
  int seg = 0, r0 = 0;  // segment and first row of the current tile
  int nrows = 0, vec = -1;
  bool s_aligned = false;
  const uint16_t *sglob = nullptr;  // this lane's scale in global memory, row 0 of the segment
  float *tp = nullptr;              // this lane's T entry, row 0 of the segment
  uint4 x[4];
  int gs8 = 0;
  float sqg = 0.0f;
  const unsigned char *st = data + cs * kStageStride;
#pragma unroll 1
  for (int t = 0; t < ntiles; ++t) {
    if (r0 == 0) {  // first tile of a segment: block-uniform
      const RowSeg &sg = cur->seg[seg];
      nrows = sg.nrows;
      sglob = sg.S + (size_t)rt * G + (hc >> 1);
      s_aligned = (reinterpret_cast<uintptr_t>(sg.S) & 15u) == 0;
      tp = T + (size_t)(sg.trow + rt) * G + (hc >> 1);
      if (sg.vec != vec) {
        vec = sg.vec;
        const uint4 *xv = act.x + (size_t)vec * 4 * HPR + hc;
        x[0] = xv[0]; x[1] = xv[HPR]; x[2] = xv[2 * HPR]; x[3] = xv[3 * HPR];
        gs8 = 8 * act.gsum[vec * G + (hc >> 1)];
        sqg = act.sq[vec * G + (hc >> 1)];
      }
    }
    const int rows = nrows - r0 < RPI ? nrows - r0 : RPI;
    const bool live = even && rt < rows;
    mbar_wait(ring, &ring->full[cs], cph);
    const uint4 wa = *reinterpret_cast<const uint4 *>(st + tid * 32);
    const uint4 wb = *reinterpret_cast<const uint4 *>(st + tid * 32 + 16);
    uint32_t sraw = 0;
    if (live) {
      if (s_aligned && ((rows * G * 2) & 15) == 0) sraw = reinterpret_cast<const uint16_t *>(st + kTileBytes)[tid >> 1];
      else sraw = __ldg(sglob + (size_t)r0 * G);
    }
    __syncwarp();
    if ((tid & 31) == 0) mbar_arrive(&ring->empty[cs]);
    // the issuing thread refills the stage of the previous tile
    if (tid == 0 && t >= 1 && issued < ntot) {
      const uint32_t ps = cs == 0 ? nst - 1 : cs - 1, pph = cs == 0 ? cph ^ 1u : cph;
      mbar_wait(ring, &ring->empty[ps], pph);
      if (!in_next && issued == (uint32_t)ntiles) { pr.open(next); in_next = true; }
      pr.issue(ring, data, nst);
      ++issued;
      ring->issued += 1;
    }
    int lo = 0, hi = 0;
    dot64_biased(wa, wb, x, lo, hi);
    int d = lo + (hi >> 4);
    d += __shfl_xor_sync(kFull, d, 1);
    if (live) {
      float v = (float)(d - gs8) * __uint_as_float(sraw << 16);
      tp[(size_t)r0 * G] = v * sqg;
    }
    r0 += RPI;
    if (r0 >= nrows) {
      ++seg;
      r0 = 0;
    }
    st += kStageStride;
    if (++cs == nst) {
      cs = 0;
      cph ^= 1u;
      st = data;
    }
  }
  if (tid == 0) {
    ring->c_stage = cs;
    ring->c_phase = cph;
    ring->pre = issued > (uint32_t)ntiles ? issued - (uint32_t)ntiles : 0;
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
