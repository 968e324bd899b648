// Block-level INT4 (group 128) x INT8 dot over a list of row segments, fed by
// the weight ring (weight_ring.cuh).
//
// On B200 the kernel is bound by the integer pipe, not by HBM, unless its inner
// loop is lean: at 6.5 TB/s an SM receives a 16 KB tile every ~710 cycles and
// the integer pipe retires 64 lane-operations per cycle, so a tile may cost at
// most ~180 integer operations per thread (64 of them are the dp4a and masks). The loop is built around that:
//   * a lane owns a WHOLE group of a row: 64 contiguous bytes = 128 weights of a
//     16 KB tile that a bulk copy has put in shared memory. It moves them into
//     registers (four 16-byte reads in a lane-rotated order that keeps every
//     quarter-warp on distinct banks) and releases the stage at once (one
//     arrival per warp);
//   * the lane's 128 activations and their scale stay in registers for as long
//     as consecutive tiles use the same staged vector;
//   * nibbles are two's complement, so a nibble moved to the top of its byte IS
//     the signed byte 16*v: high nibbles are masked in place, low nibbles are
//     shifted by a multiply (which runs on the other arithmetic pipe) and
//     masked; both feed signed dp4a and the sum is divided by 16 at the end
//     (exact: it is a multiple of 16). No bias term, no shuffle;
//   * the lane stores t[g][row] = ((float)group_sum * weight_scale) * act_scale[g];
//   * after one __syncthreads a single thread per row adds t[row][0..G) in
//     ascending group order (the reference's accumulation order,
//     tools/cmdlist/kernels.cpp:157-191) and runs the row's epilogue.
// Integer sums are associative and the fp32 sum keeps the reference order, so
// results are bit-identical to the one-work-item-per-row loop.
//
// Lane l (0..255) of the block holds bytes [64*l, 64*l+64) of a tile: row
// l / G of the tile, group l % G (G = K/128 divides 256).
#pragma once
#include "common.cuh"
#include "weight_ring.cuh"

namespace ainfer {

// Staged activations, group-major layout: for vector v, group g and q in 0..7
// the uint4 x[(v*8 + q) * G + g] holds the de-interleaved INT8 bytes of weights
// g*128 + 16q .. +15: {even(0..7), odd(0..7), even(8..15), odd(8..15)} where
// even = bytes (x0,x2,x4,x6), odd = (x1,x3,x5,x7) of an 8-weight word. Lanes of
// a warp own consecutive groups, so their 16-byte reads are conflict-free.
struct StagedAct4 {
  const uint4 *x;
  const float *sq;   // [M][K/128] activation scales
};
__host__ __device__ inline uint32_t staged4_bytes(int K, int M) {
  return (uint32_t)((size_t)M * K + (size_t)M * (K / 128) * 4);
}
// word index (in 32-bit words) of 8-weight piece pc of vector v, parity 0 even / 1 odd
__device__ __forceinline__ int staged4_word(int K, int v, int pc, int parity) {
  const int G = K / 128;
  int g = pc >> 4, i = pc & 15;
  return (((v * 8 + (i >> 1)) * G + g) << 2) + ((i & 1) << 1) + parity;
}

// Stages M natural-order INT8 vectors (global memory) with their fp32 group scales.
__device__ __forceinline__ StagedAct4 stage4(unsigned char *smem, const int8_t *xq, const float *sq, int K,
                                             int M, long xq_stride, long sq_stride) {
  uint32_t *xw = reinterpret_cast<uint32_t *>(smem);
  const int G = K / 128;
  float *sqs = reinterpret_cast<float *>(smem + (size_t)M * K);
  for (int i = threadIdx.x; i < M * (K / 8); i += blockDim.x) {
    int m = i / (K / 8), pc = i % (K / 8);
    uint2 v = __ldcg(reinterpret_cast<const uint2 *>(xq + m * xq_stride + (long)pc * 8));
    xw[staged4_word(K, m, pc, 0)] = __byte_perm(v.x, v.y, 0x6420);
    xw[staged4_word(K, m, pc, 1)] = __byte_perm(v.x, v.y, 0x7531);
  }
  for (int i = threadIdx.x; i < M * G; i += blockDim.x) {
    int m = i / G, g = i % G;
    sqs[i] = __ldcg(sq + m * sq_stride + g);
  }
  __syncthreads();
  return StagedAct4{reinterpret_cast<const uint4 *>(smem), sqs};
}

// stage4() of one vector (K <= 8 * 256 * kPer) with every global load issued before
// `between()` runs and before the first shared-memory store: a caller puts a load
// that depends on something fetched earlier into `between`, so that it is in flight
// together with these instead of a round trip later (a warp issues in order).
template <class F>
__device__ __forceinline__ StagedAct4 stage4_issue_first(unsigned char *smem, const int8_t *xq, const float *sq,
                                                        int K, F between) {
  constexpr int kPer = 4;  // 8-byte pieces per thread: K <= 8192 with 256 threads
  uint32_t *xw = reinterpret_cast<uint32_t *>(smem);
  const int G = K / 128;
  float *sqs = reinterpret_cast<float *>(smem + (size_t)K);
  uint2 v[kPer];
  float sc = 0.0f;
#pragma unroll
  for (int r = 0; r < kPer; ++r) {
    const int pc = threadIdx.x + r * blockDim.x;
    if (pc < K / 8) v[r] = __ldcg(reinterpret_cast<const uint2 *>(xq + (long)pc * 8));
  }
  if (threadIdx.x < G) sc = __ldcg(sq + threadIdx.x);
  between();
#pragma unroll
  for (int r = 0; r < kPer; ++r) {
    const int pc = threadIdx.x + r * blockDim.x;
    if (pc < K / 8) {
      xw[staged4_word(K, 0, pc, 0)] = __byte_perm(v[r].x, v[r].y, 0x6420);
      xw[staged4_word(K, 0, pc, 1)] = __byte_perm(v[r].x, v[r].y, 0x7531);
    }
  }
  if (threadIdx.x < G) sqs[threadIdx.x] = sc;
  __syncthreads();
  return StagedAct4{reinterpret_cast<const uint4 *>(smem), sqs};
}

// Quantises one group of 128 fp32 values held four per lane (per-128 activation
// quantiser, tools/cmdlist/kernels.cpp:551-579) into the staged form. One warp;
// one out-of-line copy of this code however many loops call it.
static __device__ __noinline__ void quant_group_staged(uint32_t *xw, float *sqs, int K, int m, int g, float4 v) {
  const int lane = threadIdx.x & 31;
  float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
  mx = warp_max(mx);
  float s = mx / 127.0f;
  if (s == 0.0f) s = 1.0f;
  int q0 = quant_round(v.x, s), q1 = quant_round(v.y, s), q2 = quant_round(v.z, s), q3 = quant_round(v.w, s);
  uint32_t own = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) |
                 ((uint32_t)(q3 & 0xFF) << 24);
  uint32_t other = __shfl_xor_sync(kFull, own, 1);
  int pc = g * 16 + (lane >> 1);  // 8-weight piece: two lanes of 4 weights each
  if (lane & 1) xw[staged4_word(K, m, pc, 1)] = __byte_perm(other, own, 0x7531);
  else xw[staged4_word(K, m, pc, 0)] = __byte_perm(own, other, 0x6420);
  if (lane == 0) sqs[m * (K / 128) + g] = s;
}

// Quantises M fp32 vectors straight into the staged form, one warp per group.
// A global source is fetched four groups per warp at a time so that the loads
// overlap; a shared-memory source is simply walked.
template <bool kGlobalSrc>
__device__ __forceinline__ StagedAct4 stage4_from_f32(unsigned char *smem, const float *x, int K, int M,
                                                      long x_stride) {
  uint32_t *xw = reinterpret_cast<uint32_t *>(smem);
  const int G = K / 128;
  float *sqs = reinterpret_cast<float *>(smem + (size_t)M * K);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (kGlobalSrc) {
    constexpr int kRB = 4;
#pragma unroll 1
    for (int i0 = warp; i0 < M * G; i0 += warps * kRB) {
      float4 vv[kRB];
#pragma unroll
      for (int r = 0; r < kRB; ++r) {
        const int i = i0 + r * warps;
        if (i < M * G)
          vv[r] = __ldcg(reinterpret_cast<const float4 *>(x + (i / G) * x_stride + (long)(i % G) * 128 + lane * 4));
      }
#pragma unroll
      for (int r = 0; r < kRB; ++r) {
        const int i = i0 + r * warps;
        if (i < M * G) quant_group_staged(xw, sqs, K, i / G, i % G, vv[r]);
      }
    }
  } else {
#pragma unroll 1
    for (int i = warp; i < M * G; i += warps) {
      const float4 v = *reinterpret_cast<const float4 *>(x + (i / G) * x_stride + (long)(i % G) * 128 + lane * 4);
      quant_group_staged(xw, sqs, K, i / G, i % G, v);
    }
  }
  __syncthreads();
  return StagedAct4{reinterpret_cast<const uint4 *>(smem), sqs};
}

// t[][] scratch of a block: kTCap (row, group) terms, stored GROUP-major with a row stride
// of kTCap/G + 1 floats: t[g * (kTCap/G + 1) + row]. The lanes of a warp (consecutive
// groups of two rows) then write with at most a 2-way bank conflict, and the finishing
// threads (consecutive rows) read each group's term conflict-free.
constexpr int kTCap = 4096;
constexpr int kTFloats = kTCap + 64;  // allocation: kTCap plus one padding float per group

// 32-bit shared-window loads and stores (no generic address arithmetic in the loop).
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// acc += 16 * sum over the 16 weights of two packed words of v*x, v the two's
// complement nibble: a nibble at the top of its byte is the signed byte 16*v.
// The low nibbles get there by a multiply by 16 (an integer multiply-add, which
// does not run on the pipe the logic and dot instructions share).
__device__ __forceinline__ int dot16_x16(const uint4 &w4, int which, const uint4 &x, int acc) {
  const uint32_t w0 = which == 0 ? w4.x : w4.z, w1 = which == 0 ? w4.y : w4.w;
  acc = __dp4a((int)((w0 * 16u) & 0xF0F0F0F0u), (int)x.x, acc);
  acc = __dp4a((int)(w0 & 0xF0F0F0F0u), (int)x.y, acc);
  acc = __dp4a((int)((w1 * 16u) & 0xF0F0F0F0u), (int)x.z, acc);
  acc = __dp4a((int)(w1 & 0xF0F0F0F0u), (int)x.w, acc);
  return acc;
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
template <int K, bool kRegCursor>
AINFER_BLOCK_DOT_LINKAGE void block_dot(Ring *ring, const SegList *cur, const SegList *next,
                                        const StagedAct4 &act, float *T) {
  constexpr int G = K / 128;
  constexpr int RPI = 256 / G;  // rows per tile
  static_assert(256 % G == 0 && G <= 256, "K/128 must divide 256");
  const int tid = threadIdx.x;
  const int g = tid % G, rt = tid / G;
  const bool warp_lead = (tid & 31) == 0;
  const uint32_t nst = ring->nst;
  const uint32_t data_a = smem_addr(ring->data), full_a = smem_addr(&ring->full[0]),
                 empty_a = smem_addr(&ring->empty[0]), T_a = smem_addr(T);
  uint32_t cs = ring->c_stage, cph = ring->c_phase;
  const int ntiles = cur->ntiles;
  // piece order of this lane: at step s it reads piece (s + (tid >> 1)) & 3 of its 64 bytes
  const int rot = (tid >> 1) & 3;
  const uint32_t lane_off = (uint32_t)tid * 64u;

  // ---- issuing: fill the ring ----
  // kRegCursor (streaming kernels): the tiles of this call and, towards its end, of the next
  // list form one sequence j = 0, 1, ...; tile j is issued by the leader of warp j % 8, so the
  // cost of issuing (two bulk copies, ~1100 cycles) rotates over the warps instead of sitting
  // on one warp's critical path for every tile. Otherwise (persistent step: a few prefetched
  // tiles per stage, small code wanted) thread 0 issues through the cursor kept in the Ring.
  // in_flight = tiles issued and not yet consumed (this call's and the next list's)
  uint32_t in_flight = 0;
  bool more = false;  // the cursor may still have tiles to issue
  const uint32_t warp = (uint32_t)tid >> 5;
  const uint32_t pre0 = ring->pre;
  const uint32_t ntot = (uint32_t)ntiles + (next ? (uint32_t)next->ntiles : 0u);
  const uint32_t fill = ntot < nst ? ntot : nst;  // tiles in flight after the initial fill
  if (kRegCursor) {
    if (warp_lead) {
      for (uint32_t j = pre0; j < fill; ++j) {
        if ((j & 7u) != warp) continue;
        uint32_t st = cs + j;
        if (st >= nst) st -= nst;
        if (j < (uint32_t)ntiles) ring_issue_tile(ring, cur, (int)j, st);
        else ring_issue_tile(ring, next, (int)(j - (uint32_t)ntiles), st);
      }
    }
  } else if (tid == 0) {
    in_flight = pre0;
    if (in_flight == 0) ring_open(ring, cur);
    ring->p_next = next;
    more = true;
    while (more && in_flight < nst) {
      more = ring_issue_next(ring);
      if (more) ++in_flight;
    }
  }
  AINFER_STAMP(50);
  // ---- consume ----
  // A tile holds RPI consecutive flat rows of the list; this lane's row of tile t is t*RPI + rt.
  const int total = cur->total;
  int f = rt;                 // flat row of this lane in the current tile
  int seg = 0, seg_lo = 0, seg_hi = 0, vec = -1;  // segment of this lane's row (cached bounds)
  const uint16_t *sseg = nullptr;  // scales of the cached segment
  uint32_t tseg = 0;               // shared address of t[trow of the cached segment][g]
  uint4 x[8];                      // x[2s], x[2s+1]: activations of the piece read at step s
  float sqg = 0.0f;
#pragma unroll 1
  for (int t = 0; t < ntiles; ++t, f += RPI) {
    const bool live = f < total;
    if (live && f >= seg_hi) {  // this lane's row entered another segment
      while (f >= cur->seg[seg].row0 + cur->seg[seg].nrows) ++seg;
      const RowSeg &sg = cur->seg[seg];
      seg_lo = sg.row0;
      seg_hi = sg.row0 + sg.nrows;
      sseg = sg.S;
      tseg = T_a + (uint32_t)((g * (kTCap / G + 1) + sg.trow) * 4);
      if (sg.vec != vec) {
        vec = sg.vec;
        const uint4 *xv = act.x + (size_t)vec * 8 * G + g;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          const int j = (s + rot) & 3;
          x[2 * s] = xv[(2 * j) * G];
          x[2 * s + 1] = xv[(2 * j + 1) * G];
        }
        sqg = act.sq[vec * G + g];
      }
    }
    // The stage of the previous tile is refilled BEFORE this tile's data is waited for: it has
    // been free since every warp copied tile t-1 out, and a refill that waited for tile t to
    // land would leave one stage of the ring idle all the time.
    if (kRegCursor) {
      const uint32_t j = (uint32_t)t - 1u + nst;  // the tile that takes the stage of tile t-1
      if (warp_lead && t >= 1 && j < ntot && (j & 7u) == warp) {
        const uint32_t ps = cs == 0 ? nst - 1 : cs - 1, pph = cs == 0 ? cph ^ 1u : cph;
        mbar_wait_a(ring, empty_a + ps * 8, pph);
        if (j < (uint32_t)ntiles) ring_issue_tile(ring, cur, (int)j, ps);
        else ring_issue_tile(ring, next, (int)(j - (uint32_t)ntiles), ps);
      }
    } else if (tid == 0) {
      if (t >= 1) --in_flight;  // tile t-1 has been consumed by this thread; the wait below covers the others
      if (more && t >= 1) {
        mbar_wait_a(ring, empty_a + ring->p_stage * 8, ring->p_phase ^ 1u);
        more = ring_issue_next(ring);
        if (more) ++in_flight;
      }
    }
    const uint32_t st = data_a + cs * kStageStride;
    AINFER_STAMP(51);
    mbar_wait_a(ring, full_a + cs * 8, cph);
    AINFER_STAMP(52);
    const uint32_t wbase = st + lane_off;
    const uint4 w0 = lds128(wbase + (uint32_t)((rot & 3) << 4)),
                w1 = lds128(wbase + (uint32_t)(((1 + rot) & 3) << 4)),
                w2 = lds128(wbase + (uint32_t)(((2 + rot) & 3) << 4)),
                w3 = lds128(wbase + (uint32_t)(((3 + rot) & 3) << 4));
    uint32_t sraw = 0;
    if (live) {
      // the piece of this lane's segment inside this tile, as the issuing thread cut it
      const int f0 = f - rt;
      const int pa = seg_lo > f0 ? seg_lo : f0, pb = seg_hi < f0 + RPI ? seg_hi : f0 + RPI;
      const uint16_t *psrc = sseg + (size_t)(pa - seg_lo) * G;
      if (piece_scales_bulk(psrc, (uint32_t)((pb - pa) * G * 2), (uint32_t)((pa - f0) * G * 2)))
        sraw = lds_u16(st + kTileBytes + tid * 2);
      else
        sraw = __ldg(sseg + (size_t)(f - seg_lo) * G + g);
    }
    __syncwarp();
    if (warp_lead) mbar_arrive_a(empty_a + cs * 8);
    int d0 = 0, d1 = 0;
    d0 = dot16_x16(w0, 0, x[0], d0);
    d1 = dot16_x16(w0, 1, x[1], d1);
    d0 = dot16_x16(w1, 0, x[2], d0);
    d1 = dot16_x16(w1, 1, x[3], d1);
    d0 = dot16_x16(w2, 0, x[4], d0);
    d1 = dot16_x16(w2, 1, x[5], d1);
    d0 = dot16_x16(w3, 0, x[6], d0);
    d1 = dot16_x16(w3, 1, x[7], d1);
    if (live) {
      const float v = (float)((d0 + d1) >> 4) * __uint_as_float(sraw << 16);
      sts_f32(tseg + (uint32_t)((f - seg_lo) * 4), v * sqg);
    }
    if (++cs == nst) {
      cs = 0;
      cph ^= 1u;
    }
    AINFER_STAMP(53);
  }
  if (tid == 0) {
    ring->c_stage = cs;
    ring->c_phase = cph;
    if (kRegCursor) {
      // issued in total, counted from tile 0 of cur: the initial fill, then one per consumed tile but the last
      uint32_t last = (ntiles >= 1 ? (uint32_t)ntiles - 1u : 0u) + nst;
      if (last > ntot) last = ntot;
      const uint32_t total_issued = last > fill ? last : fill;
      ring->issued += total_issued - pre0;
      ring->pre = total_issued > (uint32_t)ntiles ? total_issued - (uint32_t)ntiles : 0;
    } else {
      // what is still in flight belongs to the next list (the last tile of cur was consumed above)
      ring->pre = ntiles > 0 ? in_flight - 1 : in_flight;
    }
  }
  __syncthreads();
}

// Sum of one row's group terms in ascending group order.
template <int K>
__device__ __forceinline__ float row_sum(const float *T, int trow) {
  constexpr int G = K / 128, TS = kTCap / G + 1;
  const float *t = T + trow;
  float acc = 0.0f;
#pragma unroll
  for (int g = 0; g < G; ++g) acc = acc + t[g * TS];
  return acc;
}

}  // namespace ainfer
