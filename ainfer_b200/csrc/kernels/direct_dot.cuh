// direct_dot(): the t[][] terms of every (row, group) of a segment list, like
// block_dot(), for SHORT streams (a few tens of KB per block). The weights go
// from global memory straight to registers: every thread takes (row, group)
// tasks of 64 bytes (one INT4 group), consecutive threads consecutive groups, so
// a warp reads 2 KB of contiguous weights per task round, and a thread has all
// its loads of a round in flight before it uses the first. Compared with the
// shared-memory ring this has no copy-issue cost, no barrier round trips and a
// much shorter prologue, which is what bounds a kernel whose whole share is two
// or three tiles; the ring stays the path for long streams (the LM head), where
// its deeper buffering wins.
//
// Arithmetic is that of block_dot(): exact int32 sum over the group's 128
// products, >> 4 (the nibbles are used as 16*v), times the bf16 group scale,
// times the activation group scale, stored to t[g][trow + local row].
//
// Also here: the list builders and the activation quantiser in their
// all-threads forms (the one-thread forms cost microseconds of serial time).
#pragma once
#include "block_stages.cuh"

namespace ainfer {

// Per-translation-unit fault report for a weight pointer that cannot be read 16 bytes at a time.
__device__ __forceinline__ void direct_fault(uint32_t code) {
  if (g_stream_fault_word) *reinterpret_cast<volatile unsigned int *>(g_stream_fault_word) = code;
}

__device__ __forceinline__ uint4 ldg_stream16(const uint8_t *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Every thread calls; `cur` (shared memory) is complete and visible; the caller
// synchronises before T is read. U = tasks a thread keeps in flight per round.
template <int U>
__device__ __forceinline__ void direct_dot(const SegList *cur, const StagedAct4 &act, float *T) {
  const int K = cur->K, G = K >> 7, lg = 31 - __clz(G);
  const int ntask = cur->total << lg;
  const int TS = (kTCap >> lg) + 1;
  const int nthr = blockDim.x;
  int seg = 0, seg_end = cur->seg[0].row0 + cur->seg[0].nrows;
#pragma unroll 1
  for (int q0 = threadIdx.x; q0 < ntask; q0 += nthr * U) {
    uint4 w[U][4];
    uint32_t sraw[U];
    int tix[U], xg[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int q = q0 + u * nthr;
      sraw[u] = 0;
      tix[u] = -1;
      xg[u] = 0;
      if (q < ntask) {
        const int frow = q >> lg, g = q & (G - 1);
        while (frow >= seg_end) {
          ++seg;
          seg_end = cur->seg[seg].row0 + cur->seg[seg].nrows;
        }
        const RowSeg &sg = cur->seg[seg];
        const int lr = frow - sg.row0;
        const uint8_t *p = sg.P + (size_t)lr * (K >> 1) + (g << 6);
        if (reinterpret_cast<uintptr_t>(p) & 15u) {  // report and skip, as the ring does
          direct_fault(2);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) w[u][j] = ldg_stream16(p + 16 * j);
          sraw[u] = __ldg(sg.S + (size_t)lr * G + g);
          tix[u] = g * TS + sg.trow + lr;
          xg[u] = sg.vec * G + g;  // activation group index: vector, group
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (tix[u] >= 0) {
        const int vec = xg[u] >> lg, g = xg[u] & (G - 1);
        const uint4 *xv = act.x + (size_t)vec * 8 * G + g;
        int d0 = 0, d1 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 xe = xv[(2 * j) * G], xo = xv[(2 * j + 1) * G];
          d0 = dot16_x16(w[u][j], 0, xe, d0);
          d1 = dot16_x16(w[u][j], 1, xo, d1);
        }
        const float v = (float)((d0 + d1) >> 4) * __uint_as_float(sraw[u] << 16);
        T[tix[u]] = v * act.sq[xg[u]];
      }
    }
  }
}

// ---- segment lists written by many threads at once (every thread calls; the
// ---- caller synchronises before the list is read) ----
__device__ __forceinline__ void seglist_header(SegList *l, int nseg, int K, int total) {
  const int rpi = kTileBytes * 2 / K;
  l->nseg = nseg;
  l->K = K;
  l->total = total;
  l->ntiles = (total + rpi - 1) / rpi;
}

// Table of matrices, global rows [sb, se): thread i takes matrix i.
__device__ __forceinline__ void gemv_list_par(SegList *l, const GemvMat *smats, int nmats, int K, int sb, int se) {
  const int i = threadIdx.x;
  if (i < nmats) {
    const int G = K >> 7;
    int idx = 0, cnt = 0;
    for (int j = 0; j < nmats; ++j) {
      const int a = sb > smats[j].row_start ? sb : smats[j].row_start;
      const int b = se < smats[j].row_start + smats[j].N ? se : smats[j].row_start + smats[j].N;
      if (a < b) {
        if (j < i) ++idx;
        ++cnt;
      }
    }
    const int a = sb > smats[i].row_start ? sb : smats[i].row_start;
    const int b = se < smats[i].row_start + smats[i].N ? se : smats[i].row_start + smats[i].N;
    if (a < b && idx < kMaxSegs) {
      RowSeg &s = l->seg[idx];
      s.P = smats[i].P + (size_t)(a - smats[i].row_start) * (K >> 1);
      s.S = smats[i].S + (size_t)(a - smats[i].row_start) * G;
      s.nrows = b - a;
      s.vec = 0;
      s.trow = a - sb;
      s.row0 = a - sb;
    }
    if (i == 0) seglist_header(l, cnt < kMaxSegs ? cnt : kMaxSegs, K, se > sb ? se - sb : 0);
  }
}

// Gate and up segments of pair rows [sb, se): thread j takes segment j (slot s0 + j/2, gate or up).
__device__ __forceinline__ void gateup_list_par(SegList *l, const ExpertGateUpArgs &a, const ExpertW *sew, int sb,
                                                int se) {
  const int K = a.H, G = K >> 7, SB = gateup_sub_rows(K);
  const int j = threadIdx.x;
  if (se <= sb) {
    if (j == 0) seglist_header(l, 0, K, 0);
    return;
  }
  const int s0 = sb / a.I, s1 = (se - 1) / a.I;
  int nseg = 2 * (s1 - s0 + 1);
  if (nseg > kMaxSegs) nseg = kMaxSegs;
  if (j < nseg) {
    const int s = s0 + (j >> 1);
    const int aa = sb > s * a.I ? sb : s * a.I;
    const int bb = se < (s + 1) * a.I ? se : (s + 1) * a.I;
    const ExpertW &ew = sew[s];
    const size_t r0 = (size_t)(aa - s * a.I);
    RowSeg &d = l->seg[j];
    const bool up = j & 1;
    d.P = (up ? ew.uP : ew.gP) + r0 * (K >> 1);
    d.S = (up ? ew.uS : ew.gS) + r0 * G;
    d.nrows = bb - aa;
    d.vec = 0;
    d.trow = (up ? SB : 0) + (aa - sb);
    d.row0 = 2 * (aa - sb) + (up ? bb - aa : 0);
  }
  if (j == 0) seglist_header(l, nseg, K, 2 * (se - sb));
}

// One segment per slot over output rows [sb, se): thread s takes slot s.
__device__ __forceinline__ void down_list_par(SegList *l, const ExpertDownCombineArgs &a, const ExpertW *sew, int sb,
                                              int se) {
  const int K = a.I, G = K >> 7, nr = se > sb ? se - sb : 0;
  const int s = threadIdx.x;
  const int nseg = nr > 0 ? (a.slots < kMaxSegs ? a.slots : kMaxSegs) : 0;
  if (s < nseg) {
    const ExpertW &ew = sew[s];
    RowSeg &d = l->seg[s];
    d.P = ew.dP + (size_t)sb * (K >> 1);
    d.S = ew.dS + (size_t)sb * G;
    d.nrows = nr;
    d.vec = s;
    d.trow = s * nr;
    d.row0 = s * nr;
  }
  if (s == 0) seglist_header(l, nseg, K, nseg * nr);
}

// Quantises M fp32 vectors of K (global memory, per-128 activation quantiser,
// tools/cmdlist/kernels.cpp:551-579) into the staged form. One warp per group and
// load instruction (32 lanes x 16 bytes = the group's 512 contiguous bytes), up to
// eight groups per warp in flight at once (64 groups per pass of a 256-thread
// block). Split in two so that a caller can issue the loads of the first pass
// together with its other independent loads and do the arithmetic while
// dependent loads are in flight (a warp issues in order: a load placed after the
// first use of an earlier load's result waits a round trip longer).
struct QuantWide {
  float4 v[8];  // v[r]: this lane's four values of group (pass base) + warp + 8 r
};
__device__ __forceinline__ void quant_wide_load(QuantWide &q, const float *x, int K, int M, long x_stride, int gi0) {
  const int G = K >> 7, lg = 31 - __clz(G);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int gi = gi0 + warp + nw * r;
    q.v[r] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (gi < M * G) {
      const int m = gi >> lg, g = gi & (G - 1);
      q.v[r] = __ldcg(reinterpret_cast<const float4 *>(x + (size_t)m * x_stride + (size_t)g * 128) + lane);
    }
  }
}
// All 32 lanes of a warp call (shuffles inside).
__device__ __forceinline__ void quant_wide_store(const QuantWide &q, unsigned char *smem, int K, int M, int gi0) {
  uint32_t *xw = reinterpret_cast<uint32_t *>(smem);
  const int G = K >> 7, lg = 31 - __clz(G);
  float *sqs = reinterpret_cast<float *>(smem + (size_t)M * K);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  float mx[8];
#pragma unroll
  for (int r = 0; r < 8; ++r)
    mx[r] = fmaxf(fmaxf(fabsf(q.v[r].x), fabsf(q.v[r].y)), fmaxf(fabsf(q.v[r].z), fabsf(q.v[r].w)));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
#pragma unroll
    for (int r = 0; r < 8; ++r) mx[r] = fmaxf(mx[r], __shfl_xor_sync(kFull, mx[r], off));
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int gi = gi0 + warp + nw * r;
    float s = mx[r] / 127.0f;
    if (s == 0.0f) s = 1.0f;
    const float ri = quant_recip(s);
    const int q0 = quant_round_r(q.v[r].x, s, ri), q1 = quant_round_r(q.v[r].y, s, ri),
              q2 = quant_round_r(q.v[r].z, s, ri), q3 = quant_round_r(q.v[r].w, s, ri);
    const uint32_t own = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) |
                         ((uint32_t)(q3 & 0xFF) << 24);
    const uint32_t other = __shfl_xor_sync(kFull, own, 1);
    if (gi < M * G) {
      const int m = gi >> lg, g = gi & (G - 1);
      const int pc = g * 16 + (lane >> 1);  // 8-value piece: two lanes of four values each
      if (lane & 1) xw[staged4_word(K, m, pc, 1)] = __byte_perm(other, own, 0x7531);
      else xw[staged4_word(K, m, pc, 0)] = __byte_perm(own, other, 0x6420);
      if (lane == 0) sqs[gi] = s;
    }
  }
}
// Rolled form for a contiguous [M][K] fp32 source of at most 8192 values: the block copies the
// values to shared memory (`raw`, M*K floats; all loads of a thread in flight at once), then
// each warp walks its groups in a rolled loop. Far less distinct code than the register form
// above, which matters for a kernel that runs once per layer with a cold instruction cache.
struct RawCopy {
  float4 v[8];
};
__device__ __forceinline__ void raw_copy_load(RawCopy &c, const float *x, int count4) {
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int i = threadIdx.x + u * 256;
    c.v[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (i < count4) c.v[u] = __ldcg(reinterpret_cast<const float4 *>(x) + i);
  }
}
__device__ __forceinline__ void raw_copy_store(const RawCopy &c, float *raw, int count4) {
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int i = threadIdx.x + u * 256;
    if (i < count4) reinterpret_cast<float4 *>(raw)[i] = c.v[u];
  }
}
// After raw_copy_store and a block barrier; ends with a block barrier.
__device__ __forceinline__ StagedAct4 quant_rolled(unsigned char *smem, const float *raw, int K, int M) {
  uint32_t *xw = reinterpret_cast<uint32_t *>(smem);
  const int G = K >> 7, lg = 31 - __clz(G);
  float *sqs = reinterpret_cast<float *>(smem + (size_t)M * K);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
#pragma unroll 1
  for (int gi = warp; gi < M * G; gi += nw) {
    const float4 v = reinterpret_cast<const float4 *>(raw + (size_t)gi * 128)[lane];
    float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    mx = warp_max(mx);
    float s = mx / 127.0f;
    if (s == 0.0f) s = 1.0f;
    const float ri = quant_recip(s);
    const int q0 = quant_round_r(v.x, s, ri), q1 = quant_round_r(v.y, s, ri), q2 = quant_round_r(v.z, s, ri),
              q3 = quant_round_r(v.w, s, ri);
    const uint32_t own = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) |
                         ((uint32_t)(q3 & 0xFF) << 24);
    const uint32_t other = __shfl_xor_sync(kFull, own, 1);
    const int m = gi >> lg, g = gi & (G - 1);
    const int pc = g * 16 + (lane >> 1);
    if (lane & 1) xw[staged4_word(K, m, pc, 1)] = __byte_perm(other, own, 0x7531);
    else xw[staged4_word(K, m, pc, 0)] = __byte_perm(own, other, 0x6420);
    if (lane == 0) sqs[gi] = s;
  }
  __syncthreads();
  return StagedAct4{reinterpret_cast<const uint4 *>(smem), sqs};
}

// The passes after the first (M*G > 64 groups), then the block barrier.
__device__ __forceinline__ StagedAct4 quant_wide_finish(unsigned char *smem, const float *x, int K, int M,
                                                       long x_stride) {
  const int G = K >> 7, per_pass = (blockDim.x >> 5) * 8;
#pragma unroll 1
  for (int gi0 = per_pass; gi0 < M * G; gi0 += per_pass) {
    QuantWide q;
    quant_wide_load(q, x, K, M, x_stride, gi0);
    quant_wide_store(q, smem, K, M, gi0);
  }
  __syncthreads();
  return StagedAct4{reinterpret_cast<const uint4 *>(smem), reinterpret_cast<float *>(smem + (size_t)M * K)};
}

}  // namespace ainfer
