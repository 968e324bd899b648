// DecodeStep: one whole decode token in ONE persistent cooperative launch, one block per SM.
//
// The recorded list replays hundreds of small dependent launches per token and is bound by
// their latency, not by HBM. Here the blocks stay resident for the whole token and the work
// is split between two kinds of warps:
//   * one PRODUCER warp per block streams every weight byte the block will need, in the order
//     it will need it, from HBM into a ring of 16 KB shared-memory tiles with bulk
//     asynchronous copies (cp.async.bulk, completion on an mbarrier). It runs ahead of the
//     consumers across stage and layer boundaries, limited only by ring space, and stops only
//     where the addresses depend on data (the routed experts), until the consumers have
//     selected them;
//   * sixteen CONSUMER warps run the stages of a layer, separated by grid-wide barriers:
//     each stage takes its activations from global memory (L2), its weights from the ring,
//     and writes its outputs back to global memory for the next stage.
// So HBM traffic is decoupled from the dependency chain: while the consumers wait at a
// barrier, the next stages' weights are already landing in shared memory.
//
// Stages of a Gated DeltaNet layer (tools/decode/decode_l0.cpp:610-674 in the reference):
//   1 norm + quantiser, in_proj qkv/z/b/a GEMV with conv / sigmoid / decay epilogues
//   2 gated delta rule step (state in registers, read once and written once)
//   3 gated per-head norm + quantiser, out_proj GEMV + residual
//   4 post norm + quantiser, router logits
//   5 softmax top-k (every block selects for itself), expert gate/up GEMV + SiLU-mul
//   6 quantiser, expert down GEMV, rank-ordered combine + residual
// Stages of a gated attention layer (decode_l0.cpp:560-608): 1 q/k/v GEMV, 2 head norm + RoPE
// + INT8 KV append + one 64-token chunk of attention per block, 3 ordered merge of the chunk
// partials + sigmoid gate + quantiser, 4 o_proj + residual, then 4-6 of the above.
// The tail is final norm, LM head, first-max-wins argmax and the control-block update.
//
// The arithmetic of every stage (operation order, reduction shapes) is that of the stand-alone
// kernels in this directory, so the two paths give bit-identical results.
//
// Every wait (mbarrier, grid barrier) is bounded by a wall-clock limit: when one runs out the
// block sets the plan's sticky error word, no wait in the grid spins again, and the kernel
// terminates with garbage results that the host refuses (the error word is read after the step).
#include "../common/step_plan.h"
#include "attention_core.cuh"
#include "block_stages.cuh"
#include "deltanet_core.cuh"
#include "gemv_stage.cuh"
#include "moe_core.cuh"
#include "tail_core.cuh"

namespace ainfer {

struct DecodeStepArgs {
  const StepPlan *plan;  // device copy of the plan (the kernel keeps its own copy in shared memory)
  int32_t mode;  // 1: final norm + lm_head + argmax, control advances to the selected token
                 // 0: prompt step, control advances to ids[position + 1]
};

constexpr int kCons = 512;          // consumer threads (16 warps)
constexpr int kStepThreads = 544;   // consumers + the producer warp
constexpr int kNT = 10;             // ring tiles
constexpr int kTileStride = kTileBytes + kTileScaleBytes;
// Limit of any single wait, in SM clock cycles (about two seconds). The waits are timed with the
// SM's own cycle counter: reading the global nanosecond timer takes about a microsecond, far too
// long for a poll loop that usually succeeds within a few hundred nanoseconds.
constexpr long long kWaitCycles = 4000000000ll;

// ---- shared-memory map (all dynamic) ----
constexpr int kHdrBytes = 5120;                 // StepShared
constexpr int kActBytes = 8704;                 // staged INT8 activations (<= 8192) + group scales (<= 512)
constexpr int kFbufFloats = 8192;               // fp32 scratch: norm input, O|Z, Act, KV chunk
constexpr int kActOff = kHdrBytes;
constexpr int kFbufOff = kActOff + kActBytes;
constexpr int kTOff = kFbufOff + kFbufFloats * 4;
constexpr int kRingOff = (kTOff + kTFloats * 4 + 127) / 128 * 128;
constexpr int kStepSmemBytes = kRingOff + kNT * kTileStride;
static_assert(kStepSmemBytes <= 232448, "shared memory of one SM");

// Contiguous rows of one matrix, as the producer streams them.
struct Seg {
  const uint8_t *P;   // first row's bytes
  const uint8_t *S;   // first row's scales (null: none)
  int32_t nrows, vec, trow, pad;
};
constexpr int kMaxSegs2 = 24;

struct StepShared {
  // the members that are copied 16 bytes at a time come first (the struct sits at a
  // 128-byte aligned address and the sizes are multiples of 16)
  StepPlan plan;                // the plan: read from here, not from global memory, by every stage
  StepLayer ly;                 // the current layer's record
  ExpertW sew[12];              // weight pointers of the selected expert slots
  unsigned long long full[kNT], empty[kNT];
  unsigned long long sel_bar;   // consumers -> producer: this layer's routing is in sew[]
  int32_t sel_idx[12];
  float sel_w[12];
  float gap, s_inv, s_m, s_sum;
  float hmax[8], hse[8], wmax[16];
  float av[16];
  int32_t ai[16];
  volatile int32_t fail;
  int32_t nstamp[2];            // stage clock: records written so far (consumer, producer)
  Seg segs[kMaxSegs2];          // the producer warp's current segment list
  int32_t nseg;
};
static_assert(sizeof(StepShared) <= kHdrBytes, "header area");
static_assert(sizeof(StepPlan) % 16 == 0 && sizeof(StepLayer) % 16 == 0 && sizeof(ExpertW) % 16 == 0 &&
                  offsetof(StepShared, ly) % 16 == 0 && offsetof(StepShared, sew) % 16 == 0,
              "records copied as 16-byte words");

// The block's shared memory and the two things every stage needs from it. (Kept out of the
// per-thread context on purpose: that lives in local memory, and with 544 threads and a
// 24 KB L1 every access to it was a trip to L2.)
extern __shared__ __align__(128) unsigned char step_smem[];
#define SH (reinterpret_cast<StepShared *>(step_smem))
#define PL (reinterpret_cast<StepShared *>(step_smem)->plan)

__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }
__device__ __forceinline__ void hsync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }  // threads 0..255
__device__ __forceinline__ unsigned long long gtime_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void step_fail(int code) {
  SH->fail = code;
  atomicExch(PL.error, code);
}
// Bounded wait on an mbarrier phase; false when it gave up (now or earlier).
__device__ __forceinline__ bool mbar_wait_b(uint32_t addr, uint32_t parity, int code) {
  if (mbar_try_a(addr, parity)) return true;
  if (SH->fail) return false;
  const long long t0 = clock64();
#pragma unroll 1
  for (unsigned i = 1;; ++i) {
    if (mbar_try_a(addr, parity)) return true;
    if ((i & 63u) == 0u) {
      if (SH->fail) return false;
      if (clock64() - t0 > kWaitCycles) {
        step_fail(code);
        return false;
      }
    }
  }
}

// Optional stage clock (plan->stage_stamps non-null): block 0 appends (id << 48 | %globaltimer)
// records, consumer thread 0 to the first half of the buffer, the producer thread to the second.
// Consumer ids: 1 a grid barrier was passed, 2 a stage's prologue (norm / quantiser) is done, 3 its
// GEMV and epilogues are done, 4 the recurrence's barrier was passed, 5 the experts are selected,
// 6 their pointer records are fetched, 20-24 inside the attention stage (chunk staged, heads
// prepared, scores, softmax, values). Producer ids: 10-12 the tiles of the first projections, the
// output projection and the router are issued, 13 the selection arrived, 14 / 15 the gate/up and
// the down tiles are issued. A record costs a few hundred nanoseconds, so a stamped step is a few
// per cent slower than the product's.
static __device__ __noinline__ void stamp(int id) {
  if (PL.stage_stamps && blockIdx.x == 0 && (threadIdx.x == 0 || threadIdx.x == kCons)) {
    const int who = threadIdx.x == 0 ? 0 : 1, half = PL.stage_stamp_cap / 2;
    const int n = SH->nstamp[who];
    if (n < half)
      PL.stage_stamps[who * half + n] = ((unsigned long long)id << 48) | (gtime_ns() & 0xFFFFFFFFFFFFull);
    SH->nstamp[who] = n + 1;
  }
}

// Rows [lo, hi) of `total` for block blk of nblk, cut at multiples of `unit` rows.
__device__ __forceinline__ void deal(int total, int unit, int blk, int nblk, int &lo, int &hi) {
  const long units = (total + unit - 1) / unit;
  lo = (int)(units * blk / nblk) * unit;
  hi = (int)(units * (blk + 1) / nblk) * unit;
  if (hi > total) hi = total;
  if (lo > total) lo = total;
}
// Row unit that keeps a block's share of the bf16 group scales 16-byte aligned (2*K/128 bytes per row).
__device__ __forceinline__ int row_unit(int K) {
  const int G = K >> 7;
  return G >= 8 ? 1 : 8 / G;
}

// ------------------------------------------------------------------ grid barrier ---
// Two halves, so that loads which do not depend on other blocks (recurrent state, KV rows of
// earlier tokens, epilogue operands) can be issued between arriving and waiting.
static __device__ __noinline__ void grid_arrive() {
  csync();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(PL.bar_count, 1u);
  }
}
// epoch: how many barriers this block has arrived at, this one included
static __device__ __noinline__ void grid_wait(unsigned epoch) {
  if (threadIdx.x == 0 && !SH->fail) {
    const unsigned target = epoch * gridDim.x;
    const long long t0 = clock64();
#pragma unroll 1
    for (unsigned i = 0;; ++i) {
      if (ld_acquire_u32(PL.bar_count) >= target) break;
      if ((i & 63u) == 63u) {
        if (*(volatile int *)PL.error != 0) { SH->fail = 1; break; }
        if (clock64() - t0 > kWaitCycles) { step_fail(1); break; }
      }
    }
  }
  csync();
  stamp(1);
}

// ====================================================================== producer ===

// Streams the rows of the segment list in shared memory (SH->segs), laid end to end, through
// the ring in tiles of 16 KB. Called by the whole producer warp: lane l (l < kNT) owns ring slot
// l and issues the tiles whose running index is l modulo kNT, so up to kNT tiles are prepared and
// issued at once. Tile j of the call holds rows [j * rpt, (j + 1) * rpt) of the list, so the
// consumers know what every tile holds without being told. The group scales of a piece travel
// by bulk copy when source, size and offset are 16-byte aligned; otherwise (small matrices) the
// lane copies them itself before it completes the tile. `tile` is the running index of the
// call's first tile; returns the index after its last.
static __device__ __noinline__ uint32_t prod_emit(uint32_t tile, int row_bytes, int sc_row_bytes) {
  const Seg *segs = SH->segs;
  const int nseg = SH->nseg;
  const int rpt = kTileBytes / row_bytes;
  int total = 0;
  for (int i = 0; i < nseg; ++i) total += segs[i].nrows;
  const int ntiles = (total + rpt - 1) / rpt;
  const uint32_t base = tile;
  const int lane = threadIdx.x & 31;
  if (lane < kNT && ntiles > 0) {
    unsigned char *ring = step_smem + kRingOff;
    int j = (int)(((uint32_t)lane + kNT - base % kNT) % kNT);  // first tile of this call that lands in slot `lane`
#pragma unroll 1
    for (; j < ntiles; j += kNT) {
      const uint32_t g = base + (uint32_t)j, slot = (uint32_t)lane, use = g / kNT;
      if (use > 0 && !mbar_wait_b(smem_addr(&SH->empty[slot]), (use - 1u) & 1u, 3)) break;
      unsigned char *dst = ring + slot * kTileStride;
      unsigned long long *bar = &SH->full[slot];
      const int f0 = j * rpt, f1 = f0 + rpt < total ? f0 + rpt : total;
      int row0 = 0;  // flat row of the current segment's first row
#pragma unroll 1
      for (int si = 0; si < nseg && row0 < f1; ++si) {
        const Seg sg = segs[si];
        const int a = row0 > f0 ? row0 : f0, b = row0 + sg.nrows < f1 ? row0 + sg.nrows : f1;
        if (a < b) {
          const int sr = a - row0, take = b - a, rows = a - f0;
          const uint8_t *src = sg.P + (size_t)sr * row_bytes;
          const uint8_t *ssrc = sg.S ? sg.S + (size_t)sr * sc_row_bytes : nullptr;
          const uint32_t wb = (uint32_t)(take * row_bytes), sb = (uint32_t)(take * sc_row_bytes);
          const bool sc_bulk = ssrc != nullptr &&
                               ((reinterpret_cast<uintptr_t>(ssrc) | sb | (uint32_t)(rows * sc_row_bytes)) & 15u) == 0;
          if (ssrc != nullptr && !sc_bulk) {
            const uint16_t *s16 = reinterpret_cast<const uint16_t *>(ssrc);
            uint16_t *d16 = reinterpret_cast<uint16_t *>(dst + kTileBytes + (size_t)rows * sc_row_bytes);
            for (uint32_t i = 0; i < sb / 2; ++i) d16[i] = __ldg(s16 + i);
          }
          if (reinterpret_cast<uintptr_t>(src) & 15u) {  // cannot be copied in bulk: report, skip
            if (g_stream_fault_word) *reinterpret_cast<volatile unsigned int *>(g_stream_fault_word) = 2;
          } else {
            mbar_expect_tx(bar, wb + (sc_bulk ? sb : 0u));
            bulk_g2s(dst + (size_t)rows * row_bytes, src, wb, bar);
            if (sc_bulk) bulk_g2s(dst + kTileBytes + (size_t)rows * sc_row_bytes, ssrc, sb, bar);
          }
        }
        row0 += sg.nrows;
      }
      mbar_arrive(bar);  // releases this lane's own stores and completes the phase once the bytes have landed
    }
  }
  __syncwarp();  // the list may be rewritten once every lane is done with it
  return base + (uint32_t)ntiles;
}

__device__ __forceinline__ int mats_rows(const GemvMat *m, int nm) {
  int t = 0;
  for (int i = 0; i < nm; ++i) t += m[i].N;
  return t;
}

// Segment list of rows [lo, hi) of a table of matrices whose rows are numbered end to end
// (written by lane 0 of the producer warp).
__device__ __forceinline__ void segs_gemv(const GemvMat *m, int nm, int K, int lo, int hi) {
  if ((threadIdx.x & 31) == 0) {
    Seg *out = SH->segs;
    int n = 0, rs = 0;
    for (int i = 0; i < nm; ++i) {
      const int N = m[i].N;
      const int a = lo > rs ? lo : rs, b = hi < rs + N ? hi : rs + N;
      if (a < b) {
        out[n].P = m[i].P + (size_t)(a - rs) * (K >> 1);
        out[n].S = reinterpret_cast<const uint8_t *>(m[i].S + (size_t)(a - rs) * (K >> 7));
        out[n].nrows = b - a;
        out[n].vec = 0;
        out[n].trow = a - lo;
        ++n;
      }
      rs += N;
    }
    SH->nseg = n;
  }
  __syncwarp();
}

static __device__ __noinline__ uint32_t prod_gemv(uint32_t tile, const GemvMat *m, int nm, int K) {
  int lo, hi;
  deal(mats_rows(m, nm), row_unit(K), (int)blockIdx.x, (int)gridDim.x, lo, hi);
  segs_gemv(m, nm, K, lo, hi);
  return prod_emit(tile, K >> 1, (K >> 7) * 2);
}

// The producer warp's whole token. Returns the number of tiles issued.
static __device__ __noinline__ uint32_t producer_main(int mode) {
  const StepPlan &P = PL;
  const int H = P.H, blk = (int)blockIdx.x, nblk = (int)gridDim.x;
  const bool lead = (threadIdx.x & 31) == 0;
  uint32_t tile = 0;
  for (int L = 0; L < P.layers; ++L) {
    const StepLayer &ly = P.L[L];
    const bool lin = ly.type == 0;
    tile = prod_gemv(tile, &ly.m[0], lin ? 4 : 3, H);
    stamp(10);
    tile = prod_gemv(tile, &ly.m[4], 1, lin ? P.nV * 128 : P.nQ * 256);
    stamp(11);
    {  // router rows (bf16) and the shared-expert gate row
      const int rows = P.E + (ly.shared_gate ? 1 : 0);
      int lo, hi;
      deal(rows, 1, blk, nblk, lo, hi);
      if (lead) {
        Seg *segs = SH->segs;
        int n = 0;
        const int b = hi < P.E ? hi : P.E;
        if (lo < b) segs[n++] = Seg{reinterpret_cast<const uint8_t *>(ly.router + (size_t)lo * H), nullptr, b - lo, 0, 0, 0};
        if (hi > P.E) segs[n++] = Seg{reinterpret_cast<const uint8_t *>(ly.shared_gate), nullptr, 1, 0, P.E - lo, 0};
        SH->nseg = n;
      }
      __syncwarp();
      tile = prod_emit(tile, H * 2, 0);
    }
    // the expert weights depend on the routing: wait for the consumers' selection
    stamp(12);
    if (!mbar_wait_b(smem_addr(&SH->sel_bar), (uint32_t)L & 1u, 4)) return tile;
    stamp(13);
    {  // gate and up rows of pair rows [lo, hi) over slots x I
      int lo, hi;
      deal(P.slots * P.I, row_unit(H), blk, nblk, lo, hi);
      if (lead) {
        Seg *segs = SH->segs;
        int n = 0;
        if (lo < hi) {
          const int s0 = lo / P.I, s1 = (hi - 1) / P.I;
          for (int s = s0; s <= s1 && n + 2 <= kMaxSegs2; ++s) {
            const int a = lo > s * P.I ? lo : s * P.I, b = hi < (s + 1) * P.I ? hi : (s + 1) * P.I;
            const ExpertW &ew = SH->sew[s];
            const size_t r0 = (size_t)(a - s * P.I);
            segs[n++] = Seg{ew.gP + r0 * (H >> 1), reinterpret_cast<const uint8_t *>(ew.gS + r0 * (H >> 7)), b - a, 0, a - lo, 0};
            segs[n++] = Seg{ew.uP + r0 * (H >> 1), reinterpret_cast<const uint8_t *>(ew.uS + r0 * (H >> 7)), b - a, 0,
                            (hi - lo) + (a - lo), 0};
          }
        }
        SH->nseg = n;
      }
      __syncwarp();
      tile = prod_emit(tile, H >> 1, (H >> 7) * 2);
    }
    stamp(14);
    {  // down rows [lo, hi) of every slot
      int lo, hi;
      deal(H, row_unit(P.I), blk, nblk, lo, hi);
      if (lead) {
        Seg *segs = SH->segs;
        int n = 0;
        if (lo < hi) {
          const int nr = hi - lo;
          for (int s = 0; s < P.slots; ++s) {
            const ExpertW &ew = SH->sew[s];
            segs[n++] = Seg{ew.dP + (size_t)lo * (P.I >> 1), reinterpret_cast<const uint8_t *>(ew.dS + (size_t)lo * (P.I >> 7)),
                            nr, s, s * nr, 0};
          }
        }
        SH->nseg = n;
      }
      __syncwarp();
      tile = prod_emit(tile, P.I >> 1, (P.I >> 7) * 2);
    }
    stamp(15);
  }
  if (mode != 0) tile = prod_gemv(tile, &P.lm_head, 1, H);
  return tile;
}

// ====================================================================== consumers ===
// Dots the tiles of one stage with staged activations. The stage's rows are numbered 0..total-1
// in the order the producer streams them (tile j holds rows [j * rpt, (j + 1) * rpt)); row f is
// dotted with activation vector f / vec_rows (vec_rows = 0: always vector 0) and its group terms
// go to t[g][f - row_base]. Rows [row_base, row_base + nrows) are done by this call, starting at
// running tile index `tile`; returns the index after the last tile consumed. A tile is 256
// (row, group) tasks of 64 bytes; two adjacent lanes share a task (32 bytes each) and add their
// exact integer sums with one shuffle.
__device__ __forceinline__ uint32_t dot_tiles(uint32_t tile, int K, const uint4 *xa, const float *sq, float *T,
                                              int row_base, int nrows, int total, int vec_rows) {
  const int G = K >> 7, lg = 31 - __clz(G);
  const int TS = (kTCap >> lg) + 1, rpt = 256 >> lg;
  const int task = threadIdx.x >> 1, half = threadIdx.x & 1, lane = threadIdx.x & 31;
  const int r = task >> lg, g = task & (G - 1);
  const uint32_t rot = (uint32_t)(lane >> 2) & 1u;
  const uint32_t ring_a = smem_addr(step_smem + kRingOff);
  const int ntiles = (nrows + rpt - 1) / rpt;
  int cvec = -1;
  uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0, x2 = x0, x3 = x0;
  float sqg = 0.0f;
#pragma unroll 1
  for (int j = 0; j < ntiles; ++j) {
    const uint32_t slot = tile % kNT, use = tile / kNT;
    // a wait that gave up ends the stage for the whole warp (the results are lost anyway)
    if (!__all_sync(kFull, mbar_wait_b(smem_addr(&SH->full[slot]), use & 1u, 5))) break;
    const uint32_t tb = ring_a + slot * kTileStride;
    const uint32_t wbase = tb + (uint32_t)task * 64u + (uint32_t)half * 32u;
    const uint4 wa = lds128(wbase + (rot << 4)), wb = lds128(wbase + ((rot ^ 1u) << 4));
    const uint32_t sraw = lds_u16(tb + kTileBytes + (uint32_t)task * 2u);
    __syncwarp();
    if (lane == 0) mbar_arrive_a(smem_addr(&SH->empty[slot]));
    const int f = row_base + j * rpt + r;
    const bool live = j * rpt + r < nrows && f < total;
    int dsum = 0;
    if (live) {
      const int vec = vec_rows ? f / vec_rows : 0;
      if (vec != cvec) {
        cvec = vec;
        const uint4 *xv = xa + (size_t)vec * 8 * G + g;
        const int q0 = half * 4 + (int)rot * 2, q1 = half * 4 + (int)(rot ^ 1u) * 2;
        x0 = xv[q0 * G];
        x1 = xv[(q0 + 1) * G];
        x2 = xv[q1 * G];
        x3 = xv[(q1 + 1) * G];
        sqg = sq[vec * G + g];
      }
      int d0 = dot16_x16(wa, 0, x0, 0), d1 = dot16_x16(wa, 1, x1, 0);
      d0 = dot16_x16(wb, 0, x2, d0);
      d1 = dot16_x16(wb, 1, x3, d1);
      dsum = d0 + d1;
    }
    dsum += __shfl_xor_sync(kFull, dsum, 1);
    if (live && half == 0) {
      const float v = (float)(dsum >> 4) * __uint_as_float(sraw << 16);
      T[g * TS + (f - row_base)] = v * sqg;
    }
    tile += 1;
  }
  return tile;
}

// (1+w) RMSNorm + per-128 quantiser of one H-vector into the staged form, by the whole
// consumer group (RMSNormW + ScalesMax + Quantize, tools/cmdlist/kernels.cpp:73-114,551-579).
// Sum of squares: fp64 over 256 strided lanes (thread j < 256 adds x[j], x[j+256], ... in
// order), then the stride-halving tree, whose levels 128, 64 and 32 every warp evaluates for
// itself from the 256 partial sums in shared memory (lane l: ((p[l]+p[l+128]) + (p[l+64]+
// p[l+192])) + ((p[l+32]+p[l+160]) + (p[l+96]+p[l+224]))) and whose last five levels are the xor
// butterfly. Double-precision arithmetic is slow on this GPU (a few lanes per cycle and SM), so
// the element-wise part is done once, not once per warp.
// src: fp32 vector in global memory, or (emb != null) a bf16 embedding row. hn (optional): the
// normalised fp32 vector, shared memory. xout (optional): copy of the input, global.
static __device__ __noinline__ void norm_quant(const float *src, const uint16_t *emb, const float *w, int H, float *hn,
                                               float *xout) {
  float *xs = reinterpret_cast<float *>(step_smem + kFbufOff);
  double *ps = reinterpret_cast<double *>(step_smem + kTOff);
  unsigned char *act = step_smem + kActOff;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float4 v[2];  // H <= 4096: at most two float4 per thread
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int j = (tid + kCons * u) * 4;
    v[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (j < H) {
      if (emb) {
        const uint2 e = __ldg(reinterpret_cast<const uint2 *>(emb + j));
        v[u] = make_float4(u2f(e.x << 16), u2f(e.x & 0xFFFF0000u), u2f(e.y << 16), u2f(e.y & 0xFFFF0000u));
      } else {
        v[u] = __ldcg(reinterpret_cast<const float4 *>(src + j));
      }
    }
  }
  float4 wv[2];  // the weights of this warp's groups, in flight during the reduction
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int g = warp + 16 * i;
    wv[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (g < H / 128) wv[i] = __ldg(reinterpret_cast<const float4 *>(w + g * 128) + lane);
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int j = (tid + kCons * u) * 4;
    if (j < H) {
      *reinterpret_cast<float4 *>(xs + j) = v[u];
      if (xout) *reinterpret_cast<float4 *>(xout + j) = v[u];
    }
  }
  csync();
  if (tid < 256) {
    double ss = 0;
#pragma unroll 1
    for (int j = tid; j < H; j += 256) {
      const double dv = (double)xs[j];
      ss = ss + dv * dv;
    }
    ps[tid] = ss;
  }
  csync();
  double t = ((ps[lane] + ps[lane + 128]) + (ps[lane + 64] + ps[lane + 192])) +
             ((ps[lane + 32] + ps[lane + 160]) + (ps[lane + 96] + ps[lane + 224]));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) t = t + __shfl_xor_sync(kFull, t, off);
  const float inv = 1.0f / sqrtf((float)(t / (double)H) + PL.eps);
  uint32_t *xw = reinterpret_cast<uint32_t *>(act);
  float *sqs = reinterpret_cast<float *>(act + H);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int g = warp + 16 * i;
    if (g < H / 128) {
      const int j = g * 128 + lane * 4;
      const float4 x = *reinterpret_cast<const float4 *>(xs + j);
      float4 y;
      y.x = (x.x * inv) * (1.0f + wv[i].x);
      y.y = (x.y * inv) * (1.0f + wv[i].y);
      y.z = (x.z * inv) * (1.0f + wv[i].z);
      y.w = (x.w * inv) * (1.0f + wv[i].w);
      if (hn) *reinterpret_cast<float4 *>(hn + j) = y;
      quant_group_staged(xw, sqs, H, 0, g, y);
    }
  }
  csync();
}

// Stages an already quantised vector (INT8 + group scales in global memory).
static __device__ __noinline__ void stage_q8(const int8_t *xq, const float *sqg, int K) {
  unsigned char *act = step_smem + kActOff;
  uint32_t *xw = reinterpret_cast<uint32_t *>(act);
  float *sqs = reinterpret_cast<float *>(act + K);
  for (int pc = threadIdx.x; pc < K / 8; pc += kCons) {
    const uint2 v = __ldcg(reinterpret_cast<const uint2 *>(xq + (size_t)pc * 8));
    xw[staged4_word(K, 0, pc, 0)] = __byte_perm(v.x, v.y, 0x6420);
    xw[staged4_word(K, 0, pc, 1)] = __byte_perm(v.x, v.y, 0x7531);
  }
  for (int g = threadIdx.x; g < K / 128; g += kCons) sqs[g] = __ldcg(sqg + g);
  csync();
}

// Quantises M contiguous fp32 vectors of K (global memory, M * K <= 8192) into the staged form.
static __device__ __noinline__ void quant_rows(const float *x, int K, int M) {
  float *raw = reinterpret_cast<float *>(step_smem + kFbufOff);
  unsigned char *act = step_smem + kActOff;
  const int n4 = M * K / 4;
  float4 v[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = threadIdx.x + kCons * u;
    v[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (i < n4) v[u] = __ldcg(reinterpret_cast<const float4 *>(x) + i);
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = threadIdx.x + kCons * u;
    if (i < n4) reinterpret_cast<float4 *>(raw)[i] = v[u];
  }
  csync();
  uint32_t *xw = reinterpret_cast<uint32_t *>(act);
  float *sqs = reinterpret_cast<float *>(act + (size_t)M * K);
  const int G = K >> 7, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll 1
  for (int gi = warp; gi < M * G; gi += 16) {
    const float4 q = reinterpret_cast<const float4 *>(raw + (size_t)gi * 128)[lane];
    quant_group_staged(xw, sqs, K, gi / G, gi % G, q);
  }
  csync();
}

// Gated per-head norm + quantiser (RmsInv + NormGated + ScalesMax + Quantize,
// kernels.cpp:619-644,551-579), one warp per head, into the staged form (K = nV * 128).
static __device__ __noinline__ void gated_norm_quant(const float *O, const float *Z, const float *W, int nV) {
  float *os = reinterpret_cast<float *>(step_smem + kFbufOff), *zs = os + 4096;
  unsigned char *act = step_smem + kActOff;
  const int n4 = nV * 32, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float4 wn = __ldg(reinterpret_cast<const float4 *>(W) + lane);
  float4 vo[2], vz[2];  // nV * 128 <= 4096 values: at most two float4 of each per thread
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = threadIdx.x + kCons * u;
    vo[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    vz[u] = vo[u];
    if (i < n4) {
      vo[u] = __ldcg(reinterpret_cast<const float4 *>(O) + i);
      vz[u] = __ldcg(reinterpret_cast<const float4 *>(Z) + i);
    }
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = threadIdx.x + kCons * u;
    if (i < n4) {
      reinterpret_cast<float4 *>(os)[i] = vo[u];
      reinterpret_cast<float4 *>(zs)[i] = vz[u];
    }
  }
  csync();
  const int K = nV * 128;
  uint32_t *xw = reinterpret_cast<uint32_t *>(act);
  float *sqs = reinterpret_cast<float *>(act + K);
#pragma unroll 1
  for (int h = warp; h < nV; h += 16) {
    const float *o = os + h * 128, *z = zs + h * 128;
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float ov = o[lane + 32 * i];
      ss = fmaf(ov, ov, ss);
    }
    ss = warp_tree_sum(ss);
    const float inv = 1.0f / sqrtf(ss / 128.0f + PL.eps);
    const float4 ov = reinterpret_cast<const float4 *>(o)[lane], zv = reinterpret_cast<const float4 *>(z)[lane];
    float4 y;
    y.x = ((wn.x * ov.x) * inv) * (zv.x / (1.0f + det_expf(-zv.x)));
    y.y = ((wn.y * ov.y) * inv) * (zv.y / (1.0f + det_expf(-zv.y)));
    y.z = ((wn.z * ov.z) * inv) * (zv.z / (1.0f + det_expf(-zv.z)));
    y.w = ((wn.w * ov.w) * inv) * (zv.w / (1.0f + det_expf(-zv.w)));
    quant_group_staged(xw, sqs, K, 0, h, y);
  }
  csync();
}

// Matrix and local row of flat row `flat` of a table of matrices.
__device__ __forceinline__ int mat_of_row(const GemvMat *m, int nm, int flat, int &n) {
  int rs = 0, i = 0;
  while (i < nm - 1 && flat >= rs + m[i].N) {
    rs += m[i].N;
    ++i;
  }
  n = flat - rs;
  return i;
}

// One GEMV stage: this block's rows of the matrices, activations already staged. The operands
// of the rows' epilogues (residual, conv state, decay constants) are fetched before the dot and
// stay in flight during it: dot_tiles is inlined here, because across a real call the compiler
// would have to spill the registers the loads land in, and the spill would wait for the loads.
static __device__ __noinline__ uint32_t gemv_stage_run(uint32_t tile, const GemvMat *m, int nm, int K) {
  int lo, hi;
  deal(mats_rows(m, nm), row_unit(K), (int)blockIdx.x, (int)gridDim.x, lo, hi);
  if (lo >= hi) return tile;
  float *T = reinterpret_cast<float *>(step_smem + kTOff);
  unsigned char *act = step_smem + kActOff;
  const int G = K >> 7, nr = hi - lo;
  EpiOperands eo;
  int mi = 0, n = 0;
  if ((int)threadIdx.x < nr) {
    mi = mat_of_row(m, nm, lo + threadIdx.x, n);
    gemv_epilogue_fetch(&m[mi], n, 0, eo);
  }
  tile = dot_tiles(tile, K, reinterpret_cast<const uint4 *>(act), reinterpret_cast<const float *>(act + K), T, 0, nr, nr, 0);
  csync();
  if ((int)threadIdx.x < nr) gemv_epilogue_with(&m[mi], n, 0, row_sum_rt(T, threadIdx.x, G), eo);
  for (int r = threadIdx.x + kCons; r < nr; r += kCons) {
    mi = mat_of_row(m, nm, lo + r, n);
    gemv_epilogue(&m[mi], n, 0, row_sum_rt(T, r, G));
  }
  return tile;
}

// Router logits of this block's rows from the ring (bf16 rows), activations hn in shared memory.
// logits[e] = sum_k bf16(W[e][k]) * hn[k]: lane l takes k = (i*32+l)*8+j, fma chain in (i, j)
// order, then the lane tree (as RouterTopK).
static __device__ __noinline__ uint32_t router_stage(uint32_t tile, const float *hn, int H, int rows_total) {
  int lo, hi;
  deal(rows_total, 1, (int)blockIdx.x, (int)gridDim.x, lo, hi);
  if (lo >= hi) return tile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = H / 256;
  const int rpt = kTileBytes / (H * 2), total = hi - lo, ntiles = (total + rpt - 1) / rpt;
  const uint32_t ring_a = smem_addr(step_smem + kRingOff);
#pragma unroll 1
  for (int j = 0; j < ntiles; ++j) {
    const uint32_t slot = tile % kNT, use = tile / kNT;
    if (!__all_sync(kFull, mbar_wait_b(smem_addr(&SH->full[slot]), use & 1u, 5))) break;
    const uint32_t tb = ring_a + slot * kTileStride;
    const int nr = total - j * rpt < rpt ? total - j * rpt : rpt;
    for (int r = warp; r < nr; r += 16) {
      float acc = 0.0f;
      for (int i = 0; i < n; ++i) {
        const int k0 = (i * 32 + lane) * 8;
        const uint4 wv = lds128(tb + (uint32_t)r * (uint32_t)(H * 2) + (uint32_t)k0 * 2u);
        const float4 a0 = *reinterpret_cast<const float4 *>(hn + k0), a1 = *reinterpret_cast<const float4 *>(hn + k0 + 4);
        acc = fmaf(u2f(wv.x << 16), a0.x, acc);
        acc = fmaf(u2f(wv.x & 0xFFFF0000u), a0.y, acc);
        acc = fmaf(u2f(wv.y << 16), a0.z, acc);
        acc = fmaf(u2f(wv.y & 0xFFFF0000u), a0.w, acc);
        acc = fmaf(u2f(wv.z << 16), a1.x, acc);
        acc = fmaf(u2f(wv.z & 0xFFFF0000u), a1.y, acc);
        acc = fmaf(u2f(wv.w << 16), a1.z, acc);
        acc = fmaf(u2f(wv.w & 0xFFFF0000u), a1.w, acc);
      }
      acc = warp_tree_sum(acc);
      if (lane == 0) PL.RLogits[lo + j * rpt + r] = acc;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive_a(smem_addr(&SH->empty[slot]));
    tile += 1;
  }
  return tile;
}

// Softmax over the E router logits, top-k by (probability desc, index asc), renormalised
// weights, shared-expert gate: the selection of RouterTopK, run by every block for itself.
static __device__ __noinline__ void router_select_cons(int E, int k, bool has_shared) {
  float *lg = reinterpret_cast<float *>(step_smem + kFbufOff), *sp = lg + 2048;  // logits, probabilities (E <= 1024)
  unsigned *ck = reinterpret_cast<unsigned *>(step_smem + kTOff), *ci = ck + kTopkWarps * kTopkMaxSel;
  StepShared *sh = SH;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int e = tid; e <= E; e += kCons)
    if (e < E || has_shared) lg[e] = __ldcg(PL.RLogits + e);
  csync();
  // maximum and sum keep the one-warp partition (lane l takes entries l, l+32, ... in ascending
  // order, then the xor butterfly); every warp evaluates them for itself, which gives every warp
  // the same bits and saves two block barriers and two one-warp sections
  float m = -INFINITY;
  for (int e = lane; e < E; e += 32) m = fmaxf(m, lg[e]);
  m = warp_max(m);
  for (int e = tid; e < E; e += kCons) sp[e] = det_expf(lg[e] - m);
  if (tid == 0 && has_shared) sp[E] = lg[E];
  csync();
  float sum = 0.0f;
  for (int e = lane; e < E; e += 32) sum = sum + sp[e];
  sum = warp_tree_sum(sum);
  csync();  // every warp has read the exponentials
  for (int e = tid; e < E; e += kCons) sp[e] = sp[e] / sum;
  csync();
  const int nsel = k + 1 < kTopkMaxSel ? k + 1 : kTopkMaxSel;
  if (warp < kTopkWarps) {
    const int per = (E + kTopkWarps - 1) / kTopkWarps;
    unsigned key[4], idx[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int o = lane + 32 * i, e = warp * per + o;
      const bool ok = o < per && e < E;
      key[i] = ok ? __float_as_uint(sp[e]) + 1u : 0u;
      idx[i] = ok ? (unsigned)e : 0x7FFFFFFFu;
    }
#pragma unroll 1
    for (int j = 0; j < nsel; ++j) {
      unsigned wv, wi;
      topk_extract<4>(key, idx, wv, wi);
      if (lane == 0) {
        ck[warp * nsel + j] = wv;
        ci[warp * nsel + j] = wi;
      }
    }
  }
  csync();
  if (warp == 0) {
    const int ncand = kTopkWarps * nsel;
    if (ncand <= 128) topk_level2<4>(ck, ci, ncand, sp, E, k, has_shared, sh->sel_idx, sh->sel_w, &sh->gap);
    else topk_level2<9>(ck, ci, ncand, sp, E, k, has_shared, sh->sel_idx, sh->sel_w, &sh->gap);
  }
  csync();
}

// ------------------------------------------------------------ gated delta rule ---
// One (head, column slice) item per block, 256 threads, state in registers; the arithmetic is
// DeltaNetStep's (deltanet_core.cuh). The state of the block's first item is loaded before the
// grid barrier is waited for: it was last written one token ago by this same block.
static __device__ __noinline__ void deltanet_stage(unsigned epoch, const StepLayer &ly) {
  const StepPlan &P = PL;
  constexpr int D = 128, SEG = kDnSeg;
  DeltaNetStepArgs a{P.O, P.Mx, ly.S, P.Bt, P.Gt, P.nK, P.nV};
  const int nitems = P.nV * kDnSlices;
  const bool worker = threadIdx.x < 256;
  float s[SEG];
  if (worker && (int)blockIdx.x < nitems) deltanet_load_state(a, (int)blockIdx.x, s);
  grid_wait(epoch);
  if (!worker) return;
  float *qs = reinterpret_cast<float *>(step_smem + kFbufOff), *ks = qs + D;
  float(*part)[32] = reinterpret_cast<float(*)[32]>(ks + D);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll 1
  for (int item = (int)blockIdx.x; item < nitems; item += (int)gridDim.x) {
    const int h = item / kDnSlices, slice = item % kDnSlices;
    const int kh = h / (a.nV / a.nK);
    const int col = slice * 32 + lane;
    float *Sh = a.S + (size_t)h * D * D;
    if (item != (int)blockIdx.x) deltanet_load_state(a, item, s);
    if (warp < 2) {
      const float *src = a.Mx + (warp == 0 ? (size_t)kh * D : (size_t)a.nK * D + (size_t)kh * D);
      float x[4];
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[i] = __ldcg(src + lane + 32 * i);
        ss = fmaf(x[i], x[i], ss);
      }
      ss = warp_tree_sum(ss);
      const float inv = 1.0f / sqrtf(ss + 1e-6f);
      const float f = inv * (warp == 0 ? 0.0883883476483184405f : 1.0f);
      float *dst = warp == 0 ? qs : ks;
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = x[i] * f;
    }
    const float val = __ldcg(a.Mx + (size_t)2 * a.nK * D + (size_t)h * D + col);
    const float beta = __ldcg(a.Bt + h);
    const float gt = det_expf(__ldcg(a.Gt + h));
    hsync();
    float acc = 0.0f;
#pragma unroll
    for (int r = 0; r < SEG; ++r) {
      s[r] = s[r] * gt;
      acc = fmaf(s[r], ks[warp * SEG + r], acc);
    }
    part[warp][lane] = acc;
    hsync();
    const float kv = ((part[0][lane] + part[1][lane]) + (part[2][lane] + part[3][lane])) +
                     ((part[4][lane] + part[5][lane]) + (part[6][lane] + part[7][lane]));
    const float dl = (val - kv) * beta;
    hsync();
    acc = 0.0f;
#pragma unroll
    for (int r = 0; r < SEG; ++r) {
      s[r] = fmaf(ks[warp * SEG + r], dl, s[r]);
      acc = fmaf(s[r], qs[warp * SEG + r], acc);
      Sh[(size_t)(warp * SEG + r) * D + col] = s[r];
    }
    part[warp][lane] = acc;
    hsync();
    if (warp == 0) {
      const float o = ((part[0][lane] + part[1][lane]) + (part[2][lane] + part[3][lane])) +
                      ((part[4][lane] + part[5][lane]) + (part[6][lane] + part[7][lane]));
      a.Out[(size_t)h * D + col] = o;
    }
    hsync();
  }
}

// ------------------------------------------------------------------- attention ---
// One 64-token chunk of one KV head per item: head norm + RoPE of the group's query heads
// (and, in the chunk that holds the new position, of the new key; INT8 append of key and
// value), scores, chunk softmax, weighted values. Arithmetic of AttnPrep + AttnSplit
// (attention_core.cuh). K/V rows of earlier tokens are fetched before the grid barrier is
// waited for (they were written by earlier steps).
template <int GQ>
static __device__ __noinline__ void attn_stage_t(unsigned epoch, const StepLayer &ly, int pos, int T) {
  const StepPlan &P = PL;
  constexpr int D = kHeadDim, C = kAttnChunk;
  constexpr int GH = (GQ + 1) / 2;  // query heads per half of the block in the value pass
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nKV = P.nKV;
  const int nch = (T + C - 1) / C, nitems = nch * nKV;
  unsigned char *kvs = step_smem + kFbufOff;  // K rows [C][D], then V rows [C][D]
  float *qs = reinterpret_cast<float *>(step_smem + kTOff);  // [GQ][D]
  float *sc = qs + GQ * D;                                // [C][GQ]: per token the heads' scores, then weights
  uint16_t *kss = reinterpret_cast<uint16_t *>(sc + GQ * C), *vss = kss + C;
  StepShared *sh = SH;
  const int p = pos < P.max_ctx ? pos : P.max_ctx - 1;  // clamp, kernels.cpp:456
  const float scale = 1.0f / sqrtf((float)D);

  uint4 kvr[4];
  uint16_t scr = 0;
  auto load_chunk = [&](int item) {
    const int ch = item / nKV, kv = item % nKV, t0 = ch * C;
    const int nt = (T < t0 + C ? T : t0 + C) - t0;
    const size_t rs = (size_t)nKV * (D / 16);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = tid + kCons * u, which = i >> 10, row = (i & 1023) >> 4, pc = i & 15;
      kvr[u] = make_uint4(0, 0, 0, 0);
      if (row < nt && t0 + row != p) {
        const int8_t *base = which ? ly.Vc : ly.Kc;
        kvr[u] = __ldcg(reinterpret_cast<const uint4 *>(base + ((size_t)t0 * nKV + kv) * D) + row * rs + pc);
      }
    }
    if (tid < 2 * C) {
      const int row = tid & (C - 1);
      scr = 0;
      if (row < nt && t0 + row != p) scr = __ldcg((tid < C ? ly.Ks : ly.Vs) + (size_t)(t0 + row) * nKV + kv);
    }
  };
  if ((int)blockIdx.x < nitems) load_chunk((int)blockIdx.x);
  grid_wait(epoch);
#pragma unroll 1
  for (int item = (int)blockIdx.x; item < nitems; item += (int)gridDim.x) {
    const int ch = item / nKV, kv = item % nKV, t0 = ch * C;
    const int nt = (T < t0 + C ? T : t0 + C) - t0;
    if (item != (int)blockIdx.x) load_chunk(item);
#pragma unroll
    for (int u = 0; u < 4; ++u) reinterpret_cast<uint4 *>(kvs)[tid + kCons * u] = kvr[u];
    if (tid < C) kss[tid] = scr;
    else if (tid < 2 * C) vss[tid - C] = scr;
    csync();
    stamp(20);
    // query heads of the group: warp g. New key row: warp GQ, new value row: warp GQ+1.
    if (warp < GQ || ((warp == GQ || warp == GQ + 1) && p >= t0 && p < t0 + nt)) {
      float x[8];
      if (warp == GQ + 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = __ldcg(P.V16 + (size_t)kv * D + lane + 32 * i);
      } else {
        const bool isq = warp < GQ;
        const float *src = isq ? P.Q16 + (size_t)(kv * GQ + warp) * 2 * D : P.K16 + (size_t)kv * D;
        const float *w = isq ? ly.q_norm : ly.k_norm;
        double ss = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          x[i] = __ldcg(src + lane + 32 * i);
          const double dv = (double)x[i];
          ss = ss + dv * dv;
        }
        ss = warp_tree_sum(ss);
        const float inv = 1.0f / sqrtf((float)(ss / (double)D) + P.eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (x[i] * inv) * (1.0f + __ldg(w + lane + 32 * i));
        if (P.rot / 2 == 32) {
          const float cs = P.Cos[(size_t)pos * P.rot + lane], sn = P.Sin[(size_t)pos * P.rot + lane];
          const float x0 = x[0], x1 = x[1];
          x[0] = x0 * cs - x1 * sn;
          x[1] = x0 * sn + x1 * cs;
        }
      }
      if (warp < GQ) {
#pragma unroll
        for (int i = 0; i < 8; ++i) qs[warp * D + lane + 32 * i] = x[i];
      } else {
        // quantise the new row into the staged chunk, then copy it to the cache
        const bool isk = warp == GQ;
        int8_t *srow = reinterpret_cast<int8_t *>(kvs) + (isk ? 0 : C * D) + (p - t0) * D;
        uint16_t *ssc = (isk ? kss : vss) + (p - t0);
        kv_quant_store(x, lane, srow, ssc);
        __syncwarp();
        int8_t *grow = (isk ? ly.Kc : ly.Vc) + ((size_t)p * nKV + kv) * D;
        reinterpret_cast<uint2 *>(grow)[lane] = reinterpret_cast<const uint2 *>(srow)[lane];
        if (lane == 0) ((isk ? ly.Ks : ly.Vs))[(size_t)p * nKV + kv] = *ssc;
      }
    }
    csync();
    stamp(21);
    // scores: warp w takes tokens w, w+16, ...
#pragma unroll 1
    for (int tt = warp; tt < nt; tt += 16) {
      const uint2 kw = reinterpret_cast<const uint2 *>(kvs)[tt * (D / 8) + lane];
      const float ksf = f16_to_f32(kss[tt]);
      float kf[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        kf[j] = (float)(int)(int8_t)((kw.x >> (8 * j)) & 0xFF);
        kf[4 + j] = (float)(int)(int8_t)((kw.y >> (8 * j)) & 0xFF);
      }
      float part[GQ];
#pragma unroll
      for (int g = 0; g < GQ; ++g) {
        const float4 q0 = *reinterpret_cast<const float4 *>(qs + g * D + lane * 8),
                     q1 = *reinterpret_cast<const float4 *>(qs + g * D + lane * 8 + 4);
        float acc = 0.0f;
        acc = fmaf(q0.x, kf[0], acc);
        acc = fmaf(q0.y, kf[1], acc);
        acc = fmaf(q0.z, kf[2], acc);
        acc = fmaf(q0.w, kf[3], acc);
        acc = fmaf(q1.x, kf[4], acc);
        acc = fmaf(q1.y, kf[5], acc);
        acc = fmaf(q1.z, kf[6], acc);
        acc = fmaf(q1.w, kf[7], acc);
        part[g] = acc;
      }
      attn_store_scores<GQ>(part, lane, sc + tt * GQ, ksf, scale);   // one butterfly for all heads
    }
    csync();
    stamp(22);
    if (tid < GQ) {
      float mx = -INFINITY;
      for (int tt = 0; tt < nt; ++tt) mx = fmaxf(mx, sc[tt * GQ + tid]);
      sh->hmax[tid] = mx;
    }
    csync();
    for (int i = tid; i < GQ * nt; i += kCons) sc[i] = det_expf(sc[i] - sh->hmax[i % GQ]);
    csync();
    if (tid < GQ) {
      float se = 0.0f;
      for (int tt = 0; tt < nt; ++tt) se = se + sc[tt * GQ + tid];
      sh->hse[tid] = se;
    }
    csync();
    for (int i = tid; i < GQ * nt; i += kCons) sc[i] = sc[i] * f16_to_f32(vss[i / GQ]);
    csync();
    stamp(23);
    // weighted values: thread (dim, half) accumulates its dim for the heads of its half
    {
      const int dim = tid & 255, g0 = (tid >> 8) * GH;
      float acc[GH];
#pragma unroll
      for (int g = 0; g < GH; ++g) acc[g] = 0.0f;
      const int8_t *vs = reinterpret_cast<const int8_t *>(kvs + C * D) + dim;
      if constexpr (GQ == 8) {   // four heads per half: one 16-byte read gives a token's four weights
#pragma unroll 8
        for (int tt = 0; tt < nt; ++tt) {
          const float v = (float)(int)vs[tt * D];
          const float4 pw = *reinterpret_cast<const float4 *>(sc + tt * GQ + g0);
          acc[0] = fmaf(pw.x, v, acc[0]);
          acc[1] = fmaf(pw.y, v, acc[1]);
          acc[2] = fmaf(pw.z, v, acc[2]);
          acc[3] = fmaf(pw.w, v, acc[3]);
        }
      } else {
#pragma unroll 2
        for (int tt = 0; tt < nt; ++tt) {
          const float v = (float)(int)vs[tt * D];
#pragma unroll
          for (int g = 0; g < GH; ++g)
            if (g0 + g < GQ) acc[g] = fmaf(sc[tt * GQ + g0 + g], v, acc[g]);
        }
      }
#pragma unroll
      for (int g = 0; g < GH; ++g) {
        if (g0 + g < GQ) {
          const size_t slot = (size_t)(kv * GQ + g0 + g) * P.max_chunks + ch;
          P.Pacc[slot * D + dim] = acc[g];
          if (dim == 0) {
            P.Pm[slot] = sh->hmax[g0 + g];
            P.Pse[slot] = sh->hse[g0 + g];
          }
        }
      }
    }
    stamp(24);
    csync();
  }
}
static __device__ __noinline__ void attn_stage(unsigned epoch, const StepLayer &ly, int pos, int T) {
  switch (PL.nQ / PL.nKV) {
    case 1: attn_stage_t<1>(epoch, ly, pos, T); break;
    case 2: attn_stage_t<2>(epoch, ly, pos, T); break;
    case 4: attn_stage_t<4>(epoch, ly, pos, T); break;
    case 6: attn_stage_t<6>(epoch, ly, pos, T); break;
    case 8: attn_stage_t<8>(epoch, ly, pos, T); break;
    default: grid_wait(epoch); break;  // rejected on the host
  }
}

// Ordered merge of the chunk partials of one query head per block (256 threads), sigmoid
// gate, quantiser: AttnCombine's arithmetic (attention_core.cuh).
static __device__ __noinline__ void attn_combine_stage(int T) {
  const StepPlan &P = PL;
  constexpr int D = kHeadDim, C = kAttnChunk;
  if (threadIdx.x >= 256) return;
  float *s_pm = reinterpret_cast<float *>(step_smem + kFbufOff), *s_pf = s_pm + 2048;
  float *wmax = SH->wmax;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nch = (T + C - 1) / C;
#pragma unroll 1
  for (int h = (int)blockIdx.x; h < P.nQ; h += (int)gridDim.x) {
    const float *pm = P.Pm + (size_t)h * P.max_chunks;
    const float *pse = P.Pse + (size_t)h * P.max_chunks;
    const float *pacc = P.Pacc + (size_t)h * P.max_chunks * D;
    const float gate = __ldcg(P.Q16 + (size_t)h * 2 * D + D + tid);
    float M = -INFINITY, se = 0.0f, acc = 0.0f;
    if (nch <= 2048) {
      hsync();
      for (int ch = tid; ch < nch; ch += 256) {
        s_pm[ch] = __ldcg(pm + ch);
        s_pf[ch] = __ldcg(pse + ch);
      }
      hsync();
      for (int ch = 0; ch < nch; ++ch) M = fmaxf(M, s_pm[ch]);
      hsync();
      for (int ch = tid; ch < nch; ch += 256) s_pm[ch] = det_expf(s_pm[ch] - M);
      hsync();
      for (int ch = 0; ch < nch; ++ch) se = fmaf(s_pf[ch], s_pm[ch], se);
#pragma unroll 16
      for (int ch = 0; ch < nch; ++ch) acc = fmaf(__ldcg(pacc + (size_t)ch * D + tid), s_pm[ch], acc);
    } else {
      for (int ch = 0; ch < nch; ++ch) M = fmaxf(M, __ldcg(pm + ch));
      for (int ch = 0; ch < nch; ++ch) {
        const float f = det_expf(__ldcg(pm + ch) - M);
        se = fmaf(__ldcg(pse + ch), f, se);
        acc = fmaf(__ldcg(pacc + (size_t)ch * D + tid), f, acc);
      }
    }
    const float o = acc / se;
    const float y = o / (1.0f + det_expf(-gate));
    float m = warp_max(fabsf(y));
    if (lane == 0) wmax[warp] = m;
    hsync();
    const int g0 = (warp >> 2) * 4;
    m = fmaxf(fmaxf(wmax[g0], wmax[g0 + 1]), fmaxf(wmax[g0 + 2], wmax[g0 + 3]));
    float s = m / 127.0f;
    if (s == 0.0f) s = 1.0f;
    if ((tid & 127) == 0) P.SQ[(size_t)h * 2 + (tid >> 7)] = s;
    P.Q8[(size_t)h * D + tid] = (int8_t)quant_round(y, s);
    hsync();
  }
}

// ------------------------------------------------------------------- MoE stages ---
static __device__ __noinline__ uint32_t gateup_stage(uint32_t tile) {
  const StepPlan &P = PL;
  const int H = P.H, I = P.I;
  int lo, hi;
  deal(P.slots * I, row_unit(H), (int)blockIdx.x, (int)gridDim.x, lo, hi);
  if (lo >= hi) return tile;
  float *T = reinterpret_cast<float *>(step_smem + kTOff);
  unsigned char *act = step_smem + kActOff;
  const int np = hi - lo, G = H >> 7;
  tile = dot_tiles(tile, H, reinterpret_cast<const uint4 *>(act), reinterpret_cast<const float *>(act + H), T, 0, 2 * np,
                   2 * np, 0);
  csync();
  // the producer streams, slot by slot, the slot's gate rows and then its up rows: the pair row
  // lo + r of slot s (rows a .. a + n - 1 of the share belong to it) has its gate term at
  // 2 (a - lo) + i and its up term n rows later
  for (int r = threadIdx.x; r < np; r += kCons) {
    const int s = (lo + r) / I;
    const int a = lo > s * I ? lo : s * I, b = hi < (s + 1) * I ? hi : (s + 1) * I;
    const int n = b - a, i = lo + r - a, fg = 2 * (a - lo) + i;
    const float g = row_sum_rt(T, fg, G), u = row_sum_rt(T, fg + n, G);
    P.Act[lo + r] = silu_mul(g, u);
  }
  return tile;
}

static __device__ __noinline__ uint32_t down_stage(uint32_t tile, int L) {
  const StepPlan &P = PL;
  const int H = P.H, I = P.I;
  int lo, hi;
  deal(H, row_unit(I), (int)blockIdx.x, (int)gridDim.x, lo, hi);
  quant_rows(P.Act, I, P.slots);
  stamp(2);
  if (lo >= hi) return tile;
  // residual input of this block's rows: in flight while the tiles are dotted (dot_tiles is inlined)
  float res0 = 0.0f;
  if (lo + (int)threadIdx.x < hi) res0 = __ldcg(P.Tmp + lo + threadIdx.x);
  float *T = reinterpret_cast<float *>(step_smem + kTOff);
  unsigned char *act = step_smem + kActOff;
  tile = dot_tiles(tile, I, reinterpret_cast<const uint4 *>(act), reinterpret_cast<const float *>(act + (size_t)P.slots * I), T,
                   0, P.slots * (hi - lo), P.slots * (hi - lo), hi - lo);
  csync();
  const int nr = hi - lo, G = I >> 7;
  for (int r = threadIdx.x; r < nr; r += kCons) {
    const float res = r < kCons ? res0 : __ldcg(P.Tmp + lo + r);
    float acc = 0.0f;
    for (int s = 0; s < P.slots; ++s) acc = acc + SH->sel_w[s] * row_sum_rt(T, s * nr + r, G);
    const float x = res + acc;
    P.X[lo + r] = x;
    if (P.layer_out) P.layer_out[(size_t)L * H + lo + r] = x;
  }
  return tile;
}

// LM head in sub-blocks of 16 tiles (t[][] holds 256 rows of K = 2048), running argmax per thread.
static __device__ __noinline__ uint32_t lm_head_stage(uint32_t tile, float &bv, int &bi) {
  const StepPlan &P = PL;
  const int K = P.H, G = K >> 7;
  int lo, hi;
  deal(P.vocab, row_unit(K), (int)blockIdx.x, (int)gridDim.x, lo, hi);
  float *T = reinterpret_cast<float *>(step_smem + kTOff);
  unsigned char *act = step_smem + kActOff;
  const int sub = kTCap / G;  // rows whose terms fit t[][]: a whole number of tiles
#pragma unroll 1
  for (int base = 0; base < hi - lo; base += sub) {
    const int nrows = (hi - lo) - base < sub ? (hi - lo) - base : sub;
    tile = dot_tiles(tile, K, reinterpret_cast<const uint4 *>(act), reinterpret_cast<const float *>(act + K), T, base, nrows,
                     hi - lo, 0);
    csync();
    for (int r = threadIdx.x; r < nrows; r += kCons) {
      const float v = row_sum_rt(T, r, G);
      const int n = lo + base + r;
      P.Logits[n] = v;
      argmax_merge(bv, bi, v, n);
    }
    csync();
  }
  return tile;
}

// Block-wide first-max-wins argmax over the consumer threads; result valid in thread 0.
static __device__ __noinline__ void cons_argmax(float &bv, int &bi) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
    argmax_merge(bv, bi, __shfl_xor_sync(kFull, bv, off), __shfl_xor_sync(kFull, bi, off));
  if (lane == 0) {
    SH->av[warp] = bv;
    SH->ai[warp] = bi;
  }
  csync();
  if (warp == 0) {
    bv = lane < 16 ? SH->av[lane] : -INFINITY;
    bi = lane < 16 ? SH->ai[lane] : 0x7FFFFFFF;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      argmax_merge(bv, bi, __shfl_xor_sync(kFull, bv, off), __shfl_xor_sync(kFull, bi, off));
  }
}

static __device__ __noinline__ void consumer_main(int mode) {
  const StepPlan &P = PL;
  StepShared *sh = SH;
  const int H = P.H, tid = threadIdx.x;
  uint32_t tile = 0;   // running index of the next ring tile to consume
  unsigned epoch = 0;  // grid barriers this block has arrived at
  const int token = __ldcg(P.ctrl + CTRL_TOKEN), pos = __ldcg(P.ctrl + CTRL_POS);
  int T = __ldcg(P.ctrl + CTRL_LEN);
  if (T > P.max_ctx) T = P.max_ctx;
  const int tok = token < 0 ? 0 : (token >= P.vocab ? P.vocab - 1 : token);
  float *hn = reinterpret_cast<float *>(step_smem + kFbufOff) + 4096;

  for (int L = 0; L < P.layers; ++L) {
    // the layer's record into shared memory (the previous layer's is no longer read: every
    // consumer has passed the grid barrier that ended it)
    {
      const uint4 *src = reinterpret_cast<const uint4 *>(P.L + L);
      if (tid < (int)(sizeof(StepLayer) / 16)) reinterpret_cast<uint4 *>(&sh->ly)[tid] = __ldg(src + tid);
      csync();
    }
    const StepLayer &ly = sh->ly;
    const bool lin = ly.type == 0;
    // ---- stage 1: input norm + quantiser, first projections ----
    norm_quant(P.X, L == 0 ? P.emb + (size_t)tok * H : nullptr, ly.in_norm, H, nullptr,
               (L == 0 && (int)blockIdx.x == 0) ? P.X : nullptr);
    stamp(2);
    tile = gemv_stage_run(tile, &ly.m[0], lin ? 4 : 3, H);
    stamp(3);
    grid_arrive();
    ++epoch;
    if (lin) {
      // ---- stage 2: gated delta rule ----
      deltanet_stage(epoch, ly);  // waits for the barrier inside, after its state loads
      grid_arrive();
    ++epoch;
      grid_wait(epoch);
      // ---- stage 3: gated norm, out_proj + residual ----
      stamp(4);
      gated_norm_quant(P.O, P.Z, ly.lin_norm, P.nV);
      stamp(2);
      tile = gemv_stage_run(tile, &ly.m[4], 1, P.nV * 128);
      stamp(3);
    } else {
      attn_stage(epoch, ly, pos, T);  // waits for the barrier inside, after its KV loads
      grid_arrive();
    ++epoch;
      grid_wait(epoch);
      attn_combine_stage(T);
      grid_arrive();
    ++epoch;
      grid_wait(epoch);
      stage_q8(P.Q8, P.SQ, P.nQ * 256);
      tile = gemv_stage_run(tile, &ly.m[4], 1, P.nQ * 256);
    }
    grid_arrive();
    ++epoch;
    grid_wait(epoch);
    // ---- stage 4: post norm + quantiser (kept staged for the experts), router logits ----
    norm_quant(P.Tmp, nullptr, ly.post_norm, H, hn, nullptr);
    stamp(2);
    tile = router_stage(tile, hn, H, P.E + (ly.shared_gate ? 1 : 0));
    stamp(3);
    grid_arrive();
    ++epoch;
    grid_wait(epoch);
    // ---- stage 5: selection, expert gate/up ----
    router_select_cons(P.E, P.topk, ly.shared_gate != nullptr);
    stamp(5);
    if (tid < P.slots * 3) {
      const uint4 *src = reinterpret_cast<const uint4 *>(ly.experts + sh->sel_idx[tid / 3]) + tid % 3;
      reinterpret_cast<uint4 *>(sh->sew + tid / 3)[tid % 3] = __ldg(src);
    }
    csync();
    if (tid == 0) mbar_arrive(&sh->sel_bar);  // the producer may now stream the experts
    stamp(6);
    if ((int)blockIdx.x == 0 && tid <= P.topk) {
      P.SelIdx[tid] = sh->sel_idx[tid];
      P.SelW[tid] = sh->sel_w[tid];
      if (tid == 0) *P.NearGap = sh->gap;
      if (P.routed) {
        P.routed[(size_t)L * (P.topk + 1) + tid] = sh->sel_idx[tid];
        if (tid == 0) P.near_gap[L] = sh->gap;
      }
    }
    tile = gateup_stage(tile);
    stamp(3);
    grid_arrive();
    ++epoch;
    grid_wait(epoch);
    // ---- stage 6: expert down, combine, residual ----
    tile = down_stage(tile, L);
    stamp(3);
    grid_arrive();
    ++epoch;
    grid_wait(epoch);
  }

  if (mode == 0) {
    // prompt step: no logits; move on to the next prompt id
    if ((int)blockIdx.x == 0 && tid == 0) {
      const int np = pos + 1;
      P.ctrl[CTRL_POS] = np;
      P.ctrl[CTRL_LEN] = P.ctrl[CTRL_LEN] + 1;
      if (np < P.max_ctx) P.ctrl[CTRL_TOKEN] = P.ids[np];
      P.ctrl[CTRL_SELECTED] = -1;
    }
    return;
  }
  // ---- tail: final norm, LM head, first-max-wins argmax, control update ----
  norm_quant(P.X, nullptr, P.final_norm, H, nullptr, nullptr);
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  tile = lm_head_stage(tile, bv, bi);
  cons_argmax(bv, bi);
  if (tid == 0) {
    P.PV[(int)blockIdx.x] = bv;
    P.PI[(int)blockIdx.x] = bi;
  }
  grid_arrive();
    ++epoch;
  grid_wait(epoch);
  if ((int)blockIdx.x == 0) {
    bv = -INFINITY;
    bi = 0x7FFFFFFF;
    for (int i = tid; i < (int)gridDim.x; i += kCons) argmax_merge(bv, bi, __ldcg(P.PV + i), __ldcg(P.PI + i));
    csync();
    cons_argmax(bv, bi);
    if (tid == 0) {
      P.out_tok[0] = bi;
      if (P.history && P.history_cap > 0) P.history[pos % P.history_cap] = bi;
      P.ctrl[CTRL_SELECTED] = bi;
      P.ctrl[CTRL_TOKEN] = bi;
      P.ctrl[CTRL_POS] = pos + 1;
      P.ctrl[CTRL_LEN] = P.ctrl[CTRL_LEN] + 1;
    }
  }
}

__global__ void __launch_bounds__(kStepThreads, 1) DecodeStep(const DecodeStepArgs args) {
  StepShared *sh = SH;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kNT; ++i) {
      mbar_init(&sh->full[i], 1);
      mbar_init(&sh->empty[i], kCons / 32);  // one arrival per consumer warp
    }
    mbar_init(&sh->sel_bar, 1);
    sh->fail = 0;
    sh->nstamp[0] = 0;
    sh->nstamp[1] = 0;
    sh->nseg = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < sizeof(StepPlan) / 16)
    reinterpret_cast<uint4 *>(&sh->plan)[threadIdx.x] = __ldg(reinterpret_cast<const uint4 *>(args.plan) + threadIdx.x);
  __syncthreads();
  if (*(volatile int *)PL.error != 0) return;  // a previous launch failed: stay out
  if (threadIdx.x >= kCons) {
    const uint32_t issued = producer_main(args.mode);
    // Nothing may still be landing in this block's shared memory when it retires: every slot
    // owner waits (bounded) for the last tile it issued. In a run without faults the consumers
    // have waited for all of them already.
    const uint32_t lane = threadIdx.x & 31;
    if (lane < (uint32_t)kNT && issued > lane) {
      const uint32_t t = issued - 1u - ((issued - 1u - lane) % kNT);  // latest tile issued into slot `lane`
      const long long t0 = clock64();
      while (!mbar_try(&sh->full[lane], (t / kNT) & 1u))
        if (clock64() - t0 > kWaitCycles) break;
    }
    return;
  }
  consumer_main(args.mode);
}

static uint32_t step_smem_fn(const void *) { return (uint32_t)kStepSmemBytes; }

#define F(f) AINFER_ARG(DecodeStepArgs, f)
AINFER_REGISTER_COOP(DecodeStep, DecodeStepArgs, kStepThreads, 0, 0, step_smem_fn, F(plan), F(mode));
#undef F

}  // namespace ainfer
