// Int4GemmA8Tc: W4A8 group-128 GEMM for a batch of 1..64 activation rows on the 5th-generation
// tensor cores (tcgen05.mma kind::i8, accumulators in tensor memory), weights streamed ONCE
// whatever the batch. This is the batched form of the reference's Int4Gemv
// (tools/cmdlist/kernels.cpp:148-193; sweep protocol tools/gemv/gemv.cpp:503-601): per output
// row and batch entry, the exact int32 sum of the 128 nibble x int8 products of a group, then
// acc = acc + ((float)sum * weight_scale) * activation_scale[g] in ascending group order. The
// integer sums are exact on any hardware and the fp32 order is the reference's, so every batch
// entry is bit-identical to the one-row GEMV.
//
// One block = 128 threads = 128 weight rows (thread r owns row r of the block's row tile and,
// in the epilogue, lane r of the accumulator). Per group of 128 weights:
//   * every thread fetches its row's 64 packed bytes (the next group's are in flight while this
//     one is worked on) and widens them to INT8 in shared memory in the tensor core's K-major
//     core-matrix layout (8 rows x 16 bytes per core matrix). A nibble moved to the top of its
//     byte is the signed byte 16 * v, so no sign fix-up is needed; the sum comes out 16 times
//     too large and is shifted back (exact). Low and high nibbles of a word go to separate
//     words, which permutes k inside the group; the activations are stored with the same
//     permutation (the dot product does not care).
//   * the batch's INT8 activations of that group are copied next to it (rows beyond the batch
//     stay zero);
//   * one thread issues four tcgen05.mma (M = 128 rows, N = padded batch, K = 32 each) into
//     separate accumulators of one of two buffers in tensor memory (so that they pipeline) and
//     commits them to an mbarrier;
//   * while those run, all threads finish the PREVIOUS group: wait for its mbarrier, read their
//     lane of the accumulator with tcgen05.ld, rescale and add.
// Every wait is bounded; a wait that runs out stores a code in the host-visible fault word and
// the kernel ends (with the tensor memory freed).
#include "block_dot.cuh"

namespace ainfer {

struct Int4GemmA8TcArgs {
  const uint8_t *P;    // packed nibbles [N][K/2]
  const uint16_t *S;   // bf16 scales [N][K/128]
  const int8_t *XQ;    // [M][K] activations
  const float *SQ;     // [M][K/128] activation group scales
  float *Y;            // [M][ldy]
  int32_t N, K, M, ldy;
};

constexpr int kTcRows = 128;               // weight rows per block tile = accumulator lanes
constexpr int kTcMaxBatch = 64;
constexpr int kTcABytes = kTcRows * 128;   // one group of 128 rows as INT8
constexpr uint32_t kTcSpin = 1u << 22;

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_byte_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  // shared-memory matrix descriptor, no swizzle, K-major: start address, leading-dimension
  // byte offset (between the two 16-byte K chunks of one MMA), stride byte offset (between
  // 8-row core matrices), all in units of 16 bytes; descriptor version 1.
  return (uint64_t)((smem_byte_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}

extern __shared__ __align__(128) unsigned char tc_smem[];


__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst_smem)), "l"(src) : "memory");
}

// Shared-memory map: two stages of packed weights [128 rows][gps * 64 B] (16-byte pieces of a
// row swizzled by the row number, so that the row owners' reads spread over the banks), two
// stages of raw activations [gps][M][128 B], A (INT8 weights) [2][8 chunks][16 row blocks]
// [8 rows][16 B], B (INT8 activations) [2][8 chunks][Npad/8 blocks][8 rows][16 B], activation
// scales [M][G] fp32. gps (4, 2 or 1, dividing G) groups travel together: consecutive threads copy
// consecutive 16-byte pieces of the same row, so a warp's copy instruction reads two rows of 256
// contiguous bytes (row-sized bursts instead of one 64-byte piece from each of 32 rows, which
// left HBM at well under half its rate).
__global__ void __launch_bounds__(128) Int4GemmA8Tc(const Int4GemmA8TcArgs a) {
  __shared__ unsigned long long mma_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t s_fail;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int K = a.K, G = K >> 7, M = a.M;
  const int gps = (G & 3) == 0 ? 4 : ((G & 1) == 0 ? 2 : 1), QT = G / gps;   // groups per stage (divides G), stages per row tile
  const int ppr = gps * 4;                                    // 16-byte pieces per row and stage
  const int Npad = M <= 8 ? 8 : ((M + 15) & ~15);            // batch padded to a legal MMA N
  const uint32_t b_chunk = (uint32_t)Npad * 16u, b_bytes = 8u * b_chunk;
  const uint32_t w_stage = (uint32_t)kTcRows * (uint32_t)gps * 64u, x_stage = ((uint32_t)(gps * M) * 128u + 127u) & ~127u;
  unsigned char *Wst = tc_smem;
  unsigned char *Xst = Wst + 2 * w_stage;
  unsigned char *Abuf = Xst + 2 * x_stage;
  unsigned char *Bbuf = Abuf + 2 * kTcABytes;
  float *sqs = reinterpret_cast<float *>(Bbuf + 2 * b_bytes);
  // The four K = 32 products of a group accumulate into one accumulator (they are off the
  // critical path: the block works on the next group's bytes while they run).
  const int nacc = 1;
  const uint32_t buf_cols = (uint32_t)(nacc * Npad);
  uint32_t tmem_cols = 32;
  while (tmem_cols < 2u * buf_cols) tmem_cols <<= 1;
  // instruction descriptor: D = S32, A = B = signed 8 bit, both K-major, N = Npad, M = 128
  const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(Npad >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);

  if (tid == 0) {
    mbar_init(&mma_bar[0], 1);
    mbar_init(&mma_bar[1], 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // activation rows beyond the batch must read as zero: clear both B buffers once
  for (uint32_t i = tid; i < 2u * b_bytes / 16u; i += 128) reinterpret_cast<uint4 *>(Bbuf)[i] = make_uint4(0, 0, 0, 0);
  for (int i = tid; i < M * G; i += 128) sqs[i] = __ldg(a.SQ + i);
  if (warp == 0) {  // tensor memory: two buffers of nacc accumulators of Npad columns each
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t a_addr = smem_addr(Abuf), b_addr = smem_addr(Bbuf);
  uint32_t use0 = 0u, use1 = 0u;  // completed uses of the two accumulator buffers (parity of their barriers)

  // The block's work: its row tiles in turn; a tile is QT stages of gps groups; a stage is
  // fetched while the previous one is worked on; inside a stage one step per group. The loop
  // bookkeeping is kept in counters (no divisions): the kernel is bound by instruction issue,
  // not by the tensor core, so every instruction per step counts.
  const int ntiles = (a.N + kTcRows - 1) / kTcRows;
  const int lg_ppr = 31 - __clz(ppr);
  const int f_pc = tid & (ppr - 1), f_r0 = tid >> lg_ppr, f_rstep = 128 >> lg_ppr;  // this thread's piece and rows in a fetch
  const size_t row_bytes = (size_t)(K >> 1);
  auto fetch = [&](int t, int q, int stage) {   // stage (tile t, quad q) into buffer `stage`; t >= ntiles: nothing
    if (t < ntiles) {
      unsigned char *wd = Wst + stage * w_stage;
      const int rlast = a.N - 1 - t * kTcRows;   // rows past the end repeat the last row (not stored)
      const uint8_t *src0 = a.P + (size_t)(t * kTcRows) * row_bytes + (size_t)q * (gps * 64) + f_pc * 16;
#pragma unroll 4
      for (int r = f_r0; r < kTcRows; r += f_rstep) {
        const int rr = r < rlast ? r : rlast;
        cp_async16(wd + r * (gps * 64) + ((f_pc ^ (r & (ppr - 1))) << 4), src0 + (size_t)rr * row_bytes);
      }
      unsigned char *xd = Xst + stage * x_stage;
      for (int idx = tid; idx < gps * M * 8; idx += 128) {  // [group][m][8 pieces]
        const int gl = idx / (M * 8), rem = idx - gl * (M * 8);
        cp_async16(xd + idx * 16, a.XQ + (size_t)(rem >> 3) * K + (size_t)(q * gps + gl) * 128 + (rem & 7) * 16);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // the row's weight scales: bf16 [G], fetched one tile ahead into registers (G <= 32), parked in
  // shared memory at the tile boundary
  uint16_t *ssc = reinterpret_cast<uint16_t *>(sqs + M * G) + tid * G;   // this thread's G scales of the current tile
  auto load_scales = [&](int t, uint32_t (&regs)[16]) {
    if (t < ntiles) {
      const int row = t * kTcRows + tid < a.N ? t * kTcRows + tid : a.N - 1;
      const uint16_t *sp = a.S + (size_t)row * G;
      if ((G & 1) == 0) {
#pragma unroll
        for (int k = 0; k < 16; ++k)
          if (2 * k < G) regs[k] = __ldg(reinterpret_cast<const uint32_t *>(sp) + k);
      } else {
        regs[0] = __ldg(sp);
      }
    }
  };
  auto park_scales = [&](const uint32_t (&regs)[16]) {
    if ((G & 1) == 0) {
#pragma unroll
      for (int k = 0; k < 16; ++k)
        if (2 * k < G) reinterpret_cast<uint32_t *>(ssc)[k] = regs[k];
    } else {
      ssc[0] = (uint16_t)regs[0];
    }
  };

  float acc[kTcMaxBatch];
#pragma unroll
  for (int m = 0; m < kTcMaxBatch; ++m) acc[m] = 0.0f;
  uint32_t sregs[16];
  int t = (int)blockIdx.x;
  const bool sc_smem = G <= 32;   // longer rows read their scales from global memory at use
  if (sc_smem) {
    load_scales(t, sregs);
    park_scales(sregs);
    load_scales(t + (int)gridDim.x, sregs);
  }
  fetch(t, 0, 0);
  int stage = 0;        // buffer of the stage being worked on
  int buf = 0;          // accumulator / staging buffer of the step being staged
  int have_prev = 0, prev_g = 0, prev_t = 0;   // the step whose products are in flight
#pragma unroll 1
  for (; t < ntiles || have_prev; t += (int)gridDim.x) {
    const bool live = t < ntiles;
#pragma unroll 1
    for (int q = 0; q < (live ? QT : 1); ++q) {
      if (live) {
        // next stage: the next quad of this tile, or the first of the block's next tile
        const bool last_q = q + 1 == QT;
        fetch(last_q ? t + (int)gridDim.x : t, last_q ? 0 : q + 1, stage ^ 1);
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();  // every thread's copies of this stage have landed
      }
#pragma unroll 1
      for (int gl = 0; gl < (live ? gps : 1); ++gl) {
        if (live) {
          // ---- stage this step: the row's 128 weights as INT8 (16 * v), and the batch's activations ----
          const unsigned char *wrow = Wst + stage * w_stage + tid * (gps * 64);
          unsigned char *ab = Abuf + buf * kTcABytes + (tid >> 3) * 128 + (tid & 7) * 16;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const uint4 cur = *reinterpret_cast<const uint4 *>(wrow + (((gl * 4 + jj) ^ (tid & (ppr - 1))) << 4));
            // packed words (x, y) -> chunk 2jj, (z, w) -> chunk 2jj + 1: [low nibbles, high nibbles] per word
            const uint4 c0 = make_uint4((cur.x << 4) & 0xF0F0F0F0u, cur.x & 0xF0F0F0F0u, (cur.y << 4) & 0xF0F0F0F0u, cur.y & 0xF0F0F0F0u);
            const uint4 c1 = make_uint4((cur.z << 4) & 0xF0F0F0F0u, cur.z & 0xF0F0F0F0u, (cur.w << 4) & 0xF0F0F0F0u, cur.w & 0xF0F0F0F0u);
            *reinterpret_cast<uint4 *>(ab + (2 * jj) * 2048) = c0;
            *reinterpret_cast<uint4 *>(ab + (2 * jj + 1) * 2048) = c1;
          }
          const unsigned char *xg = Xst + stage * x_stage + gl * (M * 128);
          for (int qq = tid; qq < M * 8; qq += 128) {
            const int m = qq >> 3, c = qq & 7;
            const uint4 v = *reinterpret_cast<const uint4 *>(xg + qq * 16);
            const uint4 pp = make_uint4(__byte_perm(v.x, v.y, 0x6420), __byte_perm(v.x, v.y, 0x7531), __byte_perm(v.z, v.w, 0x6420),
                                        __byte_perm(v.z, v.w, 0x7531));
            *reinterpret_cast<uint4 *>(Bbuf + buf * b_bytes + c * b_chunk + (m >> 3) * 128 + (m & 7) * 16) = pp;
          }
          // generic-proxy writes -> visible to the tensor core's reads, then everyone has written
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncthreads();
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (tid == 0) {
            const uint32_t d = tmem_base + (uint32_t)buf * buf_cols;
#pragma unroll
            for (int qq = 0; qq < 4; ++qq) {
              const uint64_t da = umma_desc(a_addr + buf * kTcABytes + qq * 2 * 2048, 2048u, 128u);
              const uint64_t db = umma_desc(b_addr + buf * b_bytes + qq * 2 * b_chunk, b_chunk, 128u);
              umma_i8(d, da, db, idesc, qq > 0 ? 1u : 0u);
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&mma_bar[buf]))
                         : "memory");
          }
        }
        if (have_prev) {
          // ---- finish the previous step (group prev_g of tile prev_t), whose products ran meanwhile ----
          const int pb = buf ^ 1;
          const uint32_t par = (pb ? use1 : use0) & 1u;
          bool ok = mbar_try(&mma_bar[pb], par);
          for (uint32_t n = 0; !ok && n < kTcSpin && !*reinterpret_cast<volatile uint32_t *>(&s_fail); ++n) ok = mbar_try(&mma_bar[pb], par);
          if (!ok) {
            s_fail = 1;
            if (g_stream_fault_word) *reinterpret_cast<volatile unsigned int *>(g_stream_fault_word) = 1;
          }
          if (pb) use1 += 1; else use0 += 1;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const int prow = prev_t * kTcRows + tid < a.N ? prev_t * kTcRows + tid : a.N - 1;
          const float sc = bf16_to_f32(sc_smem ? ssc[prev_g] : __ldg(a.S + (size_t)prow * G + prev_g));
          const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)pb * buf_cols;
          const float *sqg = sqs + prev_g;
#pragma unroll
          for (int m0 = 0; m0 < kTcMaxBatch; m0 += 8) {
            if (m0 < M) {  // uniform across the block
              int32_t v[8];
              tmem_ld8(taddr + (uint32_t)m0, v);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
              for (int jj = 0; jj < 8; ++jj)
                if (m0 + jj < M) acc[m0 + jj] = acc[m0 + jj] + ((float)(v[jj] >> 4) * sc) * sqg[(m0 + jj) * G];
            }
          }
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          if (prev_g == G - 1) {
            // the row tile is complete: store it, start the next one from zero, and switch to the
            // next tile's scales (prefetched when this tile began)
            const bool in_range = prev_t * kTcRows + tid < a.N;
#pragma unroll
            for (int m = 0; m < kTcMaxBatch; ++m) {
              if (m < M && in_range) a.Y[(size_t)m * a.ldy + prev_t * kTcRows + tid] = acc[m];
              acc[m] = 0.0f;
            }
            if (sc_smem) {
              park_scales(sregs);
              load_scales(prev_t + 2 * (int)gridDim.x, sregs);
            }
          }
        }
        if (live) {
          have_prev = 1;
          prev_g = q * gps + gl;
          prev_t = t;
          buf ^= 1;
        } else {
          have_prev = 0;
        }
      }
      if (live) stage ^= 1;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
}

static uint32_t tc_smem_fn(const void *args) {
  const Int4GemmA8TcArgs *a = (const Int4GemmA8TcArgs *)args;
  const uint32_t M = (uint32_t)a->M, G = (uint32_t)a->K >> 7, gps = (G & 3) == 0 ? 4u : ((G & 1) == 0 ? 2u : 1u);
  const uint32_t Npad = M <= 8 ? 8 : ((M + 15) & ~15u);
  return 2 * kTcRows * gps * 64 + 2 * ((gps * M * 128u + 127u) & ~127u) + 2 * kTcABytes + 2 * 8 * Npad * 16 + M * G * 4 +
         kTcRows * G * 2;
}

#define F(f) AINFER_ARG(Int4GemmA8TcArgs, f)
AINFER_REGISTER(Int4GemmA8Tc, Int4GemmA8TcArgs, 128, 0, 0, tc_smem_fn, F(P), F(S), F(XQ), F(SQ), F(Y), F(N), F(K), F(M), F(ldy));
#undef F

}  // namespace ainfer
