// Int4GemmA8Tc / Int4GemmA8TcGrouped: W4A8 group-128 GEMM for batches of 1..64 activation rows
// on the 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators in tensor memory),
// weights streamed ONCE whatever the batch. This is the batched form of the reference's Int4Gemv
// (tools/cmdlist/kernels.cpp:148-193; sweep protocol tools/gemv/gemv.cpp:503-601): per output
// row and batch entry, the exact int32 sum of the 128 nibble x int8 products of a group, then
// acc = acc + ((float)sum * weight_scale) * activation_scale[g] in ascending group order. The
// integer sums are exact on any hardware and the fp32 order is the reference's, so every batch
// entry is bit-identical to the one-row GEMV.
//
// The grouped form runs a list of problems of the same shape (N, K) in one launch: problem i has
// its own weight matrix and its own range of activation rows (an expert and the tokens routed to
// it). The list and its length live in device memory, so routing never goes through the host.
//
// One block = 256 threads = 128 weight rows x 2 halves. Thread (r, h) owns row r of the block's
// row tile: it widens half of the row's packed bytes of a group and, in the epilogue, handles
// half of the batch columns of accumulator lane r. Per group of 128 weights (one step):
//   * the row tile's packed bytes arrive by cp.async, four groups (256 contiguous bytes per row)
//     per stage, two stages; the next stage is in flight while this one is worked on;
//   * every thread widens its 32 bytes to INT8 in shared memory in the tensor core's K-major
//     core-matrix layout (8 rows x 16 bytes per core matrix). A nibble moved to the top of its
//     byte is the signed byte 16 * v, so no sign fix-up is needed; the sum comes out 16 times
//     too large and is shifted back (exact). Low and high nibbles of a word go to separate
//     words, which permutes k inside the group; the activations are stored with the same
//     permutation (the dot product does not care);
//   * the batch's INT8 activations of that group (fetched into registers one step earlier) are
//     stored next to it;
//   * one thread issues four tcgen05.mma (M = 128 rows, N = padded batch, K = 32 each) into one
//     of two accumulator buffers in tensor memory and commits them to an mbarrier;
//   * while those run, all threads finish the PREVIOUS step: wait for its mbarrier, read their
//     lane of the accumulator with tcgen05.ld, rescale and add.
// The kernel is bound by instruction issue, not by the tensor core or by memory: the loop keeps
// its bookkeeping in counters and per-tile records in shared memory.
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

// One problem of a grouped launch: Y[x_row0 + m][y_col + n] = sum_k W[n][k] * X[x_row0 + m][k].
struct TcGroup {
  const uint8_t *P;    // packed nibbles [N][K/2]
  const uint16_t *S;   // bf16 scales [N][K/128]
  int32_t x_row0;      // first activation / output row
  int32_t M;           // rows (1..64)
  int32_t y_col;       // first output column
  int32_t pad;
};
static_assert(sizeof(TcGroup) == 32, "two 16-byte loads");
struct Int4GemmA8TcGroupedArgs {
  const TcGroup *Groups;       // [*NGroups] problems
  const int32_t *NGroups;      // device word: number of problems (0 allowed)
  const int8_t *XQ;            // [rows][K]
  const float *SQ;             // [rows][K/128]
  float *Y;                    // [rows][ldy]
  int32_t N, K, max_m, ldy;    // max_m: upper bound of every problem's M (sizes shared memory)
};

constexpr int kTcRows = 128;               // weight rows per block tile = accumulator lanes
constexpr int kTcThreads = 256;
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
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, int32_t (&v)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "r"(taddr)
               : "memory");
}

#ifndef TC_STAMP
#define TC_STAMP(id)   // stand-alone timing builds record a clock here
#define TC_STAMP_DECL
#endif

extern __shared__ __align__(128) unsigned char tc_smem[];

__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void *dst_smem, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr(dst_smem)), "l"(src) : "memory");
}

// A row tile of a problem, as the block's loop needs it (kept in a ring of eight in shared memory).
struct TcTile {
  const uint8_t *P;    // first packed row of the tile
  const uint16_t *S;   // scales of the problem's row 0
  int32_t x_row0, M, y_col, row0;
};
static_assert(sizeof(TcTile) == 32, "ring slot");

struct TcShape {
  const TcGroup *groups;   // null: the one problem `single`
  TcGroup single;
  const int8_t *XQ;
  const float *SQ;
  float *Y;
  int32_t N, K, ldy, max_m, ntiles;
};

__host__ __device__ inline uint32_t tc_npad(uint32_t M) { return M <= 8u ? 8u : ((M + 15u) & ~15u); }
// Buffers of per-tile scales. A step is finished two steps after it was staged, so a tile's scales
// are still read during the first two steps that follow it, while the scales of later tiles
// already arrive (with the first stage of their weights, one stage ahead).
__host__ __device__ inline uint32_t tc_nsc(uint32_t G) { return G == 1 ? 4u : ((G & 3u) == 0 && G >= 8 ? 2u : 3u); }
__host__ __device__ inline uint32_t tc_gps(uint32_t G) { return (G & 3u) == 0 ? 4u : ((G & 1u) == 0 ? 2u : 1u); }
// Shared-memory map: the ring of tile records, two stages of packed weights [128 rows][gps * 64 B] (16-byte pieces of a row
// swizzled by the row number, so that the row owners' reads spread over the banks), A (INT8
// weights) [2][8 chunks][16 row blocks][8 rows][16 B], B (INT8 activations) [2][8 chunks]
// [Npad/8 blocks][8 rows][16 B], per tile the activation scales [max_m][G] fp32 and the row
// tile's weight scales [128][G] bf16 (two to four buffers of each, see tc_nsc). gps (4, 2 or 1, dividing G) groups travel together: consecutive
// threads copy consecutive 16-byte pieces of the same row, so a warp's copy instruction reads
// rows of 256 contiguous bytes (one 64-byte piece from each of 32 rows left HBM at well under
// half its rate).
__host__ __device__ inline uint32_t tc_smem_bytes(uint32_t K, uint32_t max_m) {
  const uint32_t G = K >> 7, gps = tc_gps(G), npad = tc_npad(max_m);
  const uint32_t nsc = tc_nsc(G);
  return 2 * kTcRows * gps * 64 + 2 * kTcABytes + 2 * 8 * npad * 16 + nsc * max_m * G * 4 + nsc * kTcRows * G * 2 +
         8 * (uint32_t)sizeof(TcTile);
}

__device__ __forceinline__ void tc_body(const TcShape &c) {
  __shared__ unsigned long long mma_bar[3];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t s_fail;
  const int tid = threadIdx.x, warp = tid >> 5, r = tid & 127, h = tid >> 7;
  TC_STAMP_DECL;
  const int K = c.K, G = K >> 7;
  const int gps = (int)tc_gps((uint32_t)G), QT = G / gps;     // groups per stage, stages per row tile
  const int ppr = gps * 4, lg_ppr = 31 - __clz(ppr);           // 16-byte pieces per row and stage
  const int npad_max = (int)tc_npad((uint32_t)c.max_m);
  const uint32_t w_stage = (uint32_t)kTcRows * (uint32_t)gps * 64u, b_bytes = 8u * (uint32_t)npad_max * 16u;
  TcTile *ring = reinterpret_cast<TcTile *>(tc_smem);                    // [8]
  unsigned char *Wst = tc_smem + 8 * sizeof(TcTile);
  unsigned char *Abuf = Wst + 2 * w_stage;
  unsigned char *Bbuf = Abuf + 2 * kTcABytes;
  const int nsc = (int)tc_nsc((uint32_t)G);                              // scale buffers (tile number mod nsc)
  const int sq_stride = c.max_m * G, sc_stride = kTcRows * G;
  float *sqs = reinterpret_cast<float *>(Bbuf + 2 * b_bytes);            // [nsc][max_m * G]
  uint16_t *ssc = reinterpret_cast<uint16_t *>(sqs + nsc * sq_stride);   // [nsc][128][G]
  uint32_t tmem_cols = 32;
  while (tmem_cols < 3u * (uint32_t)npad_max) tmem_cols <<= 1;
  const int tpg = (c.N + kTcRows - 1) / kTcRows;   // row tiles per problem
  const size_t row_bytes = (size_t)(K >> 1);
  const int ntiles = c.ntiles, stride = (int)gridDim.x;

  // record of the block's n-th tile (global tile blockIdx.x + n * gridDim.x), from a problem record
  auto make_tile = [&](int t, const TcGroup &g) {
    const int rt = t % tpg;
    TcTile ti;
    ti.P = g.P + (size_t)rt * kTcRows * row_bytes;
    ti.S = g.S;
    ti.x_row0 = g.x_row0; ti.M = g.M; ti.y_col = g.y_col; ti.row0 = rt * kTcRows;
    return ti;
  };
  auto load_group = [&](int t) {   // t < ntiles
    if (!c.groups) return c.single;
    const uint4 *p = reinterpret_cast<const uint4 *>(c.groups + t / tpg);
    union { uint4 q[2]; TcGroup g; } u;
    u.q[0] = __ldg(p); u.q[1] = __ldg(p + 1);
    return u.g;
  };

  if (tid == 0) {
    mbar_init(&mma_bar[0], 1);
    mbar_init(&mma_bar[1], 1);
    mbar_init(&mma_bar[2], 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int n = 0; n < 2; ++n) {
      const int t = (int)blockIdx.x + n * stride;
      if (t < ntiles) ring[n] = make_tile(t, load_group(t));
    }
  }
  if (warp == 0) {  // tensor memory: three accumulator buffers of npad_max columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t a_addr = smem_addr(Abuf), b_addr = smem_addr(Bbuf);
  uint32_t phases = 0u;  // bit s: parity of the next completion of accumulator buffer s's barrier

  // thread 0 keeps the problem record of the tile after next in flight
  TcGroup pend = c.single;
  if (tid == 0 && (int)blockIdx.x + 2 * stride < ntiles) pend = load_group((int)blockIdx.x + 2 * stride);

  const bool sc_smem = (G & 1) == 0 && G <= 64;   // else the epilogue reads the scales from global memory
  const int f_pc = tid & (ppr - 1), f_r0 = tid >> lg_ppr, f_rstep = kTcThreads >> lg_ppr;  // this thread's piece and rows in a fetch
  // stage (n-th tile, quad q) into buffer `stage`; an empty commit when the block has no such tile
  auto fetch = [&](int n, int sb, int q, int stage) {   // sb: scale buffer of tile n
    if ((int)blockIdx.x + n * stride < ntiles) {
      const TcTile &ti = ring[n & 7];
      unsigned char *wd = Wst + stage * w_stage;
      const int rlast = c.N - 1 - ti.row0;   // rows past the end repeat the last row (never stored)
      const uint8_t *src0 = ti.P + (size_t)q * (gps * 64) + f_pc * 16;
#pragma unroll 4
      for (int rr = f_r0; rr < kTcRows; rr += f_rstep) {
        const int rs = rr < rlast ? rr : rlast;
        cp_async16(wd + rr * (gps * 64) + ((f_pc ^ (rr & (ppr - 1))) << 4), src0 + (size_t)rs * row_bytes);
      }
      if (q == 0) {   // the tile's activation scales [M][G] and the rows' weight scales [128][G]
        float *sd = sqs + sb * sq_stride;
        const float *ss = c.SQ + (size_t)ti.x_row0 * G;
        for (int i = tid; i < ti.M * G; i += kTcThreads) cp_async4(sd + i, ss + i);
        if (sc_smem) {
          // pairs of bf16 scales; a row's G scales are contiguous, and so are the tile's rows
          const int nrows = rlast + 1 < kTcRows ? rlast + 1 : kTcRows;
          const uint32_t *sw = reinterpret_cast<const uint32_t *>(ti.S + (size_t)ti.row0 * G);
          uint32_t *dw = reinterpret_cast<uint32_t *>(ssc + sb * sc_stride);
          for (int i = tid; i < nrows * G / 2; i += kTcThreads) cp_async4(dw + i, sw + i);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // activations of (n-th tile, group g) as 16-byte pieces [m][8]: a thread's first and second piece
  const int x_src0 = (tid >> 3) * K + (tid & 7) * 16, x_src1 = x_src0 + (kTcThreads >> 3) * K;   // batch entry tid / 8 (+ 32), piece tid % 8
  const int x_dst0 = (tid >> 6) * 128 + ((tid >> 3) & 7) * 16, x_dst1 = x_dst0 + (kTcThreads >> 6) * 128;
  auto load_x = [&](int n, int g, uint4 (&x)[2]) {
    if ((int)blockIdx.x + n * stride < ntiles) {
      const TcTile &ti = ring[n & 7];
      const int8_t *xb = c.XQ + (size_t)ti.x_row0 * K + g * 128;
      if (tid < ti.M * 8) x[0] = __ldg(reinterpret_cast<const uint4 *>(xb + x_src0));
      if (tid + kTcThreads < ti.M * 8) x[1] = __ldg(reinterpret_cast<const uint4 *>(xb + x_src1));
    }
  };
  float acc[kTcMaxBatch / 2];   // batch entry m = 8 * i + 4 * h + j lives in acc[4 * i + j]
#pragma unroll
  for (int m = 0; m < kTcMaxBatch / 2; ++m) acc[m] = 0.0f;
  uint4 xr[2], xn[2];
  xr[0] = xr[1] = xn[0] = xn[1] = make_uint4(0, 0, 0, 0);
  fetch(0, 0, 0, 0);
  load_x(0, 0, xr);

  int n = 0, q = 0, gl = 0, g = 0;   // tile of the block, stage of the tile, group of the stage / of the tile
  int stage = 0;                      // buffer of the stage being worked on
  int buf = 0;                        // accumulator / staging buffer of the step being staged
  bool live = (int)blockIdx.x < ntiles;
  // Steps whose products are in flight (at most two): a step is finished two steps after it was
  // staged, so that neither the issue of its products nor their latency is waited for.
  int pending = 0, p1_g = 0, p1_n = 0, p1_sb = 0, p2_g = 0, p2_n = 0, p2_sb = 0;   // p1: the last step, p2: the one before
  int tb = 0, eb = 0;                    // accumulator buffer of the step being staged / of the oldest pending step
  int sb_cur = 0, sb_next = 1;           // scale buffers of the current / next tile
#pragma unroll 1
  while (live || pending) {
    TC_STAMP(1);
    const bool do_epi = live ? pending == 2 : pending > 0;
    const int e_g = pending == 2 ? p2_g : p1_g, e_n = pending == 2 ? p2_n : p1_n, e_sb = pending == 2 ? p2_sb : p1_sb;
    if (do_epi) {
      // the oldest pending step's products are complete: its accumulators can be read, and the
      // staging buffer it read (the one this step writes) is free
      const uint32_t par = (phases >> eb) & 1u;
      bool ok = mbar_try(&mma_bar[eb], par);
      for (uint32_t it = 0; !ok && it < kTcSpin && !*reinterpret_cast<volatile uint32_t *>(&s_fail); ++it) ok = mbar_try(&mma_bar[eb], par);
      if (!ok) {
        s_fail = 1;
        if (g_stream_fault_word) *reinterpret_cast<volatile unsigned int *>(g_stream_fault_word) = 1;
      }
      phases ^= 1u << eb;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    if (live) {
      if (__builtin_expect(gl == 0, 0)) {
        // stage boundary: start the next stage (the next quad of this tile, or the first of the
        // block's next tile), then wait for this one
        const bool last_q = q + 1 == QT;
        fetch(last_q ? n + 1 : n, last_q ? sb_next : sb_cur, last_q ? 0 : q + 1, stage ^ 1);
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();  // every thread's copies of this stage have landed
        if (g == 0 && tid == 0) {
          // tile boundary: publish the record of the tile after next, fetch the one after that
          const int t2 = (int)blockIdx.x + (n + 2) * stride, t3 = t2 + stride;
          if (t2 < ntiles) ring[(n + 2) & 7] = make_tile(t2, pend);
          if (t3 < ntiles) pend = load_group(t3);
        }
      }
      TC_STAMP(2);
      const TcTile &ti = ring[n & 7];
      const int M = ti.M, npad = (int)tc_npad((uint32_t)M);
      const uint32_t b_chunk = (uint32_t)npad * 16u;
      // the next step's activations (same tile, or the first group of the block's next tile)
      if (g + 1 < G) load_x(n, g + 1, xn); else load_x(n + 1, 0, xn);
      // ---- stage this step: half of the row's 128 weights as INT8 (16 * v), and the batch's activations ----
      {
        const unsigned char *wrow = Wst + stage * w_stage + r * (gps * 64);
        unsigned char *ab = Abuf + buf * kTcABytes + (r >> 3) * 128 + (r & 7) * 16;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int jj = 2 * h + u;
          const uint4 cur = *reinterpret_cast<const uint4 *>(wrow + (((gl * 4 + jj) ^ (r & (ppr - 1))) << 4));
          // packed words (x, y) -> chunk 2jj, (z, w) -> chunk 2jj + 1: [low nibbles, high nibbles] per word
          const uint4 c0 = make_uint4((cur.x << 4) & 0xF0F0F0F0u, cur.x & 0xF0F0F0F0u, (cur.y << 4) & 0xF0F0F0F0u, cur.y & 0xF0F0F0F0u);
          const uint4 c1 = make_uint4((cur.z << 4) & 0xF0F0F0F0u, cur.z & 0xF0F0F0F0u, (cur.w << 4) & 0xF0F0F0F0u, cur.w & 0xF0F0F0F0u);
          *reinterpret_cast<uint4 *>(ab + (2 * jj) * 2048) = c0;
          *reinterpret_cast<uint4 *>(ab + (2 * jj + 1) * 2048) = c1;
        }
        unsigned char *bb = Bbuf + buf * b_bytes + (tid & 7) * b_chunk;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (tid + u * kTcThreads < M * 8) {
            const uint4 v = xr[u];
            const uint4 pp = make_uint4(__byte_perm(v.x, v.y, 0x6420), __byte_perm(v.x, v.y, 0x7531), __byte_perm(v.z, v.w, 0x6420),
                                        __byte_perm(v.z, v.w, 0x7531));
            *reinterpret_cast<uint4 *>(bb + (u ? x_dst1 : x_dst0)) = pp;
          }
        }
      }
    }
    TC_STAMP(3);
    // generic-proxy writes -> visible to the tensor core's reads, then everyone has written
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    TC_STAMP(4);
    if (live && tid == 0) {
      const int npad = (int)tc_npad((uint32_t)ring[n & 7].M);
      const uint32_t b_chunk = (uint32_t)npad * 16u;
      // instruction descriptor: D = S32, A = B = signed 8 bit, both K-major, N = npad, M = 128
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(npad >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
      const uint32_t d = tmem_base + (uint32_t)tb * (uint32_t)npad_max;
      // the four products differ only in the start addresses (low bits of the descriptors, in 16-byte units)
      const uint64_t da = umma_desc(a_addr + buf * kTcABytes, 2048u, 128u);
      const uint64_t db = umma_desc(b_addr + buf * b_bytes, b_chunk, 128u);
#pragma unroll
      for (int qq = 0; qq < 4; ++qq)
        umma_i8(d, da + (uint64_t)(qq * (4096 >> 4)), db + (uint64_t)(qq * ((2 * b_chunk) >> 4)), idesc, qq > 0 ? 1u : 0u);
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&mma_bar[tb]))
                   : "memory");
    }
    TC_STAMP(5);
    if (do_epi) {
      // ---- finish the oldest pending step (group e_g of tile e_n) ----
      // everything that does not depend on the products first: the row's weight scale of the
      // group and the first activation scales
      const TcTile &pt = ring[e_n & 7];
      const int pM = pt.M;
      float sc;
      if (sc_smem) {
        sc = bf16_to_f32(ssc[e_sb * sc_stride + r * G + e_g]);
      } else {
        const int prow = pt.row0 + r < c.N ? pt.row0 + r : c.N - 1;
        sc = bf16_to_f32(__ldg(pt.S + (size_t)prow * G + e_g));
      }
      const float *sqg = sqs + e_sb * sq_stride + (4 * h) * G + e_g;   // this half's first batch entry
      float sq0[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) sq0[jj] = 4 * h + jj < pM ? sqg[jj * G] : 0.0f;
      const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)eb * (uint32_t)npad_max + (uint32_t)(4 * h);
      if (4 * h < pM) {   // uniform across the warp
        int32_t v[4];
        TC_STAMP(8);
        tmem_ld4(taddr, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        TC_STAMP(9);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) acc[jj] = acc[jj] + ((float)(v[jj] >> 4) * sc) * sq0[jj];   // entries past M: never stored
      }
      if (8 + 4 * h < pM) {
#pragma unroll
        for (int i = 1; i < kTcMaxBatch / 8; ++i) {
          const int m0 = 8 * i + 4 * h;
          if (m0 < pM) {
            float sqv[4];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) sqv[jj] = m0 + jj < pM ? sqg[(8 * i + jj) * G] : 0.0f;
            int32_t v[4];
            tmem_ld4(taddr + (uint32_t)(8 * i), v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) acc[4 * i + jj] = acc[4 * i + jj] + ((float)(v[jj] >> 4) * sc) * sqv[jj];
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      TC_STAMP(7);
      if (__builtin_expect(e_g == G - 1, 0)) {
        // the row tile is complete: store it, start the next one from zero, and switch to the
        // next tile's scales (prefetched when this tile began)
        const bool in_range = pt.row0 + r < c.N;
        float *yb = c.Y + (size_t)pt.x_row0 * c.ldy + pt.y_col + pt.row0 + r;
#pragma unroll
        for (int i = 0; i < kTcMaxBatch / 8; ++i)
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int m = 8 * i + 4 * h + jj;
            if (m < pM && in_range) yb[(size_t)m * c.ldy] = acc[4 * i + jj];
            acc[4 * i + jj] = 0.0f;
          }
      }
    }
    if (do_epi) {
      --pending;
      eb = eb == 2 ? 0 : eb + 1;
    }
    if (live) {
      p2_g = p1_g; p2_n = p1_n; p2_sb = p1_sb;
      p1_g = g; p1_n = n; p1_sb = sb_cur;
      ++pending;
      tb = tb == 2 ? 0 : tb + 1;
      buf ^= 1;
      xr[0] = xn[0]; xr[1] = xn[1];
      ++g; ++gl;
      if (gl == gps) { gl = 0; ++q; stage ^= 1; }
      if (g == G) {
        g = 0; q = 0; ++n;
        sb_cur = sb_next;
        sb_next = sb_next + 1 == nsc ? 0 : sb_next + 1;
        live = (int)blockIdx.x + n * stride < ntiles;
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
}

__global__ void __launch_bounds__(kTcThreads, 2) Int4GemmA8Tc(const Int4GemmA8TcArgs a) {
  TcShape c;
  c.groups = nullptr;
  c.single.P = a.P; c.single.S = a.S; c.single.x_row0 = 0; c.single.M = a.M; c.single.y_col = 0; c.single.pad = 0;
  c.XQ = a.XQ; c.SQ = a.SQ; c.Y = a.Y;
  c.N = a.N; c.K = a.K; c.ldy = a.ldy; c.max_m = a.M;
  c.ntiles = (a.N + kTcRows - 1) / kTcRows;
  tc_body(c);
}

__global__ void __launch_bounds__(kTcThreads, 2) Int4GemmA8TcGrouped(const Int4GemmA8TcGroupedArgs a) {
  TcShape c;
  c.groups = a.Groups;
  c.single = TcGroup{nullptr, nullptr, 0, 0, 0, 0};
  c.XQ = a.XQ; c.SQ = a.SQ; c.Y = a.Y;
  c.N = a.N; c.K = a.K; c.ldy = a.ldy; c.max_m = a.max_m;
  c.ntiles = __ldg(a.NGroups) * ((a.N + kTcRows - 1) / kTcRows);
  tc_body(c);
}

static uint32_t tc_smem_fn(const void *args) {
  const Int4GemmA8TcArgs *a = (const Int4GemmA8TcArgs *)args;
  return tc_smem_bytes((uint32_t)a->K, (uint32_t)a->M);
}
static uint32_t tc_grouped_smem_fn(const void *args) {
  const Int4GemmA8TcGroupedArgs *a = (const Int4GemmA8TcGroupedArgs *)args;
  return tc_smem_bytes((uint32_t)a->K, (uint32_t)a->max_m);
}

#define F(f) AINFER_ARG(Int4GemmA8TcArgs, f)
AINFER_REGISTER(Int4GemmA8Tc, Int4GemmA8TcArgs, kTcThreads, 0, 0, tc_smem_fn, F(P), F(S), F(XQ), F(SQ), F(Y), F(N), F(K), F(M), F(ldy));
#undef F
#define F(f) AINFER_ARG(Int4GemmA8TcGroupedArgs, f)
AINFER_REGISTER(Int4GemmA8TcGrouped, Int4GemmA8TcGroupedArgs, kTcThreads, 0, 0, tc_grouped_smem_fn, F(Groups), F(NGroups), F(XQ), F(SQ),
                F(Y), F(N), F(K), F(max_m), F(ldy));
#undef F

}  // namespace ainfer
