// Int4GemvA8Multi: W4A8 group-128 GEMV for 1..8 activation rows with the weights streamed ONCE
// (batched form of the reference's Int4Gemv, tools/cmdlist/kernels.cpp:148-193; sweep protocol
// tools/gemv/gemv.cpp:503-601). Same arithmetic as the single-row kernel, per (batch entry, row):
// exact int32 group sums by dp4a on nibbles moved to the top of their bytes, then
// acc = acc + ((float)sum * weight_scale) * activation_scale[g] in ascending group order, so every
// batch entry is bit-identical to the one-row GEMV.
//
// A block owns a contiguous range of row tiles. A tile is 16 KB of packed rows (256 / G rows of K,
// G = K / 128) plus its 512 B of bf16 scales; a producer warp brings tiles into a ring of shared
// memory stages with bulk asynchronous copies (cp.async.bulk on an mbarrier; no cluster multicast).
// The 256 consumer lanes each own one (row, group) of a tile: 64 packed bytes. A lane takes TWO
// tiles' worth (two rows, the same group) into registers, widens the nibbles once, releases the
// stages, and then walks the batch: per entry it reads that group's 128 activations from shared
// memory (conflict-free, group-major layout) ONCE for both rows, 32 dp4a per row, and stores the
// scaled group term. Reading the activations once per two rows halves the shared-memory traffic,
// which together with the integer pipe bounds this kernel above four entries; up to four it runs
// at the speed of the weight stream. After a pair of tiles one thread per (entry, row) adds the
// row's G terms in ascending order.
// Every wait is bounded; a wait that runs out stores a code in the host-visible fault word.
#include "block_dot.cuh"

namespace ainfer {

struct Int4GemvA8MultiArgs {
  const uint8_t *P;    // packed nibbles [N][K/2]
  const uint16_t *S;   // bf16 scales [N][K/128]
  const int8_t *XQ;    // [M][K]
  const float *SQ;     // [M][K/128]
  float *Y;            // [M][ldy]
  int32_t N, K, M, ldy;
};

constexpr int kMvStages = 4;
constexpr int kMvCons = 256;                 // consumer lanes; one more warp produces
constexpr int kMvThreads = kMvCons + 32;
constexpr uint32_t kMvTile = 16384, kMvStride = kMvTile + 512;
constexpr uint32_t kMvSpin = 1u << 22;

extern __shared__ __align__(128) unsigned char mv_smem[];

__host__ __device__ inline uint32_t mv_round128(uint32_t v) { return (v + 127u) & ~127u; }
// staged activations | group terms [M][G][2 * RPI + 1] | ring
__host__ __device__ inline uint32_t mv_t_floats(int K, int M) { return (uint32_t)M * (uint32_t)(K / 128) * (2u * (256u / (uint32_t)(K / 128)) + 1u); }
__host__ __device__ inline uint32_t mv_smem_bytes(int K, int M) {
  return mv_round128(staged4_bytes(K, M)) + mv_round128(mv_t_floats(K, M) * 4u) + kMvStages * kMvStride;
}

__device__ __forceinline__ bool mv_wait(unsigned long long *bar, uint32_t parity, uint32_t *fail) {
  if (mbar_try(bar, parity)) return true;
  if (*reinterpret_cast<volatile uint32_t *>(fail)) return false;
#pragma unroll 1
  for (uint32_t i = 0; i < kMvSpin; ++i)
    if (mbar_try(bar, parity)) return true;
  *reinterpret_cast<volatile uint32_t *>(fail) = 1;
  if (g_stream_fault_word) *reinterpret_cast<volatile unsigned int *>(g_stream_fault_word) = 1;
  return false;
}
__device__ __forceinline__ void mv_cons_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__global__ void __launch_bounds__(kMvThreads, 2) Int4GemvA8Multi(const Int4GemvA8MultiArgs a) {
  __shared__ unsigned long long full[kMvStages], empty[kMvStages];
  __shared__ uint32_t s_fail;
  const int tid = threadIdx.x, K = a.K, G = K >> 7, RPI = 256 / G, M = a.M;
  unsigned char *ring = mv_smem + mv_round128(staged4_bytes(K, M)) + mv_round128(mv_t_floats(K, M) * 4u);
  float *T = reinterpret_cast<float *>(mv_smem + mv_round128(staged4_bytes(K, M)));
  if (tid == 0) {
    for (int s = 0; s < kMvStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 8); }
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // this block's tiles: a contiguous range of the ceil(N / RPI) row tiles
  const int ntiles = (a.N + RPI - 1) / RPI;
  const int t0 = (int)((long)ntiles * blockIdx.x / gridDim.x), t1 = (int)((long)ntiles * (blockIdx.x + 1) / gridDim.x);
  const bool bulk_scales = G >= 8;   // a tile's scale bytes are then a multiple of 16 wherever the matrix ends
  const size_t row_bytes = (size_t)(K >> 1);
  StagedAct4 act = stage4(mv_smem, a.XQ, a.SQ, K, M, K, G);   // every thread; ends with a block barrier (mbarriers visible)
  if (tid >= kMvCons) {
    // ---- producer warp: one lane keeps the ring full ----
    // a source that is not 16-byte aligned cannot be bulk-copied: report it and issue nothing
    // (the consumers' bounded waits then end the launch; no access is made)
    const bool aligned = (((uintptr_t)a.P | (bulk_scales ? (uintptr_t)a.S : 0)) & 15u) == 0 && 256 % G == 0;
    if (tid == kMvCons && !aligned) {
      s_fail = 1;
      if (g_stream_fault_word) *reinterpret_cast<volatile unsigned int *>(g_stream_fault_word) = 2;
    }
    if (tid == kMvCons && aligned) {
      uint32_t st = 0, ph = 0;
      for (int t = t0; t < t1; ++t) {
        if (t - t0 >= kMvStages && !mv_wait(&empty[st], ph ^ 1u, &s_fail)) break;
        const int rows = a.N - t * RPI < RPI ? a.N - t * RPI : RPI;
        const uint32_t wb = (uint32_t)(rows * row_bytes), sb = bulk_scales ? (uint32_t)(rows * G * 2) : 0u;
        unsigned char *dst = ring + st * kMvStride;
        mbar_arrive_expect(&full[st], wb + sb);
        bulk_g2s(dst, a.P + (size_t)t * RPI * row_bytes, wb, &full[st]);
        if (sb) bulk_g2s(dst + kMvTile, a.S + (size_t)t * RPI * G, sb, &full[st]);
        if (++st == kMvStages) { st = 0; ph ^= 1u; }
      }
    }
    return;
  }
  // ---- consumers ----
  const int g = tid % G, rt = tid / G, lane = tid & 31;
  const int rot = (tid >> 1) & 3;   // piece order of this lane: step s reads piece (s + rot) & 3 (bank-conflict free)
  const uint32_t ring_a = smem_addr(ring), lane_off = (uint32_t)tid * 64u;
  const int R = 2 * RPI, TS = R + 1;   // rows of a pair of tiles; row stride of the group-major term array
  const uint4 *xg = act.x + g;
  uint32_t st = 0, ph = 0;
#pragma unroll 1
  for (int t = t0; t < t1; t += 2) {
    uint32_t w[2][32];   // both rows' nibbles as signed bytes 16 * v: [piece][low x, high x, low y, high y, ...]
    float sc[2];
    bool live[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int tt = t + u;
      live[u] = tt < t1 && tt * RPI + rt < a.N;
      sc[u] = 0.0f;
      if (tt < t1) {
        const bool ok = mv_wait(&full[st], ph, &s_fail);
        const uint32_t base = ring_a + st * kMvStride;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          uint4 p = make_uint4(0, 0, 0, 0);
          if (ok) p = lds128(base + lane_off + (uint32_t)(((s + rot) & 3) << 4));
          w[u][8 * s + 0] = (p.x * 16u) & 0xF0F0F0F0u; w[u][8 * s + 1] = p.x & 0xF0F0F0F0u;
          w[u][8 * s + 2] = (p.y * 16u) & 0xF0F0F0F0u; w[u][8 * s + 3] = p.y & 0xF0F0F0F0u;
          w[u][8 * s + 4] = (p.z * 16u) & 0xF0F0F0F0u; w[u][8 * s + 5] = p.z & 0xF0F0F0F0u;
          w[u][8 * s + 6] = (p.w * 16u) & 0xF0F0F0F0u; w[u][8 * s + 7] = p.w & 0xF0F0F0F0u;
        }
        if (live[u]) {
          const uint32_t raw = bulk_scales && ok ? lds_u16(base + kMvTile + tid * 2)
                                                 : (uint32_t)__ldg(a.S + (size_t)(tt * RPI + rt) * G + g);
          sc[u] = __uint_as_float(raw << 16);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
        if (++st == kMvStages) { st = 0; ph ^= 1u; }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) w[u][i] = 0u;
      }
    }
    // ---- the batch: activations of this lane's group once per entry, both rows ----
#pragma unroll 1
    for (int m = 0; m < M; ++m) {
      const uint4 *xv = xg + (size_t)m * 8 * G;
      const float sqg = act.sq[m * G + g];
      int d0 = 0, d1 = 0;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const int j = (s + rot) & 3;
        const uint4 xa = xv[(2 * j) * G], xb = xv[(2 * j + 1) * G];
        d0 = __dp4a((int)w[0][8 * s + 0], (int)xa.x, d0); d0 = __dp4a((int)w[0][8 * s + 1], (int)xa.y, d0);
        d0 = __dp4a((int)w[0][8 * s + 2], (int)xa.z, d0); d0 = __dp4a((int)w[0][8 * s + 3], (int)xa.w, d0);
        d0 = __dp4a((int)w[0][8 * s + 4], (int)xb.x, d0); d0 = __dp4a((int)w[0][8 * s + 5], (int)xb.y, d0);
        d0 = __dp4a((int)w[0][8 * s + 6], (int)xb.z, d0); d0 = __dp4a((int)w[0][8 * s + 7], (int)xb.w, d0);
        d1 = __dp4a((int)w[1][8 * s + 0], (int)xa.x, d1); d1 = __dp4a((int)w[1][8 * s + 1], (int)xa.y, d1);
        d1 = __dp4a((int)w[1][8 * s + 2], (int)xa.z, d1); d1 = __dp4a((int)w[1][8 * s + 3], (int)xa.w, d1);
        d1 = __dp4a((int)w[1][8 * s + 4], (int)xb.x, d1); d1 = __dp4a((int)w[1][8 * s + 5], (int)xb.y, d1);
        d1 = __dp4a((int)w[1][8 * s + 6], (int)xb.z, d1); d1 = __dp4a((int)w[1][8 * s + 7], (int)xb.w, d1);
      }
      float *tm = T + ((size_t)m * G + g) * TS;
      tm[rt] = ((float)(d0 >> 4) * sc[0]) * sqg;
      tm[RPI + rt] = ((float)(d1 >> 4) * sc[1]) * sqg;
    }
    mv_cons_sync();
    // ---- one thread per (entry, row of the pair): the row's terms in ascending group order ----
    for (int i = tid; i < M * R; i += kMvCons) {
      const int m = i / R, r = i % R;
      const int row = t * RPI + r;
      if (r < RPI ? (row < a.N) : (t + 1 < t1 && row < a.N)) {
        const float *tr = T + (size_t)m * G * TS + r;
        float acc = 0.0f;
        for (int gg = 0; gg < G; ++gg) acc = acc + tr[gg * TS];
        a.Y[(size_t)m * a.ldy + row] = acc;
      }
    }
    mv_cons_sync();   // the terms are rewritten by the next pair
  }
}

// ---- grouped form: a list of problems of one shape, each with at most 8 activation rows ----
// Problem i has its own weights and its own range of activation / output rows (an expert and the
// tokens routed to it); list and length live in device memory. Tiles of all problems form one
// sequence (problem-major) that is dealt to the blocks in contiguous ranges; a block restages the
// activations when its range enters another problem. Problems with more than 8 rows are not for
// this kernel (the caller gives them to the tensor-core form): they are skipped.
struct MvGroup {           // = the tensor-core form's problem record
  const uint8_t *P;
  const uint16_t *S;
  int32_t x_row0, M, y_col, pad;
};
static_assert(sizeof(MvGroup) == 32, "problem record");
struct Int4GemvA8MultiGroupedArgs {
  const MvGroup *Groups;
  const int32_t *NGroups;
  const int8_t *XQ;
  const float *SQ;
  float *Y;
  int32_t N, K, ldy;
};

__global__ void __launch_bounds__(kMvThreads, 2) Int4GemvA8MultiGrouped(const Int4GemvA8MultiGroupedArgs a) {
  __shared__ unsigned long long full[kMvStages], empty[kMvStages];
  __shared__ uint32_t s_fail;
  constexpr int MB = 8;
  const int tid = threadIdx.x, K = a.K, G = K >> 7, RPI = 256 / G;
  unsigned char *ring = mv_smem + mv_round128(staged4_bytes(K, MB)) + mv_round128(mv_t_floats(K, MB) * 4u);
  float *T = reinterpret_cast<float *>(mv_smem + mv_round128(staged4_bytes(K, MB)));
  if (tid == 0) {
    for (int s = 0; s < kMvStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 8); }
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int tpg = (a.N + RPI - 1) / RPI;               // tiles per problem
  const int ntiles = __ldg(a.NGroups) * tpg;
  const int t0 = (int)((long)ntiles * blockIdx.x / gridDim.x), t1 = (int)((long)ntiles * (blockIdx.x + 1) / gridDim.x);
  const bool bulk_scales = G >= 8;
  const size_t row_bytes = (size_t)(K >> 1);
  auto load_group = [&](int gi) {
    union { uint4 q[2]; MvGroup g; } u;
    const uint4 *p = reinterpret_cast<const uint4 *>(a.Groups + gi);
    u.q[0] = __ldg(p); u.q[1] = __ldg(p + 1);
    return u.g;
  };
  if (tid >= kMvCons) {
    if (tid == kMvCons) {
      uint32_t st = 0, ph = 0, issued = 0;
      int cur = -1;
      MvGroup gr{};
      bool ok = 256 % G == 0;
      for (int t = t0; t < t1 && ok; ++t) {
        const int gi = t / tpg, tg = t - gi * tpg;
        if (gi != cur) {
          gr = load_group(gi);
          cur = gi;
          if ((((uintptr_t)gr.P | (bulk_scales ? (uintptr_t)gr.S : 0)) & 15u) != 0) { ok = false; break; }
        }
        if (gr.M > MB) continue;   // not this kernel's problem: no tile is produced, the consumers skip it too
        if (issued >= (uint32_t)kMvStages && !mv_wait(&empty[st], ph ^ 1u, &s_fail)) break;
        const int rows = a.N - tg * RPI < RPI ? a.N - tg * RPI : RPI;
        const uint32_t wb = (uint32_t)(rows * row_bytes), sb = bulk_scales ? (uint32_t)(rows * G * 2) : 0u;
        unsigned char *dst = ring + st * kMvStride;
        mbar_arrive_expect(&full[st], wb + sb);
        bulk_g2s(dst, gr.P + (size_t)tg * RPI * row_bytes, wb, &full[st]);
        if (sb) bulk_g2s(dst + kMvTile, gr.S + (size_t)tg * RPI * G, sb, &full[st]);
        ++issued;
        if (++st == kMvStages) { st = 0; ph ^= 1u; }
      }
      if (!ok) {
        s_fail = 1;
        if (g_stream_fault_word) *reinterpret_cast<volatile unsigned int *>(g_stream_fault_word) = 2;
      }
    }
    return;
  }
  const int g = tid % G, rt = tid / G, lane = tid & 31;
  const int rot = (tid >> 1) & 3;
  const uint32_t ring_a = smem_addr(ring), lane_off = (uint32_t)tid * 64u;
  const int R = 2 * RPI, TS = R + 1;
  uint32_t *xw = reinterpret_cast<uint32_t *>(mv_smem);
  uint32_t st = 0, ph = 0;
  int cur = -1;
  MvGroup gr{};
  int M = 0;
  float *sqs = reinterpret_cast<float *>(mv_smem);
#pragma unroll 1
  for (int t = t0; t < t1;) {
    const int gi = t / tpg, tg = t - gi * tpg;
    if (gi != cur) {
      gr = load_group(gi);
      cur = gi;
      M = gr.M;
      if (M <= MB) {
        // restage this problem's activations (no consumer still reads the previous problem's: the
        // barrier that ended the previous pair is behind every lane)
        sqs = reinterpret_cast<float *>(mv_smem + (size_t)M * K);
        const int8_t *xq = a.XQ + (size_t)gr.x_row0 * K;
        for (int i = tid; i < M * (K / 8); i += kMvCons) {
          const int m = i / (K / 8), pc = i % (K / 8);
          const uint2 v = __ldcg(reinterpret_cast<const uint2 *>(xq + (size_t)m * K + (size_t)pc * 8));
          xw[staged4_word(K, m, pc, 0)] = __byte_perm(v.x, v.y, 0x6420);
          xw[staged4_word(K, m, pc, 1)] = __byte_perm(v.x, v.y, 0x7531);
        }
        for (int i = tid; i < M * G; i += kMvCons) sqs[i] = __ldcg(a.SQ + (size_t)gr.x_row0 * G + i);
        mv_cons_sync();
      }
    }
    if (M > MB) { t = (gi + 1) * tpg; continue; }   // skip the whole problem
    const bool second = tg + 1 < tpg && t + 1 < t1;  // the pair's second tile: same problem, inside this block's range
    uint32_t w[2][32];
    float sc[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      sc[u] = 0.0f;
      if (u == 0 || second) {
        const bool ok = mv_wait(&full[st], ph, &s_fail);
        const uint32_t base = ring_a + st * kMvStride;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          uint4 p = make_uint4(0, 0, 0, 0);
          if (ok) p = lds128(base + lane_off + (uint32_t)(((s + rot) & 3) << 4));
          w[u][8 * s + 0] = (p.x * 16u) & 0xF0F0F0F0u; w[u][8 * s + 1] = p.x & 0xF0F0F0F0u;
          w[u][8 * s + 2] = (p.y * 16u) & 0xF0F0F0F0u; w[u][8 * s + 3] = p.y & 0xF0F0F0F0u;
          w[u][8 * s + 4] = (p.z * 16u) & 0xF0F0F0F0u; w[u][8 * s + 5] = p.z & 0xF0F0F0F0u;
          w[u][8 * s + 6] = (p.w * 16u) & 0xF0F0F0F0u; w[u][8 * s + 7] = p.w & 0xF0F0F0F0u;
        }
        const int row = (tg + u) * RPI + rt;
        if (row < a.N) {
          const uint32_t raw = bulk_scales && ok ? lds_u16(base + kMvTile + tid * 2) : (uint32_t)__ldg(gr.S + (size_t)row * G + g);
          sc[u] = __uint_as_float(raw << 16);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
        if (++st == kMvStages) { st = 0; ph ^= 1u; }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) w[u][i] = 0u;
      }
    }
    const uint4 *xg = reinterpret_cast<const uint4 *>(mv_smem) + g;
#pragma unroll 1
    for (int m = 0; m < M; ++m) {
      const uint4 *xv = xg + (size_t)m * 8 * G;
      const float sqg = sqs[m * G + g];
      int d0 = 0, d1 = 0;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const int j = (s + rot) & 3;
        const uint4 xa = xv[(2 * j) * G], xb = xv[(2 * j + 1) * G];
        d0 = __dp4a((int)w[0][8 * s + 0], (int)xa.x, d0); d0 = __dp4a((int)w[0][8 * s + 1], (int)xa.y, d0);
        d0 = __dp4a((int)w[0][8 * s + 2], (int)xa.z, d0); d0 = __dp4a((int)w[0][8 * s + 3], (int)xa.w, d0);
        d0 = __dp4a((int)w[0][8 * s + 4], (int)xb.x, d0); d0 = __dp4a((int)w[0][8 * s + 5], (int)xb.y, d0);
        d0 = __dp4a((int)w[0][8 * s + 6], (int)xb.z, d0); d0 = __dp4a((int)w[0][8 * s + 7], (int)xb.w, d0);
        d1 = __dp4a((int)w[1][8 * s + 0], (int)xa.x, d1); d1 = __dp4a((int)w[1][8 * s + 1], (int)xa.y, d1);
        d1 = __dp4a((int)w[1][8 * s + 2], (int)xa.z, d1); d1 = __dp4a((int)w[1][8 * s + 3], (int)xa.w, d1);
        d1 = __dp4a((int)w[1][8 * s + 4], (int)xb.x, d1); d1 = __dp4a((int)w[1][8 * s + 5], (int)xb.y, d1);
        d1 = __dp4a((int)w[1][8 * s + 6], (int)xb.z, d1); d1 = __dp4a((int)w[1][8 * s + 7], (int)xb.w, d1);
      }
      float *tm = T + ((size_t)m * G + g) * TS;
      tm[rt] = ((float)(d0 >> 4) * sc[0]) * sqg;
      tm[RPI + rt] = ((float)(d1 >> 4) * sc[1]) * sqg;
    }
    mv_cons_sync();
    for (int i = tid; i < M * R; i += kMvCons) {
      const int m = i / R, r = i % R;
      const int row = tg * RPI + r;
      if ((r < RPI || second) && row < a.N) {
        const float *tr = T + (size_t)m * G * TS + r;
        float acc = 0.0f;
        for (int gg = 0; gg < G; ++gg) acc = acc + tr[gg * TS];
        a.Y[(size_t)(gr.x_row0 + m) * a.ldy + gr.y_col + row] = acc;
      }
    }
    mv_cons_sync();
    t += second ? 2 : 1;
  }
}

static uint32_t mv_grouped_smem_fn(const void *args) {
  return mv_smem_bytes(((const Int4GemvA8MultiGroupedArgs *)args)->K, 8);
}

static uint32_t mv_smem_fn(const void *args) {
  const Int4GemvA8MultiArgs *a = (const Int4GemvA8MultiArgs *)args;
  return mv_smem_bytes(a->K, a->M);
}
#define F(f) AINFER_ARG(Int4GemvA8MultiArgs, f)
AINFER_REGISTER(Int4GemvA8Multi, Int4GemvA8MultiArgs, kMvThreads, 0, 0, mv_smem_fn, F(P), F(S), F(XQ), F(SQ), F(Y), F(N), F(K), F(M), F(ldy));
#undef F
#define F(f) AINFER_ARG(Int4GemvA8MultiGroupedArgs, f)
AINFER_REGISTER(Int4GemvA8MultiGrouped, Int4GemvA8MultiGroupedArgs, kMvThreads, 0, 0, mv_grouped_smem_fn, F(Groups), F(NGroups), F(XQ), F(SQ), F(Y),
                F(N), F(K), F(ldy));
#undef F

}  // namespace ainfer
