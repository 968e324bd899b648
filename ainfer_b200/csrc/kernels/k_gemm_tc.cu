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
//   * one thread issues four tcgen05.mma (M = 128 rows, N = padded batch, K = 32 each) into one
//     of two accumulator buffers in tensor memory and commits them to an mbarrier;
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

extern __shared__ __align__(1024) unsigned char tc_smem[];

__global__ void __launch_bounds__(128) Int4GemmA8Tc(const Int4GemmA8TcArgs a) {
  __shared__ unsigned long long mma_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t s_fail;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int K = a.K, G = K >> 7, M = a.M;
  const int Npad = M <= 8 ? 8 : ((M + 15) & ~15);      // batch padded to a legal MMA N
  unsigned char *Abuf = tc_smem;                        // [2][8 chunks][16 row blocks][8 rows][16 B]
  unsigned char *Bbuf = tc_smem + 2 * kTcABytes;        // [2][8 chunks][Npad / 8 blocks][8 rows][16 B]
  const uint32_t b_chunk = (uint32_t)Npad * 16u, b_bytes = 8u * b_chunk;
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
  if (warp == 0) {  // tensor memory: two accumulator buffers of Npad columns (128 columns cover both)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(128u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t a_addr = smem_addr(Abuf), b_addr = smem_addr(Bbuf);
  uint32_t uses[2] = {0u, 0u};  // completed uses of each accumulator buffer / barrier (for the parity)

  const int ntiles = (a.N + kTcRows - 1) / kTcRows;
#pragma unroll 1
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int n0 = t * kTcRows;
    const int row = n0 + tid < a.N ? n0 + tid : a.N - 1;   // rows past the end repeat the last row (not stored)
    const uint8_t *prow = a.P + (size_t)row * (K >> 1);
    const uint16_t *srow = a.S + (size_t)row * G;
    float acc[kTcMaxBatch];
#pragma unroll
    for (int m = 0; m < kTcMaxBatch; ++m) acc[m] = 0.0f;
    uint4 w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = __ldg(reinterpret_cast<const uint4 *>(prow) + j);
#pragma unroll 1
    for (int g = 0; g <= G; ++g) {
      const int buf = g & 1;
      if (g < G) {
        // ---- stage group g: this row's 128 weights as INT8 (16 * v), and the batch's activations ----
        uint4 cur[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) cur[j] = w[j];
        if (g + 1 < G) {
#pragma unroll
          for (int j = 0; j < 4; ++j) w[j] = __ldg(reinterpret_cast<const uint4 *>(prow + (size_t)(g + 1) * 64) + j);
        }
        unsigned char *ab = Abuf + buf * kTcABytes + (tid >> 3) * 128 + (tid & 7) * 16;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // packed words (x, y) -> chunk 2j, (z, w) -> chunk 2j + 1: [low nibbles, high nibbles] per word
          const uint4 c0 = make_uint4((cur[j].x << 4) & 0xF0F0F0F0u, cur[j].x & 0xF0F0F0F0u, (cur[j].y << 4) & 0xF0F0F0F0u,
                                      cur[j].y & 0xF0F0F0F0u);
          const uint4 c1 = make_uint4((cur[j].z << 4) & 0xF0F0F0F0u, cur[j].z & 0xF0F0F0F0u, (cur[j].w << 4) & 0xF0F0F0F0u,
                                      cur[j].w & 0xF0F0F0F0u);
          *reinterpret_cast<uint4 *>(ab + (2 * j) * 2048) = c0;
          *reinterpret_cast<uint4 *>(ab + (2 * j + 1) * 2048) = c1;
        }
        for (int i = tid; i < M * 8; i += 128) {
          const int m = i >> 3, c = i & 7;
          const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(a.XQ + (size_t)m * K + (size_t)g * 128) + c);
          const uint4 p = make_uint4(__byte_perm(v.x, v.y, 0x6420), __byte_perm(v.x, v.y, 0x7531), __byte_perm(v.z, v.w, 0x6420),
                                     __byte_perm(v.z, v.w, 0x7531));
          *reinterpret_cast<uint4 *>(Bbuf + buf * b_bytes + c * b_chunk + (m >> 3) * 128 + (m & 7) * 16) = p;
        }
        // generic-proxy writes -> visible to the tensor core's reads, then everyone has written
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (tid == 0) {
          const uint32_t d = tmem_base + (uint32_t)buf * (uint32_t)Npad;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint64_t da = umma_desc(a_addr + buf * kTcABytes + q * 2 * 2048, 2048u, 128u);
            const uint64_t db = umma_desc(b_addr + buf * b_bytes + q * 2 * b_chunk, b_chunk, 128u);
            umma_i8(d, da, db, idesc, q > 0 ? 1u : 0u);
          }
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&mma_bar[buf]))
                       : "memory");
        }
      }
      if (g > 0) {
        // ---- finish group g - 1 ----
        const int pb = (g - 1) & 1;
        bool ok = mbar_try(&mma_bar[pb], uses[pb] & 1u);
        for (uint32_t i = 0; !ok && i < kTcSpin && !*reinterpret_cast<volatile uint32_t *>(&s_fail); ++i)
          ok = mbar_try(&mma_bar[pb], uses[pb] & 1u);
        if (!ok) {
          s_fail = 1;
          if (g_stream_fault_word) *reinterpret_cast<volatile unsigned int *>(g_stream_fault_word) = 1;
        }
        uses[pb] += 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float sc = bf16_to_f32(__ldg(srow + (g - 1)));
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)pb * (uint32_t)Npad;
#pragma unroll
        for (int m0 = 0; m0 < kTcMaxBatch; m0 += 8) {
          if (m0 < M) {  // uniform across the block
            int32_t v[8];
            tmem_ld8(taddr + (uint32_t)m0, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (m0 + j < M) acc[m0 + j] = acc[m0 + j] + ((float)(v[j] >> 4) * sc) * __ldg(a.SQ + (size_t)(m0 + j) * G + (g - 1));
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      }
    }
    if (n0 + tid < a.N) {
#pragma unroll
      for (int m = 0; m < kTcMaxBatch; ++m)
        if (m < M) a.Y[(size_t)m * a.ldy + n0 + tid] = acc[m];
    }
    __syncthreads();  // the staging buffers are rewritten by the next tile
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
}

static uint32_t tc_smem_fn(const void *args) {
  const int M = ((const Int4GemmA8TcArgs *)args)->M;
  const int Npad = M <= 8 ? 8 : ((M + 15) & ~15);
  return (uint32_t)(2 * kTcABytes + 2 * 8 * Npad * 16);
}

#define F(f) AINFER_ARG(Int4GemmA8TcArgs, f)
AINFER_REGISTER(Int4GemmA8Tc, Int4GemmA8TcArgs, 128, 0, 0, tc_smem_fn, F(P), F(S), F(XQ), F(SQ), F(Y), F(N), F(K), F(M), F(ldy));
#undef F

}  // namespace ainfer
