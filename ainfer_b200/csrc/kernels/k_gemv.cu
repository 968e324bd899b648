// Kernel entries of the INT4 x INT8 GEMV (weight ring + block_dot, block_stages.cuh).
#include "block_stages.cuh"

namespace ainfer {

extern __shared__ __align__(128) unsigned char gemv_smem[];

// One body for every batch width: activation row m = 0..M-1 is one pass of the M = 1 pipeline
// over the block's rows (the weights are streamed once per activation row: exact W4A8 batches
// are a parity surface for the operator sweep, the batched operator is Int4GemmA16).
constexpr int kGemvStages = 5;
__host__ __device__ inline uint32_t round128(uint32_t v) { return (v + 127u) & ~127u; }

// One activation row through the single-row pipeline, out of line: the batched kernels call it
// M times and it keeps the register allocation of the single-row kernel.
static __device__ __noinline__ void gemv_pass(const int8_t *xq, const float *sq, int K, const GemvMat *smats, int nmats,
                                              int total_rows, Ring *ring, SegList *lists, float *T, int m) {
  BlockScratch bs{ring, lists, T, nullptr, 0, false};
  StagedAct4 act = stage4(gemv_smem, xq, sq, K, 1, K, K / 128);
  gemv_block_dispatch(K, smats, nmats, total_rows, act, bs, blockIdx.x, gridDim.x, m);
}

template <bool kBatched>
__device__ __forceinline__ void gemv_a8_body(const Int4GemvA8Args &a) {
  __shared__ GemvMat smats[8];
  __shared__ SegList lists[2];
  __shared__ float T[kTFloats];
  __shared__ Ring ring;
  pdl_launch_dependents();
  // the matrix table and the weights are constants of the model: fetched before the wait
  if (threadIdx.x < a.nmats) smats[threadIdx.x] = a.mats[threadIdx.x];
  ring_init(&ring, gemv_smem + round128(staged4_bytes(a.K, 1)), kGemvStages);  // syncs: smats visible
  BlockScratch bs{&ring, lists, T, nullptr, 0, false};
  // start the weight stream before the activations are staged
  if (threadIdx.x == 0) gemv_first_list(&lists[0], smats, a.nmats, a.K, a.total_rows, blockIdx.x, gridDim.x);
  __syncthreads();
  ring_prefetch_all(&ring, &lists[0]);  // the warp leaders issue the first tiles in parallel
  bs.primed = true;
  pdl_wait();  // the activations come from the previous kernel
  if (!kBatched) {  // the decode kernel: no loop, so that its code is exactly the single-row pipeline
    StagedAct4 act = stage4(gemv_smem, a.XQ, a.SQ, a.K, 1, a.K, a.K / 128);
    gemv_block_dispatch(a.K, smats, a.nmats, a.total_rows, act, bs, blockIdx.x, gridDim.x, 0);
  } else {
    // (the prefetch above is consumed by the first pass: the ring remembers what is in flight)
#pragma unroll 1
    for (int m = 0; m < a.M; ++m) {
      if (m > 0) __syncthreads();  // the staged vector and t[][] of the previous pass are no longer read
      gemv_pass(a.XQ + (size_t)m * a.K, a.SQ + (size_t)m * (a.K / 128), a.K, smats, a.nmats, a.total_rows, &ring,
                lists, T, m);
    }
  }
  if (threadIdx.x == 0) ring_drain_after_fault(&ring);
}

__global__ void __launch_bounds__(256, 2) Int4GemvA8(const Int4GemvA8Args a) { gemv_a8_body<false>(a); }
__global__ void __launch_bounds__(256, 2) Int4GemvA8M2(const Int4GemvA8Args a) { gemv_a8_body<true>(a); }
__global__ void __launch_bounds__(256, 2) Int4GemvA8M4(const Int4GemvA8Args a) { gemv_a8_body<true>(a); }
__global__ void __launch_bounds__(256, 2) Int4GemvA8M8(const Int4GemvA8Args a) { gemv_a8_body<true>(a); }

// BoundedWaitProbe: one warp waits, with the ring's own bounded wait, for a shared-memory
// barrier phase that nothing completes (no copy is issued). The wait runs out after
// kRingSpinLimit polls (milliseconds), stores code 1 in the host-visible fault word and returns
// false; the kernel then ends normally. It exists so that the error path every weight-streaming
// kernel relies on (the wait gives up, control flow stays uniform, the next sync reports it) can
// be exercised without any faulting access. Out[0] = 1 if the wait succeeded, 2 if it gave up.
struct BoundedWaitProbeArgs {
  int32_t *Out;
};
__global__ void __launch_bounds__(32) BoundedWaitProbe(const BoundedWaitProbeArgs a) {
  __shared__ Ring ring;
  __shared__ __align__(128) unsigned char dummy[128];
  ring_init(&ring, dummy, 1);
  const bool ok = mbar_wait(&ring, &ring.full[0], 0u);
  __syncwarp();
  if (threadIdx.x == 0) a.Out[0] = ok ? 1 : 2;
}
#define F(f) AINFER_ARG(BoundedWaitProbeArgs, f)
AINFER_REGISTER(BoundedWaitProbe, BoundedWaitProbeArgs, 32, 0, 0, nullptr, F(Out));
#undef F

static uint32_t gemv1_smem_fn(const void *args) {
  const Int4GemvA8Args *a = (const Int4GemvA8Args *)args;
  return round128(staged4_bytes(a->K, 1)) + kGemvStages * kStageStride;
}

#define F(f) AINFER_ARG(Int4GemvA8Args, f)
#define GEMV_FIELDS F(mats), F(nmats), F(total_rows), F(XQ), F(SQ), F(K), F(M)
AINFER_REGISTER(Int4GemvA8, Int4GemvA8Args, 256, 0, 0, gemv1_smem_fn, GEMV_FIELDS);
AINFER_REGISTER(Int4GemvA8M2, Int4GemvA8Args, 256, 0, 0, gemv1_smem_fn, GEMV_FIELDS);
AINFER_REGISTER(Int4GemvA8M4, Int4GemvA8Args, 256, 0, 0, gemv1_smem_fn, GEMV_FIELDS);
AINFER_REGISTER(Int4GemvA8M8, Int4GemvA8Args, 256, 0, 0, gemv1_smem_fn, GEMV_FIELDS);
#undef F

AINFER_EARLY_LAUNCH(Int4GemvA8);
AINFER_EARLY_LAUNCH(Int4GemvA8M2);
AINFER_EARLY_LAUNCH(Int4GemvA8M4);
AINFER_EARLY_LAUNCH(Int4GemvA8M8);

}  // namespace ainfer
