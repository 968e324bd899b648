// Kernel entries of the INT4 x INT8 GEMV; row code in gemv_stage.cuh (shared
// with the persistent decode kernel).
#include "block_stages.cuh"

namespace ainfer {

extern __shared__ __align__(128) unsigned char gemv_smem[];

template <int M>
__device__ __forceinline__ void gemv_kernel(const Int4GemvA8Args &a) {
  __shared__ GemvMat smats[8];
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x < a.nmats) smats[threadIdx.x] = a.mats[threadIdx.x];  // synced by stage_act
  StagedAct act = stage_act(gemv_smem, a.XQ, a.SQ, a.K, M, a.K, a.K / 128);
  gemv_dispatch_k<M>(a, act, smats, blockIdx.x, gridDim.x);
}

// One entry point per batch width so that register allocation follows M.
// M = 1: the block-flattened form (block_dot.cuh); wider batches keep the warp-pass form.
constexpr int kGemvStages = 5;
__host__ __device__ inline uint32_t round128(uint32_t v) { return (v + 127u) & ~127u; }

__global__ void __launch_bounds__(256, 2) Int4GemvA8(const Int4GemvA8Args a) {
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
  if (threadIdx.x == 0) {
    gemv_first_list(&lists[0], smats, a.nmats, a.K, a.total_rows, blockIdx.x, gridDim.x);
    ring_prefetch(&ring, &lists[0]);
  }
  bs.primed = true;
  pdl_wait();  // the activations come from the previous kernel
  StagedAct4 act = stage4(gemv_smem, a.XQ, a.SQ, a.K, 1, a.K, a.K / 128);
  gemv_block_dispatch(a.K, smats, a.nmats, a.total_rows, act, bs, blockIdx.x, gridDim.x);
  if (threadIdx.x == 0) ring_drain_after_fault(&ring);
}
__global__ void __launch_bounds__(256, 3) Int4GemvA8M2(const Int4GemvA8Args a) { gemv_kernel<2>(a); }
__global__ void __launch_bounds__(256) Int4GemvA8M4(const Int4GemvA8Args a) { gemv_kernel<4>(a); }
__global__ void __launch_bounds__(256) Int4GemvA8M8(const Int4GemvA8Args a) { gemv_kernel<8>(a); }

static uint32_t gemv1_smem_fn(const void *args) {
  const Int4GemvA8Args *a = (const Int4GemvA8Args *)args;
  return round128(staged4_bytes(a->K, 1)) + kGemvStages * kStageStride;
}
static uint32_t gemv_smem_fn(const void *args) {
  const Int4GemvA8Args *a = (const Int4GemvA8Args *)args;
  return staged_act_bytes(a->K, a->M);
}

#define F(f) AINFER_ARG(Int4GemvA8Args, f)
#define GEMV_FIELDS F(mats), F(nmats), F(total_rows), F(XQ), F(SQ), F(K), F(M)
AINFER_REGISTER(Int4GemvA8, Int4GemvA8Args, 256, 0, 0, gemv1_smem_fn, GEMV_FIELDS);
AINFER_REGISTER(Int4GemvA8M2, Int4GemvA8Args, 256, 0, 0, gemv_smem_fn, GEMV_FIELDS);
AINFER_REGISTER(Int4GemvA8M4, Int4GemvA8Args, 256, 0, 0, gemv_smem_fn, GEMV_FIELDS);
AINFER_REGISTER(Int4GemvA8M8, Int4GemvA8Args, 256, 0, 0, gemv_smem_fn, GEMV_FIELDS);
#undef F

AINFER_EARLY_LAUNCH(Int4GemvA8);
AINFER_EARLY_LAUNCH(Int4GemvA8M2);
AINFER_EARLY_LAUNCH(Int4GemvA8M4);
AINFER_EARLY_LAUNCH(Int4GemvA8M8);

}  // namespace ainfer
