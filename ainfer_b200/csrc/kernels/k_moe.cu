// Kernel entries of the mixture-of-experts block; bodies in moe_core.cuh
// (shared with the persistent decode kernel).
#define AINFER_BLOCK_DOT_INLINE 1
#include "block_stages.cuh"

namespace ainfer {

extern __shared__ __align__(128) unsigned char moe_smem[];

__global__ void __launch_bounds__(256) RouterTopK(const RouterTopKArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ bool is_last;
  __shared__ float sp[1024 + 1];
  router_logits_rows(a, blockIdx.x, gridDim.x);
  // last block to arrive does the selection
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned prev = atomicAdd(a.Counter, 1u);
    is_last = prev == gridDim.x - 1;
    if (is_last) *a.Counter = 0u;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  router_select(a.Logits, a.E, a.k, a.Wsg != nullptr, sp, a.SelIdx, a.SelW, a.NearGap);
}

constexpr int kMoeStages = 4;
__host__ __device__ inline uint32_t moe_round128(uint32_t v) { return (v + 127u) & ~127u; }

__global__ void __launch_bounds__(256, 2) ExpertGateUp(const ExpertGateUpArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ SegList lists[2];
  __shared__ float T[kTFloats];
  __shared__ Ring ring;
  __shared__ ExpertW sew[kMaxSegs];
  fetch_expert_rows(sew, a.Experts, a.SelIdx + a.slot_begin, a.slots);
  ring_init(&ring, moe_smem + moe_round128(staged4_bytes(a.H, 1)), kMoeStages);  // syncs: sew visible
  BlockScratch bs{&ring, lists, T, sew, 0, false};
  // weight stream first (it needs only the routing), activations while the tiles are in flight
  if (threadIdx.x == 0) {
    long lo, hi;
    block_range((long)a.slots * a.I, blockIdx.x, gridDim.x, lo, hi);
    const int SB = gateup_sub_rows(a.H);
    gateup_list(&lists[0], a, sew, (int)lo, (int)(lo + SB < hi ? lo + SB : hi));
  }
  __syncthreads();
  ring_prefetch_all(&ring, &lists[0]);
  bs.primed = true;
  StagedAct4 act = stage4(moe_smem, a.XQ, a.SQ, a.H, 1, a.H, a.H / 128);
  gateup_block_dispatch_t(a, act, bs, blockIdx.x, gridDim.x);
  if (threadIdx.x == 0) ring_drain_after_fault(&ring);
}

__global__ void __launch_bounds__(256, 2) ExpertDownCombine(const ExpertDownCombineArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ SegList lists[2];
  __shared__ float T[kTFloats];
  __shared__ Ring ring;
  __shared__ ExpertW sew[kMaxSegs];
  fetch_expert_rows(sew, a.Experts, a.SelIdx, a.slots);
  ring_init(&ring, moe_smem + moe_round128(staged4_bytes(a.I, a.slots)), kMoeStages);  // syncs: sew visible
  BlockScratch bs{&ring, lists, T, sew, 0, false};
  // weight stream first (it needs only the routing), the slots' activations are quantised while
  // the tiles are in flight
  if (threadIdx.x == 0) {
    long lo, hi;
    block_range(a.H, blockIdx.x, gridDim.x, lo, hi);
    const int SB = down_sub_rows(a.I, a.slots);
    down_list(&lists[0], a, sew, (int)lo, (int)(lo + SB < hi ? lo + SB : hi));
  }
  __syncthreads();
  ring_prefetch_all(&ring, &lists[0]);
  bs.primed = true;
  StagedAct4 act = stage4_from_f32<true>(moe_smem, a.Act, a.I, a.slots, a.I);
  down_block_dispatch_t(a, act, bs, blockIdx.x, gridDim.x);
  if (threadIdx.x == 0) ring_drain_after_fault(&ring);
}

// ---- CombineSlots: the combine step of ExpertDownCombine on its own ----
// X[n] = Res[n] + sum over slots s, in slot order, of W[s] * Y[s][n]: the same
// additions in the same order as ExpertDownCombine performs on its row sums.
// Used by the expert-parallel path, where the per-slot down-projection outputs
// Y come back from the ranks that own the experts.
struct CombineSlotsArgs {
  const float *Y;    // [slots][H] unweighted down-projection outputs
  const float *W;    // [slots] routing weights (rank order, shared expert last)
  const float *Res;  // [H]
  float *X;          // [H]
  int32_t slots, H;
};
__global__ void __launch_bounds__(256) CombineSlots(const CombineSlotsArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  for (int n = blockIdx.x * 256 + threadIdx.x; n < a.H; n += gridDim.x * 256) {
    float acc = 0.0f;
    for (int s = 0; s < a.slots; ++s) acc = acc + a.W[s] * a.Y[(size_t)s * a.H + n];
    a.X[n] = a.Res[n] + acc;
  }
}

// ---- RouterTopK with its scratch in a fixed device array (no allocation) ----
// Same work as RouterTopK, but the router logits and the block counter live in
// this file-scope array instead of caller-provided buffers. The array belongs to
// the device, so calls on one device share it: the host entry point clears the
// counter before every launch, and two calls in flight at once would race.
static __device__ __align__(256) unsigned char g_router_static_scratch[kRouterStaticScratchBytes];

__global__ void __launch_bounds__(256) RouterTopKStatic(const RouterTopKArgs a, unsigned char *scratch) {
  RouterTopKArgs b = a;
  b.Logits = reinterpret_cast<float *>(scratch);
  b.Counter = reinterpret_cast<unsigned *>(scratch + kRouterStaticCounterOffset);
  __shared__ bool is_last;
  __shared__ float sp[1024 + 1];
  router_logits_rows(b, blockIdx.x, gridDim.x);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned prev = atomicAdd(b.Counter, 1u);
    is_last = prev == gridDim.x - 1;
    if (is_last) *b.Counter = 0u;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  router_select(b.Logits, b.E, b.k, b.Wsg != nullptr, sp, b.SelIdx, b.SelW, b.NearGap);
}

// Host helpers for the C entry point (which lives with the rest of the ABI).
cudaError_t router_static_scratch_address(void **ptr) {
  return cudaGetSymbolAddress(ptr, g_router_static_scratch);
}
cudaError_t router_static_launch(cudaStream_t stream, void *scratch, const void *Wr, const void *Wsg,
                                 const float *Hn, int32_t *SelIdx, float *SelW, float *NearGap, int E, int H,
                                 int k) {
  cudaError_t e = cudaMemsetAsync(static_cast<unsigned char *>(scratch) + kRouterStaticCounterOffset, 0, 4, stream);
  if (e != cudaSuccess) return e;
  RouterTopKArgs a{};
  a.Wr = static_cast<const uint16_t *>(Wr);
  a.Wsg = static_cast<const uint16_t *>(Wsg);
  a.Hn = Hn;
  a.SelIdx = SelIdx;
  a.SelW = SelW;
  a.NearGap = NearGap;
  a.E = E;
  a.H = H;
  a.k = k;
  const unsigned groups = (unsigned)((E + 1 + 7) / 8);
  RouterTopKStatic<<<groups, 256, 0, stream>>>(a, static_cast<unsigned char *>(scratch));
  return cudaGetLastError();
}

#define F(f) AINFER_ARG(CombineSlotsArgs, f)
AINFER_REGISTER(CombineSlots, CombineSlotsArgs, 256, 256, 0, nullptr, F(Y), F(W), F(Res), F(X), F(slots), F(H));
#undef F
AINFER_EARLY_LAUNCH(CombineSlots);

#define F(f) AINFER_ARG(RouterTopKArgs, f)
AINFER_REGISTER(RouterTopK, RouterTopKArgs, 256, 8, 0, nullptr, F(Wr), F(Wsg), F(Hn), F(Logits),
                F(Counter), F(SelIdx), F(SelW), F(NearGap), F(E), F(H), F(k));
#undef F

static uint32_t gateup_smem_fn(const void *args) {
  return moe_round128(staged4_bytes(((const ExpertGateUpArgs *)args)->H, 1)) + kMoeStages * kStageStride;
}
#define F(f) AINFER_ARG(ExpertGateUpArgs, f)
AINFER_REGISTER(ExpertGateUp, ExpertGateUpArgs, 256, 0, 0, gateup_smem_fn, F(Experts), F(SelIdx),
                F(XQ), F(SQ), F(Act), F(slots), F(I), F(H), F(slot_begin));
#undef F

static uint32_t down_smem_fn(const void *args) {
  const ExpertDownCombineArgs *a = (const ExpertDownCombineArgs *)args;
  return moe_round128(staged4_bytes(a->I, a->slots)) + kMoeStages * kStageStride;
}
#define F(f) AINFER_ARG(ExpertDownCombineArgs, f)
AINFER_REGISTER(ExpertDownCombine, ExpertDownCombineArgs, 256, 0, 0, down_smem_fn, F(Experts),
                F(SelIdx), F(SelW), F(Act), F(Res), F(X), F(Moe), F(slots), F(I), F(H));
#undef F

AINFER_EARLY_LAUNCH(RouterTopK);
AINFER_EARLY_LAUNCH(ExpertGateUp);
AINFER_EARLY_LAUNCH(ExpertDownCombine);

}  // namespace ainfer
