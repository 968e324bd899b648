// Kernel entries of the mixture-of-experts block; bodies in moe_core.cuh
// (shared with the persistent decode kernel).
#define AINFER_BLOCK_DOT_INLINE 1

#include "direct_dot.cuh"

namespace ainfer {

extern __shared__ __align__(128) unsigned char moe_smem[];

__global__ void __launch_bounds__(256) RouterTopK(const RouterTopKArgs a) {
  pdl_launch_dependents();
  // the router's weights do not depend on the producer of Hn: fetch the first row's share first
  RouterRowRegs first;
  {
    const int e = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (e < a.E + (a.Wsg ? 1 : 0)) router_row_load(first, router_row_ptr(a, e), 0, a.H / 256, threadIdx.x & 31);
  }
  pdl_wait();
  __shared__ bool is_last;
  __shared__ float sp[1024 + 1];
  router_logits_rows(a, blockIdx.x, gridDim.x, &first);
  AINFER_MARK(1);
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
  router_publish_rows(a);
}

__host__ __device__ inline uint32_t moe_round128(uint32_t v) { return (v + 127u) & ~127u; }
constexpr int kMoeTasks = 3;  // 64-byte weight groups a thread keeps in flight

// The down projections of the same experts are read by the next kernel: start them towards L2.
// Every thread of every block calls; the lines are dealt over the whole grid.
__device__ __forceinline__ void prefetch_down_rows(const ExpertGateUpArgs &a, const ExpertW *sew) {
  const int wl = a.H * (a.I / 2) / 128, sl = a.H * (a.I / 128) * 2 / 128;  // lines per slot: weights, scales
  const int per = wl + sl, total = a.slots * per;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int s = i / per, l = i - s * per;
    prefetch_l2(l < wl ? sew[s].dP + (size_t)l * 128
                       : reinterpret_cast<const uint8_t *>(sew[s].dS) + (size_t)(l - wl) * 128);
  }
}

// The expert kernels stream only a few tens of KB per block (top-k experts of one token), so
// they take the weights by direct loads (direct_dot.cuh), not through the shared-memory ring.
__global__ void __launch_bounds__(256, 2) ExpertGateUp(const ExpertGateUpArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ SegList list;
  __shared__ float T[kTFloats];
  __shared__ ExpertW sew[kMaxSegs];
  // the routing first, the hidden vector's loads next, then the dependent load of the selected
  // experts' pointer records (a warp issues in order)
  const int t = threadIdx.x;
  const bool row_thread = t < a.slots * 3 && t < kMaxSegs * 3;
  int sel = 0;
  if (row_thread) sel = a.SelIdx ? __ldcg(a.SelIdx + a.slot_begin + t / 3) : a.slot_begin + t / 3;
  StagedAct4 act = stage4_issue_first(moe_smem, a.XQ, a.SQ, a.H, [&] {
    if (row_thread)
      reinterpret_cast<uint4 *>(sew + t / 3)[t % 3] = __ldg(reinterpret_cast<const uint4 *>(a.Experts + sel) + t % 3);
  });  // ends with a barrier: sew visible
  AINFER_MARK(1);
  const int SB = gateup_sub_rows(a.H);  // pair rows per sub-block
  const int G = a.H / 128;
  long lo, hi;
  block_range((long)a.slots * a.I, blockIdx.x, gridDim.x, lo, hi);
#pragma unroll 1
  for (long sb = lo; sb < hi; sb += SB) {
    const long se = sb + SB < hi ? sb + SB : hi;
    gateup_list_par(&list, a, sew, (int)sb, (int)se);
    __syncthreads();  // list complete; T of the previous sub-block is no longer read
    AINFER_MARK(2);
    direct_dot<kMoeTasks>(&list, act, T);
    if (a.prefetch_down && sb == lo) prefetch_down_rows(a, sew);
    __syncthreads();
    AINFER_MARK(3);
    const long r = sb + threadIdx.x;
    if (r < se) {
      const float g = row_sum_rt(T, threadIdx.x, G), u = row_sum_rt(T, SB + threadIdx.x, G);
      a.Act[(size_t)a.slot_begin * a.I + r] = silu_mul(g, u);
    }
  }
  AINFER_MARK(9);
}

__global__ void __launch_bounds__(256, 2) ExpertDownCombine(const ExpertDownCombineArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ SegList list;
  __shared__ float T[kTFloats];
  __shared__ ExpertW sew[kMaxSegs];
  __shared__ float sw[kMaxSegs];
  // Every independent load first (routing, weights of the combine, the slots' activations),
  // then the one dependent load (the selected experts' pointer records); the activation
  // quantiser runs while that is in flight.
  const int t = threadIdx.x;
  const bool row_thread = t < a.slots * 3 && t < kMaxSegs * 3;
  int sel = 0;
  float selw = 0.0f;
  if (row_thread) sel = a.SelIdx ? __ldcg(a.SelIdx + t / 3) : t / 3;
  if (t < a.slots && t < kMaxSegs) selw = __ldcg(a.SelW + t);
  // activations: rolled shared-memory quantiser when they fit its copy (slots * I <= 8192)
  const int count4 = a.slots * a.I / 4;
  const bool rolled = count4 <= 8 * 256;
  float *raw = reinterpret_cast<float *>(moe_smem + moe_round128(staged4_bytes(a.I, a.slots)));
  StagedAct4 act;
  if (rolled) {
    RawCopy rc;
    raw_copy_load(rc, a.Act, count4);
    uint4 row = make_uint4(0, 0, 0, 0);
    if (row_thread) row = __ldg(reinterpret_cast<const uint4 *>(a.Experts + sel) + t % 3);
    raw_copy_store(rc, raw, count4);
    if (row_thread) reinterpret_cast<uint4 *>(sew + t / 3)[t % 3] = row;
    if (t < a.slots && t < kMaxSegs) sw[t] = selw;
    __syncthreads();
    act = quant_rolled(moe_smem, raw, a.I, a.slots);  // ends with a barrier
  } else {
    QuantWide qw;
    quant_wide_load(qw, a.Act, a.I, a.slots, a.I, 0);
    uint4 row = make_uint4(0, 0, 0, 0);
    if (row_thread) row = __ldg(reinterpret_cast<const uint4 *>(a.Experts + sel) + t % 3);
    quant_wide_store(qw, moe_smem, a.I, a.slots, 0);
    if (row_thread) reinterpret_cast<uint4 *>(sew + t / 3)[t % 3] = row;
    if (t < a.slots && t < kMaxSegs) sw[t] = selw;
    act = quant_wide_finish(moe_smem, a.Act, a.I, a.slots, a.I);  // ends with a barrier
  }
  AINFER_MARK(1);
  const int SB = down_sub_rows(a.I, a.slots);
  const int G = a.I / 128;
  long lo, hi;
  block_range(a.H, blockIdx.x, gridDim.x, lo, hi);
#pragma unroll 1
  for (long sb = lo; sb < hi; sb += SB) {
    const long se = sb + SB < hi ? sb + SB : hi;
    const int nr = (int)(se - sb);
    down_list_par(&list, a, sew, (int)sb, (int)se);
    const long n = sb + threadIdx.x;
    const float res = n < se ? __ldcg(a.Res + n) : 0.0f;  // in flight while the weights are fetched
    __syncthreads();
    AINFER_MARK(2);
    direct_dot<kMoeTasks>(&list, act, T);
    __syncthreads();
    AINFER_MARK(3);
    if (n < se) {
      float acc = 0.0f;
      for (int s = 0; s < a.slots; ++s) acc = acc + sw[s] * row_sum_rt(T, s * nr + threadIdx.x, G);
      if (a.Moe) a.Moe[n] = acc;
      a.X[n] = res + acc;
    }
  }
  AINFER_MARK(9);
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
                F(Counter), F(SelIdx), F(SelW), F(NearGap), F(E), F(H), F(k), F(Experts), F(SelRows));
#undef F

static uint32_t gateup_smem_fn(const void *args) {
  return moe_round128(staged4_bytes(((const ExpertGateUpArgs *)args)->H, 1));
}
#define F(f) AINFER_ARG(ExpertGateUpArgs, f)
AINFER_REGISTER(ExpertGateUp, ExpertGateUpArgs, 256, 0, 0, gateup_smem_fn, F(Experts), F(SelIdx),
                F(XQ), F(SQ), F(Act), F(slots), F(I), F(H), F(slot_begin), F(prefetch_down));
#undef F

static uint32_t down_smem_fn(const void *args) {
  const ExpertDownCombineArgs *a = (const ExpertDownCombineArgs *)args;
  const uint32_t raw = (uint32_t)a->slots * (uint32_t)a->I * 4u;  // fp32 copy for the rolled quantiser
  return moe_round128(staged4_bytes(a->I, a->slots)) + (raw <= 8192u * 4u ? raw : 0u);
}
#define F(f) AINFER_ARG(ExpertDownCombineArgs, f)
AINFER_REGISTER(ExpertDownCombine, ExpertDownCombineArgs, 256, 0, 0, down_smem_fn, F(Experts),
                F(SelIdx), F(SelW), F(Act), F(Res), F(X), F(Moe), F(slots), F(I), F(H));
#undef F

AINFER_EARLY_LAUNCH(RouterTopK);
AINFER_EARLY_LAUNCH(ExpertGateUp);
AINFER_EARLY_LAUNCH(ExpertDownCombine);

}  // namespace ainfer
