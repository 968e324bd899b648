// DecodeStepMega: one whole decode token in ONE persistent cooperative launch.
//
// The multi-kernel path replays ~450 small launches per token and is bound by
// per-kernel latency (launch, cold instruction cache, dependent loads), not by
// HBM. Here every layer stage runs inside one kernel: blocks stay resident,
// stages are separated by a grid-wide barrier, the instruction stream stays
// warm across the 48 layers, and each stage issues L2 prefetches for the
// weights of the NEXT stage before it computes, so HBM keeps streaming while
// blocks compute and wait. The arithmetic of every stage is the same device
// code the stand-alone kernels run (gemv_stage.cuh, deltanet_core.cuh,
// attention_core.cuh, moe_core.cuh), so results are bit-identical.
//
// Replaces, per token, the 66 execute+fence round trips of the reference's
// token loop (tools/decode/decode_l0.cpp:742-775) and the host-side control
// update between tokens (:753-756,816-818).
//
// Every wait is bounded: a barrier that does not complete within kSpinLimit
// polls sets plan->error and all blocks leave the kernel.
#define AINFER_STAMP(id) ::ainfer::fine_stamp(id)
namespace ainfer {
static __device__ void fine_stamp(int id);
}
#include "../common/mega_plan.h"
#include "attention_core.cuh"
#include "deltanet_core.cuh"
#include "block_stages.cuh"
#include "norm_stages.cuh"
#include "tail_core.cuh"

namespace ainfer {

struct DecodeStepMegaArgs {
  const MegaPlan *plan;
  int32_t mode;  // 1: final norm + lm_head + argmax, control advances to the selected token
                 // 0: prompt step, control advances to ids[position + 1]
};

constexpr unsigned kSpinLimit = 1u << 22;
constexpr int kStageBytes = 13056;   // staged activations: max(K<=8192 x1, I<=1024 x12)

// Fine stage clock (second half of the stamp buffer): block 0 / thread 0 appends
// (id << 48) | low 48 bits of %globaltimer at points inside the stages.
__shared__ unsigned long long *s_fine;
__shared__ int s_fine_n, s_fine_cap;
static __device__ __noinline__ void fine_stamp(int id) {
  if (threadIdx.x == 0 && s_fine != nullptr && s_fine_n < s_fine_cap) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    s_fine[s_fine_n++] = ((unsigned long long)id << 48) | (t & 0xFFFFFFFFFFFFull);
    if (id >= 60 && s_fine_n < s_fine_cap) {  // ids >= 60 also record the SM cycle counter (for the clock rate)
      long long c = clock64();
      s_fine[s_fine_n++] = ((unsigned long long)(id + 1) << 48) | ((unsigned long long)c & 0xFFFFFFFFFFFFull);
    }
  }
}

struct GridSync {
  unsigned *count;
  int *error;
  unsigned epoch;
  unsigned nblk;
  unsigned long long *stamps;  // optional stage clock (block 0 only)
  int stamp_cap;
  int nstamp;
};

// Stage clock: block 0 / thread 0 appends %globaltimer (ns) when the plan asks for it.
__device__ __forceinline__ void stage_stamp(GridSync &g) {
  if (g.stamps && threadIdx.x == 0) {
    if (g.nstamp < g.stamp_cap) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      g.stamps[g.nstamp] = t;
    }
    g.nstamp += 1;
  }
}

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Grid-wide barrier over a monotonically increasing counter (zeroed before the
// launch). Returns true when the kernel must stop (a wait ran out of polls
// here or in another block).
// The barrier comes in two halves so that work which does not depend on other
// blocks (building the next stage's tables, starting its weight copies) can run
// between announcing arrival and waiting for the others.
__device__ __forceinline__ void grid_arrive(GridSync &g) {
  __syncthreads();
  AINFER_STAMP(40);
  g.epoch += 1;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(g.count, 1u);
  }
}
__device__ __forceinline__ bool grid_wait(GridSync &g) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) {
    int fail = 0;
    const unsigned target = g.epoch * g.nblk;
    unsigned spins = 0;
    while (ld_acquire_u32(g.count) < target) {
      if (++spins > kSpinLimit) {
        atomicExch(g.error, 1);
        fail = 1;
        break;
      }
      if ((spins & 255u) == 0 && *(volatile int *)g.error != 0) {
        fail = 1;
        break;
      }
    }
    __threadfence();
    s_fail = fail;
  }
  __syncthreads();
  stage_stamp(g);
  return s_fail != 0;
}
__device__ __forceinline__ bool grid_barrier(GridSync &g) {
  grid_arrive(g);
  return grid_wait(g);
}

// Asks L2 to fetch [p, p+bytes): one 128-byte line per request, spread over the block.
__device__ __forceinline__ void prefetch_l2(const void *p, size_t bytes) {
  const char *c = reinterpret_cast<const char *>(p);
  for (size_t off = (size_t)threadIdx.x * 128; off < bytes; off += (size_t)blockDim.x * 128)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(c + off));
}

// Prefetches the weight rows this block will read in a GEMV stage (same
// contiguous row range as gemv_block deals out).
__device__ __forceinline__ void prefetch_gemv(const GemvMat *mats, int nmats, int K, int blk, int nblk) {
  long total = 0;
  for (int i = 0; i < nmats; ++i) total += mats[i].N;
  long lo, hi;
  block_range(total, blk, nblk, lo, hi);
  long rs = 0;
  for (int i = 0; i < nmats; ++i) {
    long a = lo > rs ? lo : rs, b = hi < rs + mats[i].N ? hi : rs + mats[i].N;
    if (a < b) {
      prefetch_l2(mats[i].P + (a - rs) * (K / 2), (size_t)(b - a) * (K / 2));
      prefetch_l2(mats[i].S + (a - rs) * (K / 128), (size_t)(b - a) * (K / 128) * 2);
    }
    rs += mats[i].N;
  }
}

// Leaves the kernel early (a grid barrier gave up): prefetched copies may still be landing.
__device__ __forceinline__ void mega_bail(Ring *ring) {
  if (threadIdx.x == 0) ring_drain(ring);
}

// Prepares a GEMV stage ahead of time: builds the stage's matrix table in shared
// memory (row_start assigned here) and the block's first segment list, and
// starts the bulk copies of its first tiles. Called once the previous user of
// smats / the lists / the ring is done, typically BEFORE the grid barrier that
// guards the stage's activations: the weights do not depend on them, so they
// stream into shared memory while the block waits.
static __device__ __noinline__ void gemv_prepare(const GemvMat *mats, int nmats, int K, GemvMat *smats,
                                             BlockScratch &bs, int blk, int nblk) {
  __syncthreads();  // smats / lists may still be read by the previous stage's epilogue
  if (threadIdx.x < nmats) smats[threadIdx.x] = mats[threadIdx.x];  // one round trip for all records
  __syncthreads();
  if (threadIdx.x == 0) {
    int row = 0;
    for (int i = 0; i < nmats; ++i) {
      smats[i].row_start = row;
      row += smats[i].N;
    }
    gemv_first_list(&bs.lists[bs.cur], smats, nmats, K, row, blk, nblk);
    ring_prefetch(bs.ring, &bs.lists[bs.cur]);
  }
  bs.primed = true;
}

// Runs one GEMV stage for this block over its contiguous rows.
static __device__ __noinline__ void gemv_stage(const GemvMat *mats, int nmats, int K, const StagedAct4 &act,
                                           GemvMat *smats, BlockScratch &bs, int blk, int nblk) {
  if (!bs.primed) gemv_prepare(mats, nmats, K, smats, bs, blk, nblk);
  __syncthreads();
  AINFER_STAMP(10);
  long total = 0;
  for (int i = 0; i < nmats; ++i) total += smats[i].N;
  gemv_block<false>(K, smats, nmats, total, act, bs, blk, nblk);
}

// Same for the expert down projection, once the routing is known.
static __device__ __noinline__ void down_prepare(const ExpertDownCombineArgs &xa, BlockScratch &bs, int blk,
                                             int nblk) {
  __syncthreads();
  if (threadIdx.x == 0) {
    long lo, hi;
    block_range(xa.H, blk, nblk, lo, hi);
    const int SB = down_sub_rows(xa.I, xa.slots);
    down_list(&bs.lists[bs.cur], xa, bs.sew, (int)lo, (int)(lo + SB < hi ? lo + SB : hi));
    ring_prefetch(bs.ring, &bs.lists[bs.cur]);
  }
  bs.primed = true;
}

// Prefetch of the down-projection rows this block reads in the next stage.
__device__ __forceinline__ void prefetch_down(const ExpertW *experts, const int32_t *sel, int slots, int I,
                                              int H, int blk, int nblk) {
  long lo, hi;
  block_range(H, blk, nblk, lo, hi);
  if (lo >= hi) return;
  for (int s = 0; s < slots; ++s) {
    const ExpertW &ew = experts[sel[s]];
    prefetch_l2(ew.dP + lo * (I / 2), (size_t)(hi - lo) * (I / 2));
    prefetch_l2(ew.dS + lo * (I / 128), (size_t)(hi - lo) * (I / 128) * 2);
  }
}

// The stage bodies shared with the stand-alone kernels, as separate functions:
// each gets its own register allocation instead of competing inside one huge
// kernel body (which spilled in the hot loops).
static __device__ __noinline__ void mega_deltanet(const DeltaNetStepArgs &a, int blk, int nblk) {
  deltanet_step_body(a, blk, nblk);
}
static __device__ __noinline__ void mega_attn_prep(const AttnPrepArgs &a, int blk, int nblk) {
  attn_prep_body(a, blk, nblk);
}
static __device__ __noinline__ void mega_attn_split(const AttnSplitArgs &a, int blk, int nblk) {
  attn_split_dispatch<false>(a, blk, nblk);
}
static __device__ __noinline__ void mega_attn_combine(const AttnCombineArgs &a, int blk, int nblk) {
  attn_combine_body(a, blk, nblk);
}
static __device__ __noinline__ void mega_gateup(const ExpertGateUpArgs &a, const StagedAct4 &act, BlockScratch &bs,
                                                int blk, int nblk) {
  gateup_block_dispatch<false>(a, act, bs, blk, nblk);
}
static __device__ __noinline__ void mega_down(const ExpertDownCombineArgs &a, const StagedAct4 &act,
                                              BlockScratch &bs, int blk, int nblk) {
  down_block_dispatch<false>(a, act, bs, blk, nblk);
}
static __device__ __noinline__ StagedAct4 mega_stage_rows(unsigned char *stage, const float *x, int K, int M) {
  __syncthreads();
  return stage4_from_f32<true>(stage, x, K, M, K);
}

extern __shared__ __align__(128) unsigned char mega_smem[];
constexpr int kMegaStages = 3;
constexpr int kMegaRingOff = (kStageBytes + kYsFloats * 4 + kTFloats * 4 + 127) / 128 * 128;

__global__ void __launch_bounds__(256, 2) DecodeStepMega(const DecodeStepMegaArgs args) {
  const MegaPlan &P = *args.plan;
  __shared__ GemvMat smats[8];
  __shared__ SegList s_lists[2];
  __shared__ Ring s_ring;
  __shared__ int32_t s_sel_idx[16];
  __shared__ float s_sel_w[16];
  __shared__ float s_gap;
  __shared__ float s_av[8];
  __shared__ int s_ai[8];
  unsigned char *stage = mega_smem;
  float *ys = reinterpret_cast<float *>(mega_smem + kStageBytes);
  ring_init(&s_ring, mega_smem + kMegaRingOff, kMegaStages);
  __shared__ ExpertW s_sew[kMaxSegs];
  BlockScratch bs{&s_ring, s_lists, reinterpret_cast<float *>(mega_smem + kStageBytes + kYsFloats * 4), s_sew, 0, false};
  const int blk = blockIdx.x, nblk = gridDim.x;
  if (threadIdx.x == 0) {
    s_fine = (blk == 0 && P.stage_stamps) ? P.stage_stamps + P.stage_stamp_cap / 2 : nullptr;
    s_fine_n = 0;
    s_fine_cap = P.stage_stamp_cap / 2;
  }
  GridSync gs{P.bar_count, P.error, 0u, (unsigned)nblk, blk == 0 ? P.stage_stamps : nullptr, P.stage_stamp_cap / 2, 0};
  stage_stamp(gs);
  __syncthreads();
  AINFER_STAMP(60);
  if (*(volatile int *)P.error != 0) return;  // a previous launch failed: stay out
  const int H = P.H;
  const int token = __ldcg(P.ctrl + CTRL_TOKEN);
  int tok = token < 0 ? 0 : (token >= P.vocab ? P.vocab - 1 : token);

  gemv_prepare(&P.L[0].m[0], P.L[0].type == 0 ? 4 : 3, H, smats, bs, blk, nblk);
  for (int L = 0; L < P.layers; ++L) {
    const MegaLayer &ly = P.L[L];
    // ---- mixer input: (1+w) RMSNorm + quantiser, redundantly per block ----
    StagedAct4 act = norm_quant_stage(P.X, L == 0 ? P.emb + (size_t)tok * H : nullptr, ly.in_norm, H, P.eps,
                                     stage, ys, (L == 0 && blk == 0) ? P.X : nullptr);
    if (P.layer_out && L > 0 && blk == 0)
      for (int j = threadIdx.x; j < H; j += 256) P.layer_out[(size_t)(L - 1) * H + j] = __ldcg(P.X + j);
    if (ly.type == 0) {
      // in_proj qkv (+conv+SiLU), z, b (sigmoid), a (decay)
      stage_stamp(gs);  // norm + quant done
      gemv_stage(&ly.m[0], 4, H, act, smats, bs, blk, nblk);
      stage_stamp(gs);  // this block's rows done
      grid_arrive(gs);
      gemv_prepare(&ly.m[4], 1, P.nV * 128, smats, bs, blk, nblk);  // out_proj streams in during the recurrence
      if (grid_wait(gs)) return mega_bail(&s_ring);
      DeltaNetStepArgs da{P.O, P.Mx, ly.S, P.Bt, P.Gt, P.nK, P.nV};
      mega_deltanet(da, blk, nblk);
      if (grid_barrier(gs)) return mega_bail(&s_ring);
      act = gated_norm_stage(P.O, P.Z, ly.lin_norm, P.nV, P.eps, stage, ys);
      gemv_stage(&ly.m[4], 1, P.nV * 128, act, smats, bs, blk, nblk);
    } else {
      gemv_stage(&ly.m[0], 3, H, act, smats, bs, blk, nblk);
      grid_arrive(gs);
      gemv_prepare(&ly.m[4], 1, P.nQ * 256, smats, bs, blk, nblk);  // o_proj streams in during attention
      if (grid_wait(gs)) return mega_bail(&s_ring);
      AttnPrepArgs pa{P.Q16, P.K16, P.V16, ly.q_norm, ly.k_norm, P.Cos, P.Sin, P.ctrl, P.Qn,
                      ly.Kc, ly.Vc, ly.Ks, ly.Vs, P.nQ, P.nKV, P.rot, P.max_ctx, P.eps};
      mega_attn_prep(pa, blk, nblk);
      if (grid_barrier(gs)) return mega_bail(&s_ring);
      AttnSplitArgs sa{P.Qn, ly.Kc, ly.Vc, ly.Ks, ly.Vs, P.ctrl, P.Pm, P.Pse, P.Pacc,
                       P.nQ, P.nKV, P.max_ctx, P.max_chunks};
      mega_attn_split(sa, blk, nblk);
      if (grid_barrier(gs)) return mega_bail(&s_ring);
      AttnCombineArgs ca{P.Pm, P.Pse, P.Pacc, P.Q16, P.ctrl, P.Q8, P.SQ, nullptr, P.nQ, P.max_ctx, P.max_chunks};
      mega_attn_combine(ca, blk, nblk);
      if (grid_barrier(gs)) return mega_bail(&s_ring);
      __syncthreads();
      act = stage4(stage, P.Q8, P.SQ, P.nQ * 256, 1, P.nQ * 256, P.nQ * 2);
      gemv_stage(&ly.m[4], 1, P.nQ * 256, act, smats, bs, blk, nblk);
    }
    // router rows of this block: ask for them while the projection's results settle
    {
      const int rows = P.E + (ly.shared_gate ? 1 : 0);
      for (int e = blk * 8; e < rows; e += nblk * 8) {
        int n = rows - e < 8 ? rows - e : 8;
        if (e + n <= P.E) prefetch_l2(ly.router + (size_t)e * H, (size_t)n * H * 2);
        else {
          if (e < P.E) prefetch_l2(ly.router + (size_t)e * H, (size_t)(P.E - e) * H * 2);
          prefetch_l2(ly.shared_gate, (size_t)H * 2);
        }
      }
    }
    if (grid_barrier(gs)) return mega_bail(&s_ring);
    // ---- MoE: post norm, router, top-k, experts ----
    act = norm_quant_stage(P.Tmp, nullptr, ly.post_norm, H, P.eps, stage, ys, nullptr);
    stage_stamp(gs);
    router_rows_smem(ly.router, ly.shared_gate, ys, P.RLogits, P.E, H, blk, nblk);
    stage_stamp(gs);
    // next layer's first projections (or the LM head) stream in during the MoE stages
    if (L + 1 < P.layers) {
      const MegaLayer &nx = P.L[L + 1];
      prefetch_gemv(&nx.m[0], nx.type == 0 ? 4 : 3, H, blk, nblk);
    }
    if (grid_barrier(gs)) return mega_bail(&s_ring);
    router_select(P.RLogits, P.E, P.topk, ly.shared_gate != nullptr, ys, s_sel_idx, s_sel_w, &s_gap);
    fetch_expert_rows(s_sew, ly.experts, s_sel_idx, P.slots);  // synchronised inside the gate/up stage
    stage_stamp(gs);  // selection done
    if (blk == 0 && threadIdx.x <= P.topk) {
      P.SelIdx[threadIdx.x] = s_sel_idx[threadIdx.x];
      P.SelW[threadIdx.x] = s_sel_w[threadIdx.x];
      if (threadIdx.x == 0) *P.NearGap = s_gap;
      if (P.routed) {
        P.routed[(size_t)L * (P.topk + 1) + threadIdx.x] = s_sel_idx[threadIdx.x];
        if (threadIdx.x == 0) P.near_gap[L] = s_gap;
      }
    }
    {
      ExpertGateUpArgs ga{ly.experts, s_sel_idx, nullptr, nullptr, P.Act, P.slots, P.I, H, 0};
      mega_gateup(ga, act, bs, blk, nblk);
      stage_stamp(gs);
    }
    {
      ExpertDownCombineArgs xa{ly.experts, s_sel_idx, s_sel_w, P.Act, P.Tmp, P.X, nullptr, P.slots, P.I, H};
      grid_arrive(gs);
      down_prepare(xa, bs, blk, nblk);  // the routing is known: down rows stream in during the barrier
      if (grid_wait(gs)) return mega_bail(&s_ring);
      StagedAct4 dact = mega_stage_rows(stage, P.Act, P.I, P.slots);
      stage_stamp(gs);
      mega_down(xa, dact, bs, blk, nblk);
      stage_stamp(gs);
    }
    grid_arrive(gs);
    // the next layer's first projections (or the LM head) stream in during the barrier and its norm
    if (L + 1 < P.layers) gemv_prepare(&P.L[L + 1].m[0], P.L[L + 1].type == 0 ? 4 : 3, H, smats, bs, blk, nblk);
    else if (args.mode != 0) gemv_prepare(&P.lm_head, 1, H, smats, bs, blk, nblk);
    if (grid_wait(gs)) return mega_bail(&s_ring);
  }
  if (P.layer_out && blk == 0)
    for (int j = threadIdx.x; j < H; j += 256)
      P.layer_out[(size_t)(P.layers - 1) * H + j] = __ldcg(P.X + j);

  if (args.mode == 0) {
    // prompt step: no logits; move on to the next prompt id
    if (blk == 0 && threadIdx.x == 0) {
      int pos = P.ctrl[CTRL_POS] + 1;
      P.ctrl[CTRL_POS] = pos;
      P.ctrl[CTRL_LEN] = P.ctrl[CTRL_LEN] + 1;
      if (pos < P.max_ctx) P.ctrl[CTRL_TOKEN] = P.ids[pos];
      P.ctrl[CTRL_SELECTED] = -1;
    }
    return;
  }
  // ---- tail: final norm, LM head, first-max-wins argmax, control update ----
  AINFER_STAMP(62);
  {
    StagedAct4 act = norm_quant_stage(P.X, nullptr, P.final_norm, H, P.eps, stage, ys, nullptr);
    gemv_stage(&P.lm_head, 1, H, act, smats, bs, blk, nblk);
  }
  if (grid_barrier(gs)) return mega_bail(&s_ring);
  {
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int i = blk * 256 + threadIdx.x; i < P.vocab; i += nblk * 256) argmax_merge(bv, bi, __ldcg(P.Logits + i), i);
    block_argmax(bv, bi, s_av, s_ai);
    if (threadIdx.x == 0) {
      P.PV[blk] = bv;
      P.PI[blk] = bi;
    }
  }
  if (grid_barrier(gs)) return mega_bail(&s_ring);
  if (blk == 0) {
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < nblk; i += 256) argmax_merge(bv, bi, __ldcg(P.PV + i), __ldcg(P.PI + i));
    __syncthreads();
    block_argmax(bv, bi, s_av, s_ai);
    if (threadIdx.x == 0) {
      P.out_tok[0] = bi;
      int pos = P.ctrl[CTRL_POS];
      if (P.history && P.history_cap > 0) P.history[pos % P.history_cap] = bi;
      P.ctrl[CTRL_SELECTED] = bi;
      P.ctrl[CTRL_TOKEN] = bi;
      P.ctrl[CTRL_POS] = pos + 1;
      P.ctrl[CTRL_LEN] = P.ctrl[CTRL_LEN] + 1;
    }
  }
}

static uint32_t mega_smem_fn(const void *) { return (uint32_t)(kMegaRingOff + kMegaStages * kStageStride); }

#define F(f) AINFER_ARG(DecodeStepMegaArgs, f)
AINFER_REGISTER_COOP(DecodeStepMega, DecodeStepMegaArgs, 256, 0, 0, mega_smem_fn, F(plan), F(mode));
#undef F

}  // namespace ainfer
