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
#include "../common/mega_plan.h"
#include "attention_core.cuh"
#include "deltanet_core.cuh"
#include "block_stages.cuh"
#include "tail_core.cuh"

namespace ainfer {

struct DecodeStepMegaArgs {
  const MegaPlan *plan;
  int32_t mode;  // 1: final norm + lm_head + argmax, control advances to the selected token
                 // 0: prompt step, control advances to ids[position + 1]
};

constexpr unsigned kSpinLimit = 1u << 22;
constexpr int kStageBytes = 13056;   // staged activations: max(K<=8192 x1, I<=1024 x12)
constexpr int kYsFloats = 4096;      // fp32 vector of a norm stage (hidden, value_dim, q_heads*256)

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
__device__ __forceinline__ bool grid_barrier(GridSync &g) {
  __shared__ int s_fail;
  __syncthreads();
  g.epoch += 1;
  if (threadIdx.x == 0) {
    int fail = 0;
    __threadfence();
    atomicAdd(g.count, 1u);
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

// Runs one GEMV stage for this block: builds the stage's matrix table in shared
// memory (row_start assigned here) and processes the block's contiguous rows.
__device__ __forceinline__ void gemv_stage(const GemvMat *mats, int nmats, int K, const StagedAct4 &act,
                                           GemvMat *smats, BlockScratch &bs, int blk, int nblk) {
  __syncthreads();  // smats may still be read by the previous stage
  if (threadIdx.x == 0) {
    int row = 0;
    for (int i = 0; i < nmats; ++i) {
      smats[i] = mats[i];
      smats[i].row_start = row;
      row += mats[i].N;
    }
  }
  __syncthreads();
  long total = 0;
  for (int i = 0; i < nmats; ++i) total += smats[i].N;
  // only the contraction widths a decode layer can have (the host refuses other shapes)
  switch (K) {
    case 256: gemv_block<256>(smats, nmats, total, act, bs, blk, nblk); break;
    case 512: gemv_block<512>(smats, nmats, total, act, bs, blk, nblk); break;
    case 1024: gemv_block<1024>(smats, nmats, total, act, bs, blk, nblk); break;
    case 2048: gemv_block<2048>(smats, nmats, total, act, bs, blk, nblk); break;
    case 4096: gemv_block<4096>(smats, nmats, total, act, bs, blk, nblk); break;
    default: break;
  }
}

// (1+w) RMSNorm + activation quantiser of one fp32 vector, result staged in
// shared memory for the GEMV rows; ys keeps the normalised fp32 vector (the
// router reads it). Same arithmetic as RmsNormQuant (k_norm.cu). src is either
// a global fp32 vector or a BF16 embedding row.
__device__ __forceinline__ StagedAct4 norm_quant_stage(const float *xg, const uint16_t *emb_row,
                                                      const float *w, int N, float eps,
                                                      unsigned char *stage, float *ys,
                                                      float *x_copy_out) {
  __shared__ double ps[256];
  __shared__ float s_inv;
  const int lid = threadIdx.x;
  __syncthreads();  // ys / stage may still be in use by the previous stage
  double ss = 0;
  for (int j = lid; j < N; j += 256) {
    float v = emb_row ? bf16_to_f32(emb_row[j]) : __ldcg(xg + j);
    ys[j] = v;
    if (x_copy_out) x_copy_out[j] = v;
    double d = (double)v;
    ss = ss + d * d;
  }
  ps[lid] = ss;
  __syncthreads();
  for (int st = 128; st >= 32; st >>= 1) {
    if (lid < st) ps[lid] = ps[lid] + ps[lid + st];
    __syncthreads();
  }
  if (lid < 32) {
    double v = ps[lid];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = v + __shfl_xor_sync(kFull, v, off);
    if (lid == 0) s_inv = 1.0f / sqrtf((float)(v / (double)N) + eps);
  }
  __syncthreads();
  const float inv = s_inv;
  for (int j = lid; j < N; j += 256) ys[j] = (ys[j] * inv) * (1.0f + w[j]);
  __syncthreads();
  return stage4_from_f32<false>(stage, ys, N, 1, N);
}

// Per-head gated RMSNorm (RmsInv + NormGated, tools/cmdlist/kernels.cpp:619-644)
// of all heads into ys, then the activation quantiser staged for out_proj.
// Same arithmetic as GatedNormQuant (k_norm.cu).
__device__ __forceinline__ StagedAct4 gated_norm_stage(const float *O, const float *Z, const float *W,
                                                      int heads, float eps, unsigned char *stage,
                                                      float *ys) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  for (int h = warp; h < heads; h += 8) {
    float ov[4];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ov[i] = __ldcg(O + (size_t)h * 128 + lane + 32 * i);
      ss = fmaf(ov[i], ov[i], ss);
    }
    ss = warp_tree_sum(ss);
    float inv = 1.0f / sqrtf(ss / 128.0f + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int d = lane + 32 * i;
      float zv = __ldcg(Z + (size_t)h * 128 + d);
      ys[h * 128 + d] = ((W[d] * ov[i]) * inv) * (zv / (1.0f + det_expf(-zv)));
    }
  }
  __syncthreads();
  return stage4_from_f32<false>(stage, ys, heads * 128, 1, heads * 128);
}

// Router logits with the normalised activations held in shared memory.
__device__ __forceinline__ void router_rows_smem(const uint16_t *Wr, const uint16_t *Wsg, const float *hn,
                                                 float *logits, int E, int H, int blk, int nblk) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = E + (Wsg ? 1 : 0);
  for (int e = blk * 8 + warp; e < rows; e += nblk * 8) {
    const uint16_t *w = e < E ? Wr + (size_t)e * H : Wsg;
    float acc = 0.0f;
    for (int i = 0; i < H / 256; ++i) {
      int k0 = (i * 32 + lane) * 8;
      uint4 wv = *reinterpret_cast<const uint4 *>(w + k0);
      float4 x0 = *reinterpret_cast<const float4 *>(hn + k0);
      float4 x1 = *reinterpret_cast<const float4 *>(hn + k0 + 4);
      acc = fmaf(u2f(wv.x << 16), x0.x, acc);
      acc = fmaf(u2f(wv.x & 0xFFFF0000u), x0.y, acc);
      acc = fmaf(u2f(wv.y << 16), x0.z, acc);
      acc = fmaf(u2f(wv.y & 0xFFFF0000u), x0.w, acc);
      acc = fmaf(u2f(wv.z << 16), x1.x, acc);
      acc = fmaf(u2f(wv.z & 0xFFFF0000u), x1.y, acc);
      acc = fmaf(u2f(wv.w << 16), x1.z, acc);
      acc = fmaf(u2f(wv.w & 0xFFFF0000u), x1.w, acc);
    }
    acc = warp_tree_sum(acc);
    if (lane == 0) logits[e] = acc;
  }
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

extern __shared__ __align__(128) unsigned char mega_smem[];
constexpr int kMegaStages = 3;
constexpr int kMegaRingOff = (kStageBytes + kYsFloats * 4 + kTCap * 4 + 127) / 128 * 128;

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
  BlockScratch bs{&s_ring, s_lists, reinterpret_cast<float *>(mega_smem + kStageBytes + kYsFloats * 4), 0, false};
  const int blk = blockIdx.x, nblk = gridDim.x;
  GridSync gs{P.bar_count, P.error, 0u, (unsigned)nblk, blk == 0 ? P.stage_stamps : nullptr, P.stage_stamp_cap, 0};
  stage_stamp(gs);
  if (*(volatile int *)P.error != 0) return;  // a previous launch failed: stay out
  const int H = P.H;
  const int token = __ldcg(P.ctrl + CTRL_TOKEN);
  int tok = token < 0 ? 0 : (token >= P.vocab ? P.vocab - 1 : token);

  for (int L = 0; L < P.layers; ++L) {
    const MegaLayer &ly = P.L[L];
    // ---- mixer input: (1+w) RMSNorm + quantiser, redundantly per block ----
    StagedAct4 act = norm_quant_stage(P.X, L == 0 ? P.emb + (size_t)tok * H : nullptr, ly.in_norm, H, P.eps,
                                     stage, ys, (L == 0 && blk == 0) ? P.X : nullptr);
    if (P.layer_out && L > 0 && blk == 0)
      for (int j = threadIdx.x; j < H; j += 256) P.layer_out[(size_t)(L - 1) * H + j] = __ldcg(P.X + j);
    if (ly.type == 0) {
      // in_proj qkv (+conv+SiLU), z, b (sigmoid), a (decay)
      prefetch_gemv(&ly.m[4], 1, P.nV * 128, blk, nblk);  // out_proj rows for two stages ahead
      stage_stamp(gs);  // norm + quant done
      gemv_stage(&ly.m[0], 4, H, act, smats, bs, blk, nblk);
      stage_stamp(gs);  // this block's rows done
      if (grid_barrier(gs)) return;
      DeltaNetStepArgs da{P.O, P.Mx, ly.S, P.Bt, P.Gt, P.nK, P.nV};
      deltanet_step_body(da, blk, nblk);
      if (grid_barrier(gs)) return;
      act = gated_norm_stage(P.O, P.Z, ly.lin_norm, P.nV, P.eps, stage, ys);
      gemv_stage(&ly.m[4], 1, P.nV * 128, act, smats, bs, blk, nblk);
    } else {
      prefetch_gemv(&ly.m[4], 1, P.nQ * 256, blk, nblk);
      gemv_stage(&ly.m[0], 3, H, act, smats, bs, blk, nblk);
      if (grid_barrier(gs)) return;
      AttnPrepArgs pa{P.Q16, P.K16, P.V16, ly.q_norm, ly.k_norm, P.Cos, P.Sin, P.ctrl, P.Qn,
                      ly.Kc, ly.Vc, ly.Ks, ly.Vs, P.nQ, P.nKV, P.rot, P.max_ctx, P.eps};
      attn_prep_body(pa, blk, nblk);
      if (grid_barrier(gs)) return;
      AttnSplitArgs sa{P.Qn, ly.Kc, ly.Vc, ly.Ks, ly.Vs, P.ctrl, P.Pm, P.Pse, P.Pacc,
                       P.nQ, P.nKV, P.max_ctx, P.max_chunks};
      attn_split_dispatch(sa, blk, nblk);
      if (grid_barrier(gs)) return;
      AttnCombineArgs ca{P.Pm, P.Pse, P.Pacc, P.Q16, P.ctrl, P.Q8, P.SQ, nullptr, P.nQ, P.max_ctx, P.max_chunks};
      attn_combine_body(ca, blk, nblk);
      if (grid_barrier(gs)) return;
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
    if (grid_barrier(gs)) return;
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
    if (grid_barrier(gs)) return;
    if (threadIdx.x < 32) {
      router_select(P.RLogits, P.E, P.topk, ly.shared_gate != nullptr, ys, s_sel_idx, s_sel_w, &s_gap);
    }
    __syncthreads();
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
      gateup_block_dispatch(ga, act, bs, blk, nblk);
      stage_stamp(gs);
      prefetch_down(ly.experts, s_sel_idx, P.slots, P.I, H, blk, nblk);
    }
    if (grid_barrier(gs)) return;
    {
      __syncthreads();
      StagedAct4 dact = stage4_from_f32<true>(stage, P.Act, P.I, P.slots, P.I);
      stage_stamp(gs);
      ExpertDownCombineArgs xa{ly.experts, s_sel_idx, s_sel_w, P.Act, P.Tmp, P.X, nullptr, P.slots, P.I, H};
      down_block_dispatch(xa, dact, bs, blk, nblk);
      stage_stamp(gs);
    }
    if (grid_barrier(gs)) return;
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
  {
    StagedAct4 act = norm_quant_stage(P.X, nullptr, P.final_norm, H, P.eps, stage, ys, nullptr);
    gemv_stage(&P.lm_head, 1, H, act, smats, bs, blk, nblk);
  }
  if (grid_barrier(gs)) return;
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
  if (grid_barrier(gs)) return;
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
