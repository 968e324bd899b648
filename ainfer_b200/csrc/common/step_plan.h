// Device-resident plan of the persistent decode kernel (DecodeStep): every
// pointer and dimension one token step needs, built once by the runtime when
// the session is created. Plain C layout shared by host (g++) and device code.
#pragma once
#include <cstdint>

#include "tables.h"

namespace ainfer {

struct StepLayer {
  int32_t type;            // 0 = Gated DeltaNet, 1 = gated GQA attention
  int32_t pad0;
  const float *in_norm;    // [H]
  const float *post_norm;  // [H]
  // linear: 0 qkv (conv epilogue), 1 z, 2 b, 3 a, 4 out_proj (+residual)
  // attention: 0 q, 1 k, 2 v, 4 o_proj (+residual)
  GemvMat m[5];
  float *S;                // [nV][128][128] DeltaNet state of this layer
  const float *lin_norm;   // [128]
  const float *q_norm, *k_norm;  // [256]
  int8_t *Kc, *Vc;         // [max_ctx][nKV][256] this layer's cache
  uint16_t *Ks, *Vs;       // [max_ctx][nKV]
  const uint16_t *router;       // [E][H] bf16
  const uint16_t *shared_gate;  // [H] bf16 or null
  const ExpertW *experts;       // [E+1]
};

struct StepPlan {
  int32_t H, layers, vocab;
  int32_t nQ, nKV, rot;
  int32_t nK, nV;
  int32_t E, topk, slots, I;
  int32_t max_ctx, max_chunks;
  int32_t history_cap, argmax_parts;
  float eps;
  int32_t pad0;
  const StepLayer *L;
  const uint16_t *emb;      // [vocab][H] bf16
  const float *final_norm;  // [H]
  GemvMat lm_head;          // Y = logits
  const float *Cos, *Sin;   // [max_ctx][rot]
  // scratch shared by all layers
  float *X, *Tmp, *Mx, *Z, *Bt, *Gt, *O;
  float *Q16, *K16, *V16, *Qn, *Pm, *Pse, *Pacc;
  float *RLogits, *Act, *Logits, *PV;
  int32_t *PI;
  int8_t *Q8;
  float *SQ;
  int32_t *SelIdx;          // [topk+1] copy of the last layer's routing (diagnostics)
  float *SelW, *NearGap;
  int32_t *ctrl, *history, *out_tok;
  const int32_t *ids;       // prompt ids by absolute position
  // diagnostics (null when off)
  float *layer_out;         // [layers][H]
  int32_t *routed;          // [layers][topk+1]
  float *near_gap;          // [layers]
  // optional stage clock (null when off): block 0 stores %globaltimer (ns) after every
  // grid barrier, in order, up to stage_stamp_cap entries per launch
  unsigned long long *stage_stamps;
  int32_t stage_stamp_cap;
  int32_t pad1;
  // grid barrier state: count is zeroed before every launch; error is sticky
  uint32_t *bar_count;
  int32_t *error;           // 0 ok, otherwise the code of the bounded wait that ran out
  int64_t pad2;             // size a multiple of 16 bytes: the kernel copies the plan as 16-byte words
};
static_assert(sizeof(StepPlan) % 16 == 0, "StepPlan is copied 16 bytes at a time");

}  // namespace ainfer
