// Block-executor and token loop of the decode runtime.
//
// Structure kept from the reference (tools/decode/decode_l0.cpp:270-295
// singleton scratch buffers reused by every layer, :553-677 one recorded list
// per layer from two templates, :679-699 tail list, :742-825 token loop whose
// only per-token mutation is the 16-byte control block). What changes: a layer
// is 9-10 fused launches instead of 24-28, the whole token can be recorded as
// one list, and the control block is advanced on the device so consecutive
// greedy tokens replay with no host round trip.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "../common/tables.h"
#include "model.h"

namespace ainfer {

enum SessionFlags {
  SESSION_DIAG = 1,             // keep per-layer residual stream, routed experts, near-tie gaps
  SESSION_PER_LAYER_LISTS = 2,  // one list per layer + embed + tail, executed and fenced one by one
  SESSION_MULTI_KERNEL = 4,     // one list per token of ~450 stand-alone launches (the default; flag kept for callers)
  SESSION_STAGE_CLOCK = 8,      // persistent step (implies it): keep a device timestamp after every grid barrier
  SESSION_PERSISTENT = 16       // one persistent cooperative launch per token (DecodeStep)
};

struct Prefill;

struct Session {
  DeviceModel *m = nullptr;
  ainfer_device_t dev = nullptr;
  int max_ctx = 0;
  int flags = 0;
  int sm_count = 0;
  std::string err;

  // persistent state (decode_l0.cpp:286-289): conv history, DeltaNet state, KV cache
  float *conv = nullptr;        // [n_lin][conv_dim][3]
  float *S = nullptr;           // [n_lin][nV][128][128]
  int8_t *Kc = nullptr, *Vc = nullptr;      // [n_attn(+mtp)][max_ctx][nKV][256]
  uint16_t *Ks = nullptr, *Vs = nullptr;    // [n_attn(+mtp)][max_ctx][nKV] fp16 scales
  // control + token plumbing
  int32_t *ctrl = nullptr;      // device control block
  int32_t *ids = nullptr;       // device prompt ids, indexed by absolute position
  int32_t *history = nullptr;   // device ring of selected tokens, indexed by position
  int32_t *out_tok = nullptr;   // device [1]
  int32_t *host_tok = nullptr;  // pinned [max_ctx]
  // scratch (singletons)
  float *X = nullptr, *Tmp = nullptr, *Hn = nullptr, *Mix = nullptr;
  int8_t *Q8 = nullptr; float *SQ = nullptr;
  float *Mx = nullptr, *Z = nullptr, *Bt = nullptr, *Gt = nullptr, *O = nullptr;
  float *Q16 = nullptr, *K16 = nullptr, *V16 = nullptr, *Qn = nullptr;
  float *Pm = nullptr, *Pse = nullptr, *Pacc = nullptr;
  float *RLogits = nullptr; uint32_t *Counter = nullptr; ExpertW *SelRows = nullptr; int32_t *SelIdx = nullptr;
  float *SelW = nullptr, *NearGap = nullptr, *Act = nullptr;
  float *Logits = nullptr, *PV = nullptr; int32_t *PI = nullptr;
  // MTP head (only when the model has one): its residual stream, chained hidden input,
  // [embedding ; hidden] vector, logits, control block and draft token
  float *Xm = nullptr, *Hm = nullptr, *Cat = nullptr, *LogitsM = nullptr;
  int32_t *ctrl_m = nullptr, *out_tok_m = nullptr;
  ainfer_list_t mtp_list = nullptr;
  // diagnostics
  float *layer_out = nullptr;   // [layers][H]
  int32_t *routed = nullptr;    // [layers][top_k+1]
  float *near_gap = nullptr;    // [layers]
  // matrix tables
  void *gemv_tables = nullptr;
  std::vector<unsigned char> gemv_tables_host;
  size_t gemv_tables_cap = 0;
  // recorded lists
  ainfer_list_t gen_list = nullptr;    // embed + layers + tail (argmax advances the control block)
  ainfer_list_t body_list = nullptr;   // embed + layers + ControlAdvance (prompt steps)
  std::vector<ainfer_list_t> layer_lists;  // per-layer mode
  ainfer_list_t embed_list = nullptr, tail_list = nullptr, advance_list = nullptr;
  // persistent-kernel path: device plan, barrier counter, sticky error word
  void *step_plan = nullptr, *step_layers = nullptr;
  uint32_t *bar_count = nullptr;
  int32_t *step_error = nullptr;
  bool persistent = false;
  unsigned long long *stage_stamps = nullptr;  // [stage_stamp_cap] of the last launch
  int stage_stamp_cap = 0;
  std::map<std::string, ainfer_kernel_t> kernels;
  std::vector<void *> owned;
  uint64_t launches_per_token = 0;
  // AINFER_PROFILE: host wall time per list class (control, embed, linear_layer,
  // attn_layer, tail, readback), as tools/decode/decode_l0.cpp:705-725
  bool profile = false;
  std::map<std::string, std::vector<double>> buckets;
  int max_chunks = 0;
  int argmax_parts = 0;
  Prefill *prefill = nullptr;   // created on the first ainfer_session_prefill
  // expert parallelism of the prefill's MoE block (ainfer_session_prefill_ep): world 1 = none
  int pf_rank = 0, pf_world = 1, pf_rows = 0;   // pf_rows: rows per pass (0: the default)
  unsigned char pf_id[128] = {0};
  // device sampler scratch (created on first use): probabilities, marks, seen ids, {rng state, token}
  double *samp_work = nullptr; unsigned char *samp_mark = nullptr; int32_t *samp_seen = nullptr; uint64_t *samp_io = nullptr;
  Prefill *verifier = nullptr;  // rows of the MTP loop's batched verification (created on first use)
};

int session_create(DeviceModel *m, int max_ctx, int flags, Session **out, std::string &err);
// Chunked prefill (prefill.cpp): advances the session's state over n tokens at positions start_pos..
// without producing logits; bit-identical to n decode steps. The object holds the row buffers.
struct Prefill;
// rows_cap: rows per pass (1..64); verify: also allocate what per-row predictions and rollback need.
// ep_world > 1: the MoE block of every pass runs expert-parallel over that many ranks (id128: the NCCL
// id shared by the ranks); every rank then has to run the same passes (prompts of one length).
int prefill_create(Session *s, int rows_cap, bool verify, Prefill **out, int ep_rank = 0, int ep_world = 1,
                   const void *id128 = nullptr);
void prefill_destroy(Prefill *p);
int prefill_run(Prefill *p, const int *tokens, int n, int start_pos, int *predictions);
int prefill_rollback(Prefill *p, int keep);
int prefill_row_hidden(Prefill *p, int row, float *dst);
int prefill_rows_cap(const Prefill *p);
void session_destroy(Session *s);
// Zeroes conv history, DeltaNet state and the KV cache.
int session_reset(Session *s);
// One token: control = {token, pos, pos+1, -1}, replay, read the selected
// token back (4 bytes). Returns 0 or a reference exit code (3 = context overflow).
int session_step(Session *s, int token, int pos, int *out_token);
// Samples from the last step's logits on the device (kernel SampleToken); reads back the token and
// the advanced xorshift64* state.
int session_sample(Session *s, float temp, int top_k, float top_p, float rep_penalty, const int *seen, int nseen,
                   uint64_t *rng, int *out_token);
// Greedy loop: P prompt ids starting at start_pos (no logits until the last
// prompt token, decode_l0.cpp:771), then G generated tokens; control advances
// on the device, tokens are read back once at the end. elapsed_ms (optional)
// receives the device time of the G generation steps.
// One draft of the MTP head: input token `next_token` at position `pos`, hidden input taken
// from the trunk's final residual of the last step (from_trunk != 0) or chained from the
// previous draft. Fails with code 2 when the model has no MTP head.
int session_mtp_draft(Session *s, int next_token, int pos, int from_trunk, int *draft_token);
// Greedy generation with `draft_k` MTP drafts per round, verified one by one by trunk steps
// (acceptance is draft == trunk argmax, tools/t72/mtp_accept.py:142-151). The emitted tokens
// are exactly session_generate's. stats = {rounds, drafted, accepted}.
int session_generate_mtp(Session *s, const int *prompt, int P, int G, int start_pos, int draft_k,
                         int *out_tokens, int *stats);
int session_generate(Session *s, const int *prompt, int P, int G, int start_pos, int *out_tokens,
                     float *gen_elapsed_ms);

}  // namespace ainfer
