#include "executor.h"

#include <time.h>

#include <algorithm>
#include <cstring>

#include "../common/step_plan.h"
#include "../common/tables.h"

namespace ainfer {

namespace {

// ---- recording helpers ----------------------------------------------------
struct Recorder {
  Session *s;
  ainfer_list_t list;
  int status = 0;
  // Residual stream and control block the recorded layer works on: the trunk's by default,
  // the MTP head's own when its list is recorded.
  float *x_override = nullptr;
  int32_t *ctrl_override = nullptr;
  float *X() const { return x_override ? x_override : s->X; }
  int32_t *ctrl() const { return ctrl_override ? ctrl_override : s->ctrl; }

  ainfer_kernel_t kernel(const char *name) {
    auto it = s->kernels.find(name);
    if (it != s->kernels.end()) return it->second;
    ainfer_kernel_t k = nullptr;
    if (ainfer_kernel_get(s->dev, name, &k) != AINFER_OK) {
      s->err = std::string("entry ") + name + " not found";
      status = 1;
      return nullptr;
    }
    s->kernels[name] = k;
    return k;
  }
  template <typename T>
  void set(ainfer_kernel_t k, uint32_t &idx, const T &v) {
    if (status) return;
    if (ainfer_kernel_set_arg(k, idx, sizeof(T), &v) != AINFER_OK) {
      s->err = ainfer_last_error(s->dev);
      status = 1;
    }
    ++idx;
  }
  // Appends one launch; arguments are set by index in the order given, which is
  // the member order of the kernel's argument struct.
  template <typename... A>
  void launch(const char *name, uint32_t groups, const A &...args) {
    if (status) return;
    ainfer_kernel_t k = kernel(name);
    if (!k) return;
    uint32_t idx = 0;
    (set(k, idx, args), ...);
    if (status) return;
    if (ainfer_list_append_launch(list, k, groups ? groups : 1) != AINFER_OK) {
      s->err = std::string("append failed: ") + ainfer_last_error(s->dev);
      status = 1;
    }
    s->launches_per_token += 1;
  }
  void copy(void *dst, const void *src, size_t bytes) {
    if (status) return;
    if (ainfer_list_append_memcpy(list, dst, src, bytes) != AINFER_OK) {
      s->err = std::string("append failed: ") + ainfer_last_error(s->dev);
      status = 1;
    }
  }
};

// Thread groups for a weight-streaming launch: a group should own at least one
// whole 16 KB tile (32768/K rows) and there is no point in more than two groups
// per SM (that many are resident; each pays its own start-up).
int stream_groups(long weight_rows, int K, int sm_count) {
  const long rpt = 32768 / K;
  long g = (weight_rows + rpt - 1) / rpt;
  return (int)std::max<long>(1, std::min<long>(g, 2L * sm_count));
}

struct MatSpec {
  DeviceTensor t;
  float *Y;
  int epi;
  const float *e0;
  float *e1;
  const float *e2;
};

// Adds a matrix table for one GEMV launch to the session's table arena and
// appends the launch.
void record_gemv(Recorder &r, const std::vector<MatSpec> &mats, int K, const int8_t *XQ,
                 const float *SQ) {
  Session *s = r.s;
  if (r.status) return;
  std::vector<GemvMat> tab(mats.size());
  int row = 0;
  for (size_t i = 0; i < mats.size(); ++i) {
    const MatSpec &m = mats[i];
    if (!m.t.entry) { s->err = "missing tensor for GEMV"; r.status = 1; return; }
    if ((int)m.t.entry->shape[1] != K || m.t.entry->storage != DT_INT4_SYM_G128) {
      s->err = "unexpected shape/storage of " + m.t.entry->name;
      r.status = 2;
      return;
    }
    GemvMat &g = tab[i];
    g.P = (const uint8_t *)m.t.data;
    g.S = (const uint16_t *)m.t.scales;
    g.Y = m.Y; g.e0 = m.e0; g.e1 = m.e1; g.e2 = m.e2;
    g.row_start = row;
    g.N = (int)m.t.entry->shape[0];
    g.epi = m.epi;
    g.ldy = g.N;
    row += g.N;
  }
  size_t bytes = tab.size() * sizeof(GemvMat);
  size_t off = s->gemv_tables_host.size();
  if (off + bytes > s->gemv_tables_cap) { s->err = "internal: GEMV table arena too small"; r.status = 3; return; }
  s->gemv_tables_host.resize(off + bytes);
  std::memcpy(s->gemv_tables_host.data() + off, tab.data(), bytes);
  const GemvMat *dtab = (const GemvMat *)((char *)s->gemv_tables + off);
  uint32_t groups = (uint32_t)stream_groups(row, K, s->sm_count);
  r.launch("Int4GemvA8", groups, dtab, (int32_t)mats.size(), (int32_t)row, XQ, SQ, (int32_t)K,
           (int32_t)1);
}

template <typename T>
int salloc(Session *s, size_t count, T **out, bool zero = true) {
  void *p = nullptr;
  size_t bytes = std::max<size_t>(count * sizeof(T), 16);
  if (ainfer_mem_alloc(s->dev, bytes, 256, &p) != AINFER_OK) {
    s->err = std::string("alloc ") + std::to_string(bytes) + " failed: " + ainfer_last_error(s->dev);
    return 1;
  }
  s->owned.push_back(p);
  if (zero && ainfer_mem_fill(s->dev, p, 0, bytes) != AINFER_OK) { s->err = ainfer_last_error(s->dev); return 1; }
  *out = (T *)p;
  return 0;
}

// ---- layer templates ------------------------------------------------------
// MoE block shared by both layer kinds (replaces the dense MLP of
// tools/decode/decode_l0.cpp:664-674).
void record_moe(Recorder &r, int L, const std::string &p, const float *post_norm_w) {
  Session *s = r.s;
  const ModelConfig &c = s->m->cfg;
  const int H = c.hidden, E = c.experts, k = c.top_k, I = c.expert_inter;
  const int slots = k + (c.shared_experts ? 1 : 0);
  const float eps = (float)c.rms_eps;
  r.launch("RmsNormQuant", 1, (const float *)s->Tmp, (const float *)nullptr, (float *)nullptr,
           post_norm_w, s->Hn, s->Q8, s->SQ, (int32_t)H, eps);
  DeviceTensor router = s->m->tensor(p + "mlp.gate.weight");
  DeviceTensor sgate = s->m->tensor(p + "mlp.shared_expert_gate.weight");
  if (!router.entry || (c.shared_experts && !sgate.entry)) {
    s->err = "missing " + p + "mlp.gate.weight / shared_expert_gate.weight";
    r.status = 1;
    return;
  }
  r.launch("RouterTopK", (uint32_t)((E + 1 + 7) / 8), (const uint16_t *)router.data,
           (const uint16_t *)(c.shared_experts ? sgate.data : nullptr), (const float *)s->Hn,
           s->RLogits, s->Counter, s->SelIdx, s->SelW, s->NearGap, (int32_t)E, (int32_t)H, (int32_t)k,
           (const ExpertW *)nullptr, (ExpertW *)nullptr);
  // The expert kernels chase SelIdx through the layer's table themselves: letting the router's
  // selecting block publish the records (its Experts/SelRows arguments) was measured to cost the
  // router 0.9 us per layer and to save the expert kernels nothing, their chase being hidden
  // under their activation staging.
  const ExpertW *tab = (const ExpertW *)s->m->expert_tables + (size_t)L * (E + 1);
  uint32_t g_up = (uint32_t)stream_groups(2L * slots * I, H, s->sm_count);
  r.launch("ExpertGateUp", g_up, tab, (const int32_t *)s->SelIdx, (const int8_t *)s->Q8,
           (const float *)s->SQ, s->Act, (int32_t)slots, (int32_t)I, (int32_t)H, (int32_t)0, (int32_t)1);
  uint32_t g_dn = (uint32_t)std::min<long>(stream_groups((long)H * slots, I, s->sm_count), (H + 3) / 4);
  r.launch("ExpertDownCombine", g_dn, tab, (const int32_t *)s->SelIdx, (const float *)s->SelW,
           (const float *)s->Act, (const float *)s->Tmp, r.X(), (float *)nullptr, (int32_t)slots,
           (int32_t)I, (int32_t)H);
  if (s->flags & SESSION_DIAG) {
    if (L < c.layers) {
      r.copy(s->layer_out + (size_t)L * H, s->X, (size_t)H * 4);
      r.copy(s->routed + (size_t)L * (k + 1), s->SelIdx, (size_t)(k + 1) * 4);
      r.copy(s->near_gap + L, s->NearGap, 4);
    }
  }
}

// Gated DeltaNet layer (tools/decode/decode_l0.cpp:560-561,610-663).
void record_linear_layer(Recorder &r, int L) {
  Session *s = r.s;
  DeviceModel *m = s->m;
  const ModelConfig &c = m->cfg;
  const int H = c.hidden, nK = c.lin_k_heads, nV = c.lin_v_heads, C = c.conv_dim(), VD = c.value_dim();
  const int slot = m->slot[L];
  const std::string p = layer_prefix(L);
  const float eps = (float)c.rms_eps;
  r.launch("RmsNormQuant", 1, (const float *)s->X, (const float *)nullptr, (float *)nullptr,
           (const float *)(m->in_norm + (size_t)L * H), (float *)nullptr, s->Q8, s->SQ, (int32_t)H, eps);
  record_gemv(r,
              {{m->tensor(p + "linear_attn.in_proj_qkv.weight"), s->Mx, EPI_CONV_SILU,
                m->conv_w + (size_t)slot * C * 4, s->conv + (size_t)slot * C * 3, nullptr},
               {m->tensor(p + "linear_attn.in_proj_z.weight"), s->Z, EPI_STORE, nullptr, nullptr, nullptr},
               {m->tensor(p + "linear_attn.in_proj_b.weight"), s->Bt, EPI_BETA, nullptr, nullptr, nullptr},
               {m->tensor(p + "linear_attn.in_proj_a.weight"), s->Gt, EPI_GDECAY,
                m->a_log + (size_t)slot * nV, nullptr, m->dt_bias + (size_t)slot * nV}},
              H, s->Q8, s->SQ);
  r.launch("DeltaNetStep", (uint32_t)(nV * 4), s->O, (const float *)s->Mx,
           s->S + (size_t)slot * nV * 128 * 128, (const float *)s->Bt, (const float *)s->Gt,
           (int32_t)nK, (int32_t)nV);
  r.launch("GatedNormQuant", (uint32_t)((nV + 3) / 4), (const float *)s->O, (const float *)s->Z,
           (const float *)(m->lin_norm + (size_t)slot * c.lin_head_dim), s->Q8, s->SQ,
           (float *)nullptr, (int32_t)nV, eps);
  record_gemv(r, {{m->tensor(p + "linear_attn.out_proj.weight"), s->Tmp, EPI_RESADD, s->X, nullptr, nullptr}},
              VD, s->Q8, s->SQ);
  record_moe(r, L, p, m->post_norm + (size_t)L * H);
}

// Gated GQA attention layer (tools/decode/decode_l0.cpp:560-608,663). kv_slot
// selects the cache; in_x is the residual input (X for trunk layers).
void record_attn_layer(Recorder &r, int L, const std::string &p) {
  Session *s = r.s;
  DeviceModel *m = s->m;
  const ModelConfig &c = m->cfg;
  const int H = c.hidden, nQ = c.q_heads, nKV = c.kv_heads, D = c.head_dim;
  const int slot = m->slot[L];
  const float eps = (float)c.rms_eps;
  r.launch("RmsNormQuant", 1, (const float *)r.X(), (const float *)nullptr, (float *)nullptr,
           (const float *)(m->in_norm + (size_t)L * H), (float *)nullptr, s->Q8, s->SQ, (int32_t)H, eps);
  record_gemv(r,
              {{m->tensor(p + "self_attn.q_proj.weight"), s->Q16, EPI_STORE, nullptr, nullptr, nullptr},
               {m->tensor(p + "self_attn.k_proj.weight"), s->K16, EPI_STORE, nullptr, nullptr, nullptr},
               {m->tensor(p + "self_attn.v_proj.weight"), s->V16, EPI_STORE, nullptr, nullptr, nullptr}},
              H, s->Q8, s->SQ);
  size_t kv_off = (size_t)slot * s->max_ctx * nKV;
  int8_t *Kc = s->Kc + kv_off * D, *Vc = s->Vc + kv_off * D;
  uint16_t *Ks = s->Ks + kv_off, *Vs = s->Vs + kv_off;
  r.launch("AttnPrep", (uint32_t)((nQ + 2 * nKV + 7) / 8), (const float *)s->Q16, (const float *)s->K16,
           (const float *)s->V16, (const float *)(m->q_norm + (size_t)slot * D),
           (const float *)(m->k_norm + (size_t)slot * D), (const float *)m->rope_cos,
           (const float *)m->rope_sin, (const int32_t *)r.ctrl(), s->Qn, Kc, Vc, Ks, Vs, (int32_t)nQ,
           (int32_t)nKV, (int32_t)c.rotary_dim, (int32_t)s->max_ctx, eps);
  uint32_t g_split = (uint32_t)std::min(s->max_chunks * nKV, s->sm_count * 8);
  r.launch("AttnSplit", g_split, (const float *)s->Qn, (const int8_t *)Kc, (const int8_t *)Vc,
           (const uint16_t *)Ks, (const uint16_t *)Vs, (const int32_t *)r.ctrl(), s->Pm, s->Pse, s->Pacc,
           (int32_t)nQ, (int32_t)nKV, (int32_t)s->max_ctx, (int32_t)s->max_chunks);
  r.launch("AttnCombine", (uint32_t)nQ, (const float *)s->Pm, (const float *)s->Pse,
           (const float *)s->Pacc, (const float *)s->Q16, (const int32_t *)r.ctrl(), s->Q8, s->SQ,
           (float *)nullptr, (int32_t)nQ, (int32_t)s->max_ctx, (int32_t)s->max_chunks);
  record_gemv(r, {{m->tensor(p + "self_attn.o_proj.weight"), s->Tmp, EPI_RESADD, r.X(), nullptr, nullptr}},
              nQ * D, s->Q8, s->SQ);
  record_moe(r, L, p, m->post_norm + (size_t)L * H);
}

void record_layer(Recorder &r, int L) {
  if (r.s->m->cfg.layer_types[L] == 'A') record_attn_layer(r, L, layer_prefix(L));
  else record_linear_layer(r, L);
}

void record_embed(Recorder &r) {
  Session *s = r.s;
  DeviceTensor emb = s->m->tensor("model.language_model.embed_tokens.weight");
  if (!emb.entry) { s->err = "missing model.language_model.embed_tokens.weight"; r.status = 1; return; }
  r.launch("EmbedRow", 1, s->X, (const uint16_t *)emb.data, (const int32_t *)s->ctrl,
           (int32_t)s->m->cfg.hidden, (int32_t)s->m->cfg.vocab, (int32_t)4);
}

// Tail: final norm + lm_head + argmax (tools/decode/decode_l0.cpp:679-699).
void record_tail(Recorder &r, bool advance) {
  Session *s = r.s;
  DeviceModel *m = s->m;
  const ModelConfig &c = m->cfg;
  r.launch("RmsNormQuant", 1, (const float *)s->X, (const float *)nullptr, (float *)nullptr,
           (const float *)m->final_norm, (float *)nullptr, s->Q8, s->SQ, (int32_t)c.hidden,
           (float)c.rms_eps);
  record_gemv(r, {{m->tensor("lm_head.weight"), s->Logits, EPI_STORE, nullptr, nullptr, nullptr}},
              c.hidden, s->Q8, s->SQ);
  r.launch("ArgmaxStage1", (uint32_t)s->argmax_parts, (const float *)s->Logits, s->PV, s->PI,
           (int32_t)c.vocab);
  r.launch("ArgmaxStage2", 1, (const float *)s->PV, (const int32_t *)s->PI, s->out_tok, s->ctrl,
           s->history, (int32_t)s->argmax_parts, (int32_t)(advance ? 1 : 0), (int32_t)s->max_ctx);
}

// MTP head (tools/t72/mtp_accept.py:11-16,142-151): x = fc . quant([rms1w(embed(next)) ; rms1w(h)]),
// one full-attention decoder layer with its own KV cache and MoE, mtp.norm, shared lm_head, argmax.
// Works on its own residual buffer (Xm), control block (ctrl_m) and logits (LogitsM); the hidden
// input h is Hm, and the layer's output is copied back into Hm so that drafts can be chained.
void record_mtp(Recorder &r) {
  Session *s = r.s;
  DeviceModel *m = s->m;
  const ModelConfig &c = m->cfg;
  const int H = c.hidden, L = c.layers;
  const float eps = (float)c.rms_eps;
  DeviceTensor emb = m->tensor("model.language_model.embed_tokens.weight");
  if (!emb.entry) { s->err = "missing model.language_model.embed_tokens.weight"; r.status = 1; return; }
  r.x_override = s->Xm;
  r.ctrl_override = s->ctrl_m;
  r.launch("EmbedRow", 1, s->Xm, (const uint16_t *)emb.data, (const int32_t *)s->ctrl_m, (int32_t)H,
           (int32_t)c.vocab, (int32_t)4);
  r.launch("RmsNormQuant", 1, (const float *)s->Xm, (const float *)nullptr, (float *)nullptr,
           (const float *)m->mtp_norms, s->Cat, s->Q8, s->SQ, (int32_t)H, eps);
  r.launch("RmsNormQuant", 1, (const float *)s->Hm, (const float *)nullptr, (float *)nullptr,
           (const float *)(m->mtp_norms + H), s->Cat + H, s->Q8, s->SQ, (int32_t)H, eps);
  r.launch("QuantRows", (uint32_t)((2 * H / 128 + 7) / 8), (const float *)s->Cat, s->Q8, s->SQ,
           (int32_t)(2 * H / 128));
  record_gemv(r, {{m->tensor("mtp.fc.weight"), s->Xm, EPI_STORE, nullptr, nullptr, nullptr}}, 2 * H, s->Q8, s->SQ);
  record_attn_layer(r, L, "mtp.layers.0.");
  r.launch("RmsNormQuant", 1, (const float *)s->Xm, (const float *)nullptr, (float *)nullptr,
           (const float *)(m->mtp_norms + 2 * (size_t)H), (float *)nullptr, s->Q8, s->SQ, (int32_t)H, eps);
  record_gemv(r, {{m->tensor("lm_head.weight"), s->LogitsM, EPI_STORE, nullptr, nullptr, nullptr}}, H, s->Q8,
              s->SQ);
  r.launch("ArgmaxStage1", (uint32_t)s->argmax_parts, (const float *)s->LogitsM, s->PV, s->PI, (int32_t)c.vocab);
  // advance = 0: the draft token goes to out_tok_m only; the host owns ctrl_m
  r.launch("ArgmaxStage2", 1, (const float *)s->PV, (const int32_t *)s->PI, s->out_tok_m, s->ctrl_m,
           (int32_t *)nullptr, (int32_t)s->argmax_parts, (int32_t)0, (int32_t)s->max_ctx);
  r.copy(s->Hm, s->Xm, (size_t)H * 4);
  r.x_override = nullptr;
  r.ctrl_override = nullptr;
}

GemvMat make_mat(Session *s, int &status, const std::string &name, int K, float *Y, int epi,
                 const float *e0, float *e1, const float *e2) {
  GemvMat g;
  std::memset(&g, 0, sizeof g);
  DeviceTensor t = s->m->tensor(name);
  if (!t.entry) { s->err = "missing " + name; status = 1; return g; }
  if ((int)t.entry->shape[1] != K || t.entry->storage != DT_INT4_SYM_G128) {
    s->err = "unexpected shape/storage of " + name;
    status = 2;
    return g;
  }
  g.P = (const uint8_t *)t.data;
  g.S = (const uint16_t *)t.scales;
  g.Y = Y; g.e0 = e0; g.e1 = e1; g.e2 = e2;
  g.N = (int)t.entry->shape[0];
  g.epi = epi;
  g.ldy = g.N;
  return g;
}

// Builds the device plan of the persistent decode kernel (DecodeStep, one block per SM) and
// records the two one-launch lists (token step with tail, prompt step). Fails with a message
// when a stage's share per block would not fit the kernel's shared-memory scratch.
int build_step(Session *s) {
  DeviceModel *m = s->m;
  const ModelConfig &c = m->cfg;
  const int H = c.hidden, D = c.head_dim, nQ = c.q_heads, nKV = c.kv_heads, nV = c.lin_v_heads;
  const int C = c.conv_dim(), VD = c.value_dim(), E = c.experts;
  int status = 0;
  std::vector<StepLayer> layers((size_t)c.layers);
  for (int L = 0; L < c.layers && !status; ++L) {
    StepLayer &ly = layers[(size_t)L];
    std::memset(&ly, 0, sizeof ly);
    const std::string p = layer_prefix(L);
    const int slot = m->slot[L];
    ly.in_norm = m->in_norm + (size_t)L * H;
    ly.post_norm = m->post_norm + (size_t)L * H;
    if (c.layer_types[L] == 'A') {
      ly.type = 1;
      ly.m[0] = make_mat(s, status, p + "self_attn.q_proj.weight", H, s->Q16, EPI_STORE, nullptr, nullptr, nullptr);
      ly.m[1] = make_mat(s, status, p + "self_attn.k_proj.weight", H, s->K16, EPI_STORE, nullptr, nullptr, nullptr);
      ly.m[2] = make_mat(s, status, p + "self_attn.v_proj.weight", H, s->V16, EPI_STORE, nullptr, nullptr, nullptr);
      ly.m[4] = make_mat(s, status, p + "self_attn.o_proj.weight", nQ * D, s->Tmp, EPI_RESADD, s->X, nullptr, nullptr);
      ly.q_norm = m->q_norm + (size_t)slot * D;
      ly.k_norm = m->k_norm + (size_t)slot * D;
      size_t kv_off = (size_t)slot * s->max_ctx * nKV;
      ly.Kc = s->Kc + kv_off * D; ly.Vc = s->Vc + kv_off * D;
      ly.Ks = s->Ks + kv_off; ly.Vs = s->Vs + kv_off;
    } else {
      ly.type = 0;
      ly.m[0] = make_mat(s, status, p + "linear_attn.in_proj_qkv.weight", H, s->Mx, EPI_CONV_SILU,
                         m->conv_w + (size_t)slot * C * 4, s->conv + (size_t)slot * C * 3, nullptr);
      ly.m[1] = make_mat(s, status, p + "linear_attn.in_proj_z.weight", H, s->Z, EPI_STORE, nullptr, nullptr, nullptr);
      ly.m[2] = make_mat(s, status, p + "linear_attn.in_proj_b.weight", H, s->Bt, EPI_BETA, nullptr, nullptr, nullptr);
      ly.m[3] = make_mat(s, status, p + "linear_attn.in_proj_a.weight", H, s->Gt, EPI_GDECAY,
                         m->a_log + (size_t)slot * nV, nullptr, m->dt_bias + (size_t)slot * nV);
      ly.m[4] = make_mat(s, status, p + "linear_attn.out_proj.weight", VD, s->Tmp, EPI_RESADD, s->X, nullptr, nullptr);
      ly.S = s->S + (size_t)slot * nV * 128 * 128;
      ly.lin_norm = m->lin_norm + (size_t)slot * c.lin_head_dim;
    }
    DeviceTensor router = m->tensor(p + "mlp.gate.weight"), sg = m->tensor(p + "mlp.shared_expert_gate.weight");
    if (!router.entry || (c.shared_experts && !sg.entry)) { s->err = "missing " + p + "mlp.gate.weight"; status = 1; break; }
    ly.router = (const uint16_t *)router.data;
    ly.shared_gate = c.shared_experts ? (const uint16_t *)sg.data : nullptr;
    ly.experts = (const ExpertW *)m->expert_tables + (size_t)L * (E + 1);
  }
  if (status) return status;
  StepPlan P;
  std::memset(&P, 0, sizeof P);
  P.H = H; P.layers = c.layers; P.vocab = c.vocab;
  P.nQ = nQ; P.nKV = nKV; P.rot = c.rotary_dim; P.nK = c.lin_k_heads; P.nV = nV;
  P.E = E; P.topk = c.top_k; P.slots = c.top_k + (c.shared_experts ? 1 : 0); P.I = c.expert_inter;
  P.max_ctx = s->max_ctx; P.max_chunks = s->max_chunks; P.history_cap = s->max_ctx;
  P.argmax_parts = s->argmax_parts;
  P.eps = (float)c.rms_eps;
  DeviceTensor emb = m->tensor("model.language_model.embed_tokens.weight");
  if (!emb.entry) { s->err = "missing model.language_model.embed_tokens.weight"; return 1; }
  P.emb = (const uint16_t *)emb.data;
  P.final_norm = m->final_norm;
  P.lm_head = make_mat(s, status, "lm_head.weight", H, s->Logits, EPI_STORE, nullptr, nullptr, nullptr);
  if (status) return status;
  P.Cos = m->rope_cos; P.Sin = m->rope_sin;
  P.X = s->X; P.Tmp = s->Tmp; P.Mx = s->Mx; P.Z = s->Z; P.Bt = s->Bt; P.Gt = s->Gt; P.O = s->O;
  P.Q16 = s->Q16; P.K16 = s->K16; P.V16 = s->V16; P.Qn = s->Qn; P.Pm = s->Pm; P.Pse = s->Pse; P.Pacc = s->Pacc;
  P.RLogits = s->RLogits; P.Act = s->Act; P.Logits = s->Logits; P.PV = s->PV; P.PI = s->PI;
  P.Q8 = s->Q8; P.SQ = s->SQ; P.SelIdx = s->SelIdx; P.SelW = s->SelW; P.NearGap = s->NearGap;
  P.ctrl = s->ctrl; P.history = s->history; P.out_tok = s->out_tok; P.ids = s->ids;
  P.layer_out = s->layer_out; P.routed = s->routed; P.near_gap = s->near_gap;
  if (salloc(s, 1, &s->bar_count) || salloc(s, 1, &s->step_error)) return 1;
  if (s->flags & SESSION_STAGE_CLOCK) {
    s->stage_stamp_cap = 2 * (c.layers * 64 + 64);  // first half: barrier clock, second half: fine clock
    if (salloc(s, (size_t)s->stage_stamp_cap, &s->stage_stamps)) return 1;
    P.stage_stamps = s->stage_stamps;
    P.stage_stamp_cap = s->stage_stamp_cap;
  }
  P.bar_count = s->bar_count; P.error = s->step_error;
  StepLayer *dl = nullptr;
  if (salloc(s, layers.size(), &dl, false)) return 1;
  s->step_layers = dl;
  P.L = dl;
  StepPlan *dp = nullptr;
  if (salloc(s, 1, &dp, false)) return 1;
  s->step_plan = dp;
  if (ainfer_memcpy_h2d(s->dev, dl, layers.data(), layers.size() * sizeof(StepLayer)) != AINFER_OK ||
      ainfer_memcpy_h2d(s->dev, dp, &P, sizeof P) != AINFER_OK) {
    s->err = ainfer_last_error(s->dev);
    return 1;
  }
  ainfer_kernel_t k = nullptr;
  if (ainfer_kernel_get(s->dev, "DecodeStep", &k) != AINFER_OK) { s->err = "entry DecodeStep not found"; return 1; }
  s->kernels["DecodeStep"] = k;
  const StepPlan *cdp = dp;
  int32_t mode = 1;
  ainfer_kernel_set_arg(k, 0, sizeof cdp, &cdp);
  ainfer_kernel_set_arg(k, 1, sizeof mode, &mode);
  uint32_t groups = 0;
  if (ainfer_kernel_max_groups(k, &groups) != AINFER_OK || groups == 0) {
    s->err = std::string("DecodeStep cannot be made resident: ") + ainfer_last_error(s->dev);
    return 1;
  }
  groups = std::min<uint32_t>(groups, (uint32_t)s->sm_count);
  if ((int)groups > s->argmax_parts) { s->err = "internal: argmax partial buffers too small"; return 3; }
  {
    // what one block must hold per stage: (rows x K/128) group terms <= 4096, staged activations
    // <= 8192 bytes, fp32 scratch <= 8192 values
    const long nb = groups;
    auto share = [&](long total, long unit) { return ((total / unit + nb - 1) / nb + 1) * unit; };
    auto unit = [](int K) { int G = K / 128; return G >= 8 ? 1 : 8 / G; };
    const int slots = P.slots;
    const long in_rows = (c.n_lin() ? C + VD + 2L * nV : 0), qkv_rows = (long)nQ * 2 * D + 2L * nKV * D;
    bool ok = share(std::max(in_rows, qkv_rows), unit(H)) * (H / 128) <= 4096;
    ok = ok && share(H, unit(std::max(VD, nQ * D))) * (std::max(VD, nQ * D) / 128) <= 4096;
    ok = ok && 2 * share((long)slots * P.I, unit(H)) * (H / 128) <= 4096;
    ok = ok && slots * share(H, unit(P.I)) * (P.I / 128) <= 4096;
    ok = ok && (long)slots * P.I <= 8192 && std::max(VD, nQ * D) <= 4096 && H <= 4096 && slots <= 12 && E + 1 <= 8192;
    ok = ok && (c.n_attn() == 0 || nQ / nKV <= 8);
    if (!ok) {
      s->err = "usage: this model's shapes do not fit the persistent decode kernel on " + std::to_string(groups) +
               " blocks; use the recorded list";
      return 2;
    }
  }
  for (int md = 1; md >= 0; --md) {
    ainfer_list_t *l = md ? &s->gen_list : &s->body_list;
    if (ainfer_list_create(s->dev, l) != AINFER_OK) { s->err = "list create failed"; return 1; }
    mode = md;
    ainfer_kernel_set_arg(k, 1, sizeof mode, &mode);
    if (ainfer_list_append_fill(*l, s->bar_count, 0, 4) != AINFER_OK ||
        ainfer_list_append_launch(*l, k, groups) != AINFER_OK || ainfer_list_close(*l) != AINFER_OK) {
      s->err = std::string("recording the persistent step failed: ") + ainfer_last_error(s->dev);
      return 1;
    }
  }
  s->launches_per_token = 1;
  s->persistent = true;
  return 0;
}

int close_list(Session *s, ainfer_list_t l) {
  if (ainfer_list_close(l) != AINFER_OK) { s->err = std::string("list close failed: ") + ainfer_last_error(s->dev); return 1; }
  return 0;
}

}  // namespace

int session_reset(Session *s) {
  const ModelConfig &c = s->m->cfg;
  size_t n_kv = (size_t)(c.n_attn() + c.mtp_layers) * s->max_ctx * c.kv_heads;
  int r = 0;
  r |= ainfer_mem_fill(s->dev, s->conv, 0, std::max<size_t>((size_t)c.n_lin() * c.conv_dim() * 3 * 4, 16));
  r |= ainfer_mem_fill(s->dev, s->S, 0, std::max<size_t>((size_t)c.n_lin() * c.lin_v_heads * 128 * 128 * 4, 16));
  r |= ainfer_mem_fill(s->dev, s->Kc, 0, std::max<size_t>(n_kv * c.head_dim, 16));
  r |= ainfer_mem_fill(s->dev, s->Vc, 0, std::max<size_t>(n_kv * c.head_dim, 16));
  r |= ainfer_mem_fill(s->dev, s->Ks, 0, std::max<size_t>(n_kv * 2, 16));
  r |= ainfer_mem_fill(s->dev, s->Vs, 0, std::max<size_t>(n_kv * 2, 16));
  if (r) { s->err = ainfer_last_error(s->dev); return 1; }
  return 0;
}

int session_create(DeviceModel *m, int max_ctx, int flags, Session **out, std::string &err) {
  *out = nullptr;
  if (max_ctx < 1) { err = "max_ctx must be positive"; return 2; }
  Session *s = new Session;
  s->m = m;
  s->dev = m->dev;
  s->max_ctx = max_ctx;
  s->flags = flags;
  auto fail = [&](int code) { err = s->err; session_destroy(s); return code; };
  ainfer_device_info info;
  if (ainfer_device_get_info(s->dev, &info) != AINFER_OK) { s->err = ainfer_last_error(s->dev); return fail(1); }
  s->sm_count = info.sm_count;
  const ModelConfig &c = m->cfg;
  const int H = c.hidden, D = c.head_dim, nQ = c.q_heads, nKV = c.kv_heads, nV = c.lin_v_heads;
  const int C = std::max(c.conv_dim(), 1), VD = std::max(c.value_dim(), 1);
  const int n_kv_layers = c.n_attn() + c.mtp_layers;
  s->max_chunks = (max_ctx + 63) / 64;
  s->argmax_parts = s->sm_count * 2;  // also the partial count of the persistent kernel (one per block)
  if (model_ensure_rope(m, max_ctx, s->err)) return fail(1);
  int r = 0;
  size_t n_kv = (size_t)n_kv_layers * max_ctx * nKV;
  r |= salloc(s, (size_t)c.n_lin() * C * 3, &s->conv);
  r |= salloc(s, (size_t)c.n_lin() * nV * 128 * 128, &s->S);
  r |= salloc(s, n_kv * D, &s->Kc);
  r |= salloc(s, n_kv * D, &s->Vc);
  r |= salloc(s, n_kv, &s->Ks);
  r |= salloc(s, n_kv, &s->Vs);
  r |= salloc(s, 4, &s->ctrl);
  r |= salloc(s, (size_t)max_ctx, &s->ids);
  r |= salloc(s, (size_t)max_ctx, &s->history);
  r |= salloc(s, 1, &s->out_tok);
  r |= salloc(s, (size_t)H, &s->X);
  r |= salloc(s, (size_t)H, &s->Tmp);
  r |= salloc(s, (size_t)H, &s->Hn);
  r |= salloc(s, (size_t)H, &s->Mix);
  int maxK = std::max(std::max(2 * H, VD), nQ * D);
  r |= salloc(s, (size_t)maxK, &s->Q8);
  r |= salloc(s, (size_t)maxK / 128, &s->SQ);
  r |= salloc(s, (size_t)C, &s->Mx);
  r |= salloc(s, (size_t)VD, &s->Z);
  r |= salloc(s, (size_t)std::max(nV, 1), &s->Bt);
  r |= salloc(s, (size_t)std::max(nV, 1), &s->Gt);
  r |= salloc(s, (size_t)VD, &s->O);
  r |= salloc(s, (size_t)nQ * 2 * D, &s->Q16);
  r |= salloc(s, (size_t)nKV * D, &s->K16);
  r |= salloc(s, (size_t)nKV * D, &s->V16);
  r |= salloc(s, (size_t)nQ * D, &s->Qn);
  r |= salloc(s, (size_t)nQ * s->max_chunks, &s->Pm);
  r |= salloc(s, (size_t)nQ * s->max_chunks, &s->Pse);
  r |= salloc(s, (size_t)nQ * s->max_chunks * D, &s->Pacc);
  r |= salloc(s, (size_t)c.experts + 1, &s->RLogits);
  r |= salloc(s, 1, &s->Counter);
  r |= salloc(s, (size_t)c.top_k + 1, &s->SelIdx);
  r |= salloc(s, (size_t)c.top_k + 1, &s->SelRows);
  r |= salloc(s, (size_t)c.top_k + 1, &s->SelW);
  r |= salloc(s, 1, &s->NearGap);
  r |= salloc(s, (size_t)(c.top_k + 1) * c.expert_inter, &s->Act);
  r |= salloc(s, (size_t)c.vocab, &s->Logits);
  if (c.mtp_layers) {
    r |= salloc(s, (size_t)H, &s->Xm);
    r |= salloc(s, (size_t)H, &s->Hm);
    r |= salloc(s, (size_t)2 * H, &s->Cat);
    r |= salloc(s, (size_t)c.vocab, &s->LogitsM);
    r |= salloc(s, 4, &s->ctrl_m);
    r |= salloc(s, 1, &s->out_tok_m);
  }
  r |= salloc(s, (size_t)s->argmax_parts, &s->PV);
  r |= salloc(s, (size_t)s->argmax_parts, &s->PI);
  if (flags & SESSION_DIAG) {
    r |= salloc(s, (size_t)c.layers * H, &s->layer_out);
    r |= salloc(s, (size_t)c.layers * (c.top_k + 1), &s->routed);
    r |= salloc(s, (size_t)c.layers, &s->near_gap);
  }
  s->gemv_tables_cap = (size_t)(c.layers + 2) * 8 * sizeof(GemvMat) * 2 + 4096;
  {
    unsigned char *p = nullptr;
    r |= salloc(s, s->gemv_tables_cap, &p);
    s->gemv_tables = p;
  }
  if (r) return fail(1);
  void *hp = nullptr;
  if (ainfer_host_alloc(s->dev, (size_t)max_ctx * 4 + 64, &hp) != AINFER_OK) { s->err = ainfer_last_error(s->dev); return fail(1); }
  s->host_tok = (int32_t *)hp;

  // ---- record ----
  Recorder rec{s, nullptr};
  auto new_list = [&](ainfer_list_t *l) {
    if (ainfer_list_create(s->dev, l) != AINFER_OK) { s->err = "list create failed"; rec.status = 1; }
    rec.list = *l;
  };
  if ((flags & (SESSION_PERSISTENT | SESSION_STAGE_CLOCK)) && !(flags & SESSION_PER_LAYER_LISTS)) {
    rec.status = build_step(s);
  } else if (flags & SESSION_PER_LAYER_LISTS) {
    new_list(&s->embed_list);
    record_embed(rec);
    if (!rec.status) rec.status = close_list(s, s->embed_list);
    for (int L = 0; L < c.layers && !rec.status; ++L) {
      ainfer_list_t l = nullptr;
      new_list(&l);
      s->layer_lists.push_back(l);
      record_layer(rec, L);
      if (!rec.status) rec.status = close_list(s, l);
    }
    if (!rec.status) {
      new_list(&s->tail_list);
      record_tail(rec, true);
      if (!rec.status) rec.status = close_list(s, s->tail_list);
    }
    if (!rec.status) {
      new_list(&s->advance_list);
      rec.launch("ControlAdvance", 1, s->ctrl, (const int32_t *)s->ids, (int32_t)max_ctx);
      if (!rec.status) rec.status = close_list(s, s->advance_list);
    }
  } else {
    new_list(&s->gen_list);
    s->launches_per_token = 0;
    record_embed(rec);
    for (int L = 0; L < c.layers && !rec.status; ++L) record_layer(rec, L);
    record_tail(rec, true);
    uint64_t per_token = s->launches_per_token;
    if (!rec.status) rec.status = close_list(s, s->gen_list);
    if (!rec.status) {
      new_list(&s->body_list);
      record_embed(rec);
      for (int L = 0; L < c.layers && !rec.status; ++L) record_layer(rec, L);
      rec.launch("ControlAdvance", 1, s->ctrl, (const int32_t *)s->ids, (int32_t)max_ctx);
      if (!rec.status) rec.status = close_list(s, s->body_list);
    }
    s->launches_per_token = per_token;
  }
  if (!rec.status && c.mtp_layers) {
    const uint64_t per_token = s->launches_per_token;
    new_list(&s->mtp_list);
    record_mtp(rec);
    if (!rec.status) rec.status = close_list(s, s->mtp_list);
    s->launches_per_token = per_token;
  }
  if (rec.status) return fail(rec.status);
  if (!s->gemv_tables_host.empty() &&
      ainfer_memcpy_h2d(s->dev, s->gemv_tables, s->gemv_tables_host.data(), s->gemv_tables_host.size()) != AINFER_OK) {
    s->err = ainfer_last_error(s->dev);
    return fail(1);
  }
  *out = s;
  return 0;
}

void session_destroy(Session *s) {
  if (s && s->prefill) { prefill_destroy(s->prefill); s->prefill = nullptr; }
  if (s && s->verifier) { prefill_destroy(s->verifier); s->verifier = nullptr; }
  if (!s) return;
  ainfer_sync(s->dev, UINT64_MAX);
  for (auto l : s->layer_lists) ainfer_list_destroy(l);
  for (ainfer_list_t l : {s->gen_list, s->body_list, s->embed_list, s->tail_list, s->advance_list, s->mtp_list})
    if (l) ainfer_list_destroy(l);
  for (auto &kv : s->kernels) ainfer_kernel_release(kv.second);
  for (void *p : s->owned) ainfer_mem_free(s->dev, p);
  if (s->host_tok) ainfer_host_free(s->dev, s->host_tok);
  delete s;
}

#define S_CHECK(expr)                                                        \
  do {                                                                       \
    if ((expr) != AINFER_OK) {                                               \
      s->err = std::string("device error: ") + ainfer_last_error(s->dev);    \
      return 1;                                                              \
    }                                                                        \
  } while (0)

// Executes one token's lists. with_tail: run final norm + lm_head + argmax
// (and advance the control block); otherwise advance to the next prompt id.
static double now_ns() {
  struct timespec t;
  clock_gettime(CLOCK_MONOTONIC, &t);
  return (double)t.tv_sec * 1e9 + (double)t.tv_nsec;
}

static int exec_fenced(Session *s, ainfer_list_t l, const char *label) {
  double t0 = s->profile ? now_ns() : 0;
  S_CHECK(ainfer_list_execute(l));
  S_CHECK(ainfer_sync(s->dev, UINT64_MAX));
  if (s->profile) s->buckets[label].push_back(now_ns() - t0);
  return 0;
}

static int run_token(Session *s, bool with_tail) {
  if (s->flags & SESSION_PER_LAYER_LISTS) {
    // the reference's execution model: execute + fence per list (decode_l0.cpp:714-721)
    int r = exec_fenced(s, s->embed_list, "embed");
    for (size_t L = 0; L < s->layer_lists.size() && !r; ++L)
      r = exec_fenced(s, s->layer_lists[L], s->m->cfg.layer_types[L] == 'A' ? "attn_layer" : "linear_layer");
    if (!r) r = exec_fenced(s, with_tail ? s->tail_list : s->advance_list, with_tail ? "tail" : "control");
    return r;
  }
  S_CHECK(ainfer_list_execute(with_tail ? s->gen_list : s->body_list));
  return 0;
}

// The persistent kernel reports a barrier that ran out of polls through a sticky
// error word instead of hanging; surface it as a device error.
static int check_step_error(Session *s) {
  if (!s->persistent) return 0;
  int32_t e = 0;
  S_CHECK(ainfer_memcpy_d2h(s->dev, &e, s->step_error, 4));
  if (e != 0) {
    s->err = "device error: a bounded wait of the persistent decode kernel ran out (status " +
             std::to_string(e) + ")";
    return 1;
  }
  return 0;
}

int session_step(Session *s, int token, int pos, int *out_token) {
  if (pos < 0 || pos >= s->max_ctx) {
    s->err = "context overflow: pos " + std::to_string(pos) + " >= MAXCTX " + std::to_string(s->max_ctx);
    return 3;
  }
  ainfer_control c{token, pos, pos + 1, -1};
  S_CHECK(ainfer_control_write(s->dev, s->ctrl, &c));
  int r = run_token(s, true);
  if (r) return r;
  S_CHECK(ainfer_memcpy_d2h(s->dev, s->host_tok, s->out_tok, 4));
  if (out_token) *out_token = s->host_tok[0];
  return check_step_error(s);
}

int session_sample(Session *s, float temp, int top_k, float top_p, float rep_penalty, const int *seen, int nseen,
                   uint64_t *rng, int *out_token) {
  const int V = s->m->cfg.vocab;
  if (nseen < 0 || nseen > s->max_ctx) { s->err = "usage: more seen ids than the context holds"; return 2; }
  if (!s->samp_work) {
    if (salloc(s, (size_t)V, &s->samp_work) || salloc(s, (size_t)V, &s->samp_mark) || salloc(s, (size_t)s->max_ctx, &s->samp_seen) ||
        salloc(s, (size_t)2, &s->samp_io))
      return 1;
  }
  if (nseen > 0) S_CHECK(ainfer_memcpy_h2d(s->dev, s->samp_seen, seen, (size_t)nseen * 4));
  S_CHECK(ainfer_memcpy_h2d(s->dev, s->samp_io, rng, 8));
  auto it = s->kernels.find("SampleToken");
  ainfer_kernel_t k = nullptr;
  if (it != s->kernels.end()) k = it->second;
  else {
    if (ainfer_kernel_get(s->dev, "SampleToken", &k) != AINFER_OK) { s->err = "entry SampleToken not found"; return 1; }
    s->kernels["SampleToken"] = k;
  }
  const float *logits = s->Logits;
  const int32_t *dseen = s->samp_seen;
  unsigned long long *drng = (unsigned long long *)s->samp_io;
  int32_t *dtok = (int32_t *)(s->samp_io + 1);
  float *probs = nullptr;
  int32_t *ctrl = nullptr;
  int32_t v = V, ns = nseen, tk = top_k;
  uint32_t i = 0;
  auto set = [&](size_t size, const void *p) { return ainfer_kernel_set_arg(k, i++, size, p); };
  S_CHECK(set(sizeof logits, &logits)); S_CHECK(set(sizeof dseen, &dseen)); S_CHECK(set(sizeof s->samp_work, &s->samp_work));
  S_CHECK(set(sizeof s->samp_mark, &s->samp_mark)); S_CHECK(set(sizeof drng, &drng)); S_CHECK(set(sizeof dtok, &dtok));
  S_CHECK(set(sizeof probs, &probs)); S_CHECK(set(sizeof ctrl, &ctrl)); S_CHECK(set(4, &v)); S_CHECK(set(4, &ns));
  S_CHECK(set(4, &temp)); S_CHECK(set(4, &tk)); S_CHECK(set(4, &top_p)); S_CHECK(set(4, &rep_penalty));
  S_CHECK(ainfer_kernel_launch(s->dev, k, 1));
  uint64_t back[2];
  S_CHECK(ainfer_memcpy_d2h(s->dev, back, s->samp_io, 16));
  *rng = back[0];
  *out_token = (int)(int32_t)(back[1] & 0xFFFFFFFFu);
  return 0;
}

int session_mtp_draft(Session *s, int next_token, int pos, int from_trunk, int *draft_token) {
  if (!s->mtp_list) { s->err = "usage: the model has no MTP head"; return 2; }
  if (pos < 0 || pos >= s->max_ctx) {
    s->err = "context overflow: pos " + std::to_string(pos) + " >= MAXCTX " + std::to_string(s->max_ctx);
    return 3;
  }
  if (from_trunk) S_CHECK(ainfer_memcpy_d2d(s->dev, s->Hm, s->X, (size_t)s->m->cfg.hidden * 4));
  ainfer_control c{next_token, pos, pos + 1, -1};
  S_CHECK(ainfer_control_write(s->dev, s->ctrl_m, &c));
  S_CHECK(ainfer_list_execute(s->mtp_list));
  S_CHECK(ainfer_memcpy_d2h(s->dev, s->host_tok, s->out_tok_m, 4));
  if (draft_token) *draft_token = s->host_tok[0];
  return 0;
}

int session_generate_mtp(Session *s, const int *prompt, int P, int G, int start_pos, int draft_k,
                         int *out_tokens, int *stats) {
  if (!s->mtp_list) { s->err = "usage: the model has no MTP head"; return 2; }
  if (P < 1 || G < 1 || draft_k < 1 || draft_k > 8) { s->err = "usage: need a prompt, G >= 1 and 1 <= draft_k <= 8"; return 2; }
  if (start_pos < 0 || start_pos + P + G - 1 + draft_k >= s->max_ctx) {
    s->err = "context overflow: pos " + std::to_string(start_pos + P + G - 1 + draft_k) + " >= MAXCTX " +
             std::to_string(s->max_ctx);
    return 3;
  }
  int rounds = 0, drafted = 0, accepted = 0;
  // The MTP layer runs causally over every position, as the reference's offline measurement does
  // (tools/t72/mtp_accept.py:142-151): after the trunk step at position q, whose successor token
  // is known (the next prompt id, or the trunk's own prediction), the head runs on
  // (token[q + 1], h[q]) and writes row q + 1 of its own KV slot. Its attention therefore always
  // sees true rows below its position; rows that chained drafts wrote speculatively are
  // rewritten by this call before any later position reads them. The head's output at the last
  // trunk position is the first draft of the next round.
  int y = -1, d = -1;
  for (int i = 0; i < P; ++i) {
    int r = session_step(s, prompt[i], start_pos + i, &y);
    if (r) return r;
    r = session_mtp_draft(s, i + 1 < P ? prompt[i + 1] : y, start_pos + i + 1, 1, &d);
    if (r) return r;
  }
  int p = start_pos + P - 1;  // position of the trunk step that produced y
  int g = 0;
  out_tokens[g++] = y;
  // Batched verification: the accepted token and the round's drafts go through the trunk as ONE
  // pass of up to draft_k + 1 rows (weights streamed once for all of them; prefill.cpp), which
  // returns every row's greedy prediction and keeps the DeltaNet state after every row. Drafts
  // are accepted while they equal the predictions; the state is rolled back to the last accepted
  // row (tools/t72/mtp_accept.py:66-94,142-159 measures exactly this acceptance, offline).
  if (s->verifier && prefill_rows_cap(s->verifier) < draft_k + 1) { prefill_destroy(s->verifier); s->verifier = nullptr; }
  if (!s->verifier) {
    int r = prefill_create(s, draft_k + 1, true, &s->verifier);
    if (r) return r;
  }
  while (g < G) {
    const int rows = std::min(draft_k + 1, G - g);   // tokens this round can emit
    int feed[9], pred[9];
    feed[0] = y;
    if (rows > 1) feed[1] = d;                       // d drafts the token after y
    for (int i = 2; i < rows; ++i) {                 // the rest chained from the head's own hidden state
      int r = session_mtp_draft(s, feed[i - 1], p + i, 0, &feed[i]);
      if (r) return r;
    }
    ++rounds;
    drafted += rows - 1;
    int r = prefill_run(s->verifier, feed, rows, p + 1, pred);
    if (r) return r;
    int j = 0;
    while (j < rows - 1 && feed[j + 1] == pred[j]) ++j;   // accepted drafts
    accepted += j;
    r = prefill_rollback(s->verifier, j + 1);
    if (r) return r;
    // the head's true rows for the accepted positions; the last one drafts the next round's first token
    for (int i = 0; i <= j; ++i) {
      r = prefill_row_hidden(s->verifier, i, s->X);
      if (r) return r;
      r = session_mtp_draft(s, pred[i], p + 2 + i, 1, &d);
      if (r) return r;
      out_tokens[g++] = pred[i];
    }
    p += j + 1;
    y = pred[j];
  }
  if (stats) { stats[0] = rounds; stats[1] = drafted; stats[2] = accepted; }
  return 0;
}

int session_generate(Session *s, const int *prompt, int P, int G, int start_pos, int *out_tokens,
                     float *gen_elapsed_ms) {
  if (P < 1 || G < 0) { s->err = "usage: need at least one prompt id"; return 2; }
  if (start_pos < 0 || start_pos + P + G - 1 > s->max_ctx) {
    s->err = "context overflow: pos " + std::to_string(start_pos + P + G - 1) + " >= MAXCTX " +
             std::to_string(s->max_ctx);
    return 3;
  }
  S_CHECK(ainfer_memcpy_h2d(s->dev, s->ids + start_pos, prompt, (size_t)P * 4));
  ainfer_control c{prompt[0], start_pos, start_pos + 1, -1};
  S_CHECK(ainfer_control_write(s->dev, s->ctrl, &c));
  for (int i = 0; i < P - 1; ++i) {
    int r = run_token(s, false);
    if (r) return r;
  }
  ainfer_event_t e0 = nullptr, e1 = nullptr;
  if (gen_elapsed_ms) {
    S_CHECK(ainfer_event_create(s->dev, &e0));
    S_CHECK(ainfer_event_create(s->dev, &e1));
    S_CHECK(ainfer_event_record(e0));
  }
  for (int g = 0; g < G; ++g) {
    int r = run_token(s, true);
    if (r) return r;
  }
  if (gen_elapsed_ms) {
    S_CHECK(ainfer_event_record(e1));
    S_CHECK(ainfer_event_elapsed_ms(e0, e1, gen_elapsed_ms));
    ainfer_event_destroy(e0);
    ainfer_event_destroy(e1);
  }
  if (G > 0) {
    // tokens were logged on the device at the position of the input that produced them
    S_CHECK(ainfer_memcpy_d2h(s->dev, s->host_tok, s->history + (start_pos + P - 1), (size_t)G * 4));
    for (int g = 0; g < G; ++g) out_tokens[g] = s->host_tok[g];
  } else {
    S_CHECK(ainfer_sync(s->dev, UINT64_MAX));
  }
  return check_step_error(s);
}

}  // namespace ainfer
