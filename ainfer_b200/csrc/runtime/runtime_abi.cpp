// extern "C" face of the decode runtime (include/ainfer_runtime.h).
#include <cstring>
#include <string>

#include "../../../include/ainfer_runtime.h"
#include "batch.h"
#include "ep.h"
#include "executor.h"
#include "host_sampler.h"
#include "model.h"

using namespace ainfer;

struct ainfer_model_s { DeviceModel *m; std::string cfg_json; };
struct ainfer_session_s { Session *s; };
struct ainfer_ep_s { EpMoe e; };
struct ainfer_batch_s { BatchDecode b; };

static thread_local std::string g_err;
static int set_err(int code, const std::string &e) {
  if (code) g_err = e;
  return code;
}

extern "C" {

const char *ainfer_rt_last_error(void) { return g_err.c_str(); }

int ainfer_binfer_validate(const char *path, int level) {
  Container c;
  std::string err;
  int r = container_open(path, level, c, err);
  if (r == 0) {
    ModelConfig cfg;
    if (!c.arch_json.empty() && c.arch_json.find("\"text_layers\"") != std::string::npos) {
      if (!ModelConfig::from_json(c.arch_json, cfg, err)) r = 2;
      else r = check_directory_shapes(c, cfg, err);
    }
  }
  return set_err(r, err);
}

int ainfer_synth_write(const char *path, const char *preset, uint64_t seed) {
  ModelConfig cfg;
  if (!preset || !preset_config(preset, cfg)) return set_err(2, std::string("unknown synthetic preset: ") + (preset ? preset : "(null)"));
  std::string err;
  int r = synth_write_file(path, cfg, seed, err);
  return set_err(r, err);
}

int ainfer_binfer_from_safetensors(const char *src, const char *arch_json, const char *out_path) {
  std::string err;
  int r = binfer_from_safetensors(src, arch_json, out_path, err);
  return set_err(r, err);
}

const char *ainfer_preset_config_json(const char *preset) {
  static thread_local std::string js;
  ModelConfig cfg;
  if (!preset || !preset_config(preset, cfg)) return nullptr;
  js = cfg.to_json();
  return js.c_str();
}

int ainfer_model_open(ainfer_device_t dev, const char *spec, int validate_level, ainfer_model_t *out) {
  if (!dev || !spec || !out) return set_err(2, "usage: null argument");
  *out = nullptr;
  DeviceModel *m = nullptr;
  std::string err;
  int r = model_open(dev, spec, validate_level, &m, err);
  if (r) return set_err(r, err);
  ainfer_model_t h = new ainfer_model_s{m, m->cfg.to_json()};
  *out = h;
  return 0;
}
int ainfer_model_close(ainfer_model_t m) {
  if (!m) return 2;
  model_close(m->m);
  delete m;
  return 0;
}
const char *ainfer_model_config_json(ainfer_model_t m) { return m ? m->cfg_json.c_str() : nullptr; }
int ainfer_model_tensor_count(ainfer_model_t m) { return m ? (int)m->m->dir.entries.size() : -1; }

static void fill_info(const DeviceModel *dm, const TensorEntry &e, ainfer_tensor_info *info) {
  std::memset(info, 0, sizeof *info);
  std::snprintf(info->name, sizeof info->name, "%s", e.name.c_str());
  info->storage = e.storage;
  info->ndim = e.ndim;
  for (int i = 0; i < 8; ++i) info->shape[i] = e.shape[i];
  DeviceTensor t = dm->tensor(e.name);
  info->data = t.data;
  info->data_bytes = e.d_bytes;
  info->scales = t.scales;
  info->scale_bytes = e.sc_bytes;
}
int ainfer_model_tensor_at(ainfer_model_t m, int index, ainfer_tensor_info *info) {
  if (!m || !info || index < 0 || index >= (int)m->m->dir.entries.size()) return set_err(2, "bad tensor index");
  fill_info(m->m, m->m->dir.entries[(size_t)index], info);
  return 0;
}
int ainfer_model_tensor(ainfer_model_t m, const char *name, ainfer_tensor_info *info) {
  if (!m || !name || !info) return set_err(2, "usage: null argument");
  const TensorEntry *e = m->m->dir.find(name);
  if (!e) return set_err(1, std::string("missing ") + name);
  fill_info(m->m, *e, info);
  return 0;
}
int ainfer_model_bytes(ainfer_model_t m, uint64_t *payload_bytes, uint64_t *scale_bytes) {
  if (!m) return 2;
  if (payload_bytes) *payload_bytes = m->m->pay_bytes;
  if (scale_bytes) *scale_bytes = m->m->sc_bytes;
  return 0;
}

int ainfer_session_create(ainfer_model_t m, int max_ctx, int flags, ainfer_session_t *out) {
  if (!m || !out) return set_err(2, "usage: null argument");
  *out = nullptr;
  Session *s = nullptr;
  std::string err;
  int r = session_create(m->m, max_ctx, flags, &s, err);
  if (r) return set_err(r, err);
  *out = new ainfer_session_s{s};
  return 0;
}
int ainfer_session_destroy(ainfer_session_t s) {
  if (!s) return 2;
  session_destroy(s->s);
  delete s;
  return 0;
}
int ainfer_session_reset(ainfer_session_t s) {
  if (!s) return 2;
  int r = session_reset(s->s);
  return set_err(r, s->s->err);
}
int ainfer_session_buffer(ainfer_session_t h, const char *which, void **dptr, uint64_t *bytes) {
  if (!h || !which || !dptr || !bytes) return set_err(2, "usage: null argument");
  Session *s = h->s;
  const ModelConfig &c = s->m->cfg;
  std::string w = which;
  size_t n_kv = (size_t)(c.n_attn() + c.mtp_layers) * s->max_ctx * c.kv_heads;
  if (w == "conv") { *dptr = s->conv; *bytes = (uint64_t)c.n_lin() * c.conv_dim() * 3 * 4; }
  else if (w == "S") { *dptr = s->S; *bytes = (uint64_t)c.n_lin() * c.lin_v_heads * 128 * 128 * 4; }
  else if (w == "Kc") { *dptr = s->Kc; *bytes = n_kv * c.head_dim; }
  else if (w == "Vc") { *dptr = s->Vc; *bytes = n_kv * c.head_dim; }
  else if (w == "Ks") { *dptr = s->Ks; *bytes = n_kv * 2; }
  else if (w == "Vs") { *dptr = s->Vs; *bytes = n_kv * 2; }
  else if (w == "logits") { *dptr = s->Logits; *bytes = (uint64_t)c.vocab * 4; }
  else if (w == "x") { *dptr = s->X; *bytes = (uint64_t)c.hidden * 4; }
  else if (w == "mtp_hidden") { *dptr = s->Hm; *bytes = s->Hm ? (uint64_t)c.hidden * 4 : 0; }
  else if (w == "ctrl") { *dptr = s->ctrl; *bytes = 16; }
  else if (w == "history") { *dptr = s->history; *bytes = (uint64_t)s->max_ctx * 4; }
  else if (w == "layer_out") { *dptr = s->layer_out; *bytes = s->layer_out ? (uint64_t)c.layers * c.hidden * 4 : 0; }
  else if (w == "routed") { *dptr = s->routed; *bytes = s->routed ? (uint64_t)c.layers * (c.top_k + 1) * 4 : 0; }
  else if (w == "stage_stamps") { *dptr = s->stage_stamps; *bytes = (uint64_t)s->stage_stamp_cap * 8; }
  else if (w == "near_gap") { *dptr = s->near_gap; *bytes = s->near_gap ? (uint64_t)c.layers * 4 : 0; }
  else return set_err(2, "unknown session buffer: " + w);
  return 0;
}
int ainfer_session_prefill(ainfer_session_t h, const int *tokens, int n, int start_pos) {
  if (!h || (!tokens && n > 0)) return set_err(2, "usage: null argument");
  Session *s = h->s;
  if (!s->prefill) {
    // rows per pass: the planner of the expert-parallel block takes 2048 (row, expert) items over all ranks
    const int topk = s->m->cfg.top_k > 0 ? s->m->cfg.top_k : 1;
    const int most = std::max(1, 2048 / (topk * s->pf_world));   // rows a rank may bring to a pass
    int rows = s->pf_rows > 0 ? s->pf_rows : std::min(192, most >= 8 ? most / 8 * 8 : most);
    rows = std::max(1, std::min(rows, most));
    int r = prefill_create(s, rows, false, &s->prefill, s->pf_rank, s->pf_world, s->pf_id);
    if (r) return set_err(r, s->err);
  }
  int r = prefill_run(s->prefill, tokens, n, start_pos, nullptr);
  return set_err(r, s->err);
}
int ainfer_session_prefill_rows(ainfer_session_t h, int rows) {
  if (!h || rows < 1) return set_err(2, "usage: a session and at least one row");
  Session *s = h->s;
  if (s->prefill) { prefill_destroy(s->prefill); s->prefill = nullptr; }
  s->pf_rows = rows;
  return 0;
}
int ainfer_session_prefill_ep(ainfer_session_t h, const void *id128, int rank, int world) {
  if (!h) return set_err(2, "usage: null argument");
  Session *s = h->s;
  if (world < 1 || world > 64 || 64 % world || rank < 0 || rank >= world || (world > 1 && !id128))
    return set_err(2, "usage: 0 <= rank < world, world divides 64, and an id for more than one rank");
  if (s->prefill) { prefill_destroy(s->prefill); s->prefill = nullptr; }
  s->pf_rank = rank; s->pf_world = world;
  if (id128) std::memcpy(s->pf_id, id128, 128);
  return 0;
}
int ainfer_session_step(ainfer_session_t s, int token, int pos, int *out_token) {
  if (!s) return 2;
  int r = session_step(s->s, token, pos, out_token);
  return set_err(r, s->s->err);
}
int ainfer_session_generate(ainfer_session_t s, const int *prompt, int P, int G, int start_pos,
                            int *out_tokens, float *gen_ms) {
  if (!s || !prompt) return set_err(2, "usage: null argument");
  int r = session_generate(s->s, prompt, P, G, start_pos, out_tokens, gen_ms);
  return set_err(r, s->s->err);
}
int ainfer_session_logits(ainfer_session_t s, float *host_out) {
  if (!s || !host_out) return 2;
  if (ainfer_memcpy_d2h(s->s->dev, host_out, s->s->Logits, (size_t)s->s->m->cfg.vocab * 4) != AINFER_OK)
    return set_err(1, ainfer_last_error(s->s->dev));
  return 0;
}
int ainfer_session_sample(ainfer_session_t h, const ainfer_sample_params *p, const int *seen, int nseen, uint64_t *rng,
                          int *out_token) {
  if (!h || !p || !rng || !out_token || (nseen > 0 && !seen)) return set_err(2, "usage: null argument");
  Session *s = h->s;
  int r = session_sample(s, p->temp, p->top_k, p->top_p, p->rep_penalty, seen, nseen, rng, out_token);
  return set_err(r, s->err);
}
int ainfer_session_mtp_draft(ainfer_session_t s, int next_token, int pos, int from_trunk, int *draft_token) {
  if (!s) return 2;
  int r = session_mtp_draft(s->s, next_token, pos, from_trunk, draft_token);
  return set_err(r, s->s->err);
}
int ainfer_session_mtp_logits(ainfer_session_t s, float *host_out) {
  if (!s || !host_out) return 2;
  if (!s->s->LogitsM) return set_err(2, "usage: the model has no MTP head");
  if (ainfer_memcpy_d2h(s->s->dev, host_out, s->s->LogitsM, (size_t)s->s->m->cfg.vocab * 4) != AINFER_OK)
    return set_err(1, ainfer_last_error(s->s->dev));
  return 0;
}
int ainfer_session_generate_mtp(ainfer_session_t s, const int *prompt, int P, int G, int start_pos, int draft_k,
                                int *out_tokens, int *stats) {
  if (!s || !prompt || !out_tokens) return set_err(2, "usage: null argument");
  int r = session_generate_mtp(s->s, prompt, P, G, start_pos, draft_k, out_tokens, stats);
  return set_err(r, s->s->err);
}
int ainfer_session_launches_per_token(ainfer_session_t s, uint64_t *launches) {
  if (!s || !launches) return 2;
  *launches = s->s->launches_per_token;
  return 0;
}

int ainfer_ep_unique_id(void *out128) {
  if (!out128) return set_err(2, "usage: null argument");
  std::string err;
  int r = ep_unique_id(out128, err);
  return set_err(r, err);
}
int ainfer_ep_create(ainfer_model_t m, const void *id128, int rank, int world, int batch, int flags, ainfer_ep_t *out) {
  if (!m || !out) return set_err(2, "usage: null argument");
  *out = nullptr;
  ainfer_ep_s *h = new ainfer_ep_s;
  int r = h->e.create(m->m, id128, rank, world, batch, flags);
  if (r) {
    set_err(r, h->e.err);
    h->e.destroy();
    delete h;
    return r;
  }
  *out = h;
  return 0;
}
int ainfer_ep_destroy(ainfer_ep_t ep) {
  if (!ep) return 2;
  ep->e.destroy();
  delete ep;
  return 0;
}
int ainfer_ep_buffer(ainfer_ep_t ep, const char *which, void **dptr, uint64_t *bytes) {
  if (!ep || !which || !dptr || !bytes) return set_err(2, "usage: null argument");
  EpMoe &e = ep->e;
  const std::string w = which;
  if (w == "res") { *dptr = e.Res; *bytes = (uint64_t)e.n * e.H * 4; }
  else if (w == "x") { *dptr = e.X; *bytes = (uint64_t)e.n * e.H * 4; }
  else if (w == "add") { *dptr = e.Add; *bytes = e.Add ? (uint64_t)e.n * e.H * 4 : 0; }
  else if (w == "sel_idx") { *dptr = e.SelIdx; *bytes = (uint64_t)e.n * (e.k + 1) * 4; }
  else if (w == "sel_w") { *dptr = e.SelW; *bytes = (uint64_t)e.n * (e.k + 1) * 4; }
  else if (w == "near_gap") { *dptr = e.NearGap; *bytes = (uint64_t)e.n * 4; }
  else if (w == "router_bias") { *dptr = e.Bias; *bytes = (uint64_t)e.E * 4; }
  else if (w == "counts") { *dptr = e.Counts; *bytes = 32; }
  else return set_err(2, "unknown buffer: " + w);
  return 0;
}
int ainfer_ep_moe_layer(ainfer_ep_t ep, int layer) {
  if (!ep) return 2;
  int r = ep->e.run_layer(layer, false, nullptr);
  return set_err(r, ep->e.err);
}
int ainfer_ep_moe_stack(ainfer_ep_t ep, int first, int count, float *seg_ms) {
  if (!ep) return 2;
  int r = ep->e.run_stack(first, count, seg_ms);
  return set_err(r, ep->e.err);
}

int ainfer_batch_create(ainfer_model_t m, const void *id128, int rank, int world, int batch, int max_ctx, int flags,
                        ainfer_batch_t *out) {
  if (!m || !out) return set_err(2, "usage: null argument");
  *out = nullptr;
  ainfer_batch_s *h = new ainfer_batch_s;
  int r = h->b.create(m->m, id128, rank, world, batch, max_ctx, flags);
  if (r) {
    set_err(r, h->b.err);
    h->b.destroy();
    delete h;
    return r;
  }
  *out = h;
  return 0;
}
int ainfer_batch_destroy(ainfer_batch_t h) {
  if (!h) return 2;
  h->b.destroy();
  delete h;
  return 0;
}
int ainfer_batch_buffer(ainfer_batch_t h, const char *which, void **dptr, uint64_t *bytes) {
  if (!h || !which || !dptr || !bytes) return set_err(2, "usage: null argument");
  BatchDecode &b = h->b;
  const ModelConfig &c = b.m->cfg;
  const std::string w = which;
  const uint64_t n = (uint64_t)b.n;
  if (w == "ctrl") { *dptr = b.Ctrl; *bytes = n * 16; }
  else if (w == "out_tok") { *dptr = b.OutT; *bytes = n * 4; }
  else if (w == "logits") { *dptr = b.Logits; *bytes = n * c.vocab * 4; }
  else if (w == "x") { *dptr = b.ep.Res; *bytes = n * c.hidden * 4; }
  else if (w == "S") { *dptr = b.S; *bytes = n * b.s_stride * 4; }
  else if (w == "conv") { *dptr = b.conv; *bytes = n * b.conv_stride * 4; }
  else if (w == "Kc") { *dptr = b.Kc; *bytes = n * b.kv_rows * c.kv_heads * c.head_dim; }
  else if (w == "Vc") { *dptr = b.Vc; *bytes = n * b.kv_rows * c.kv_heads * c.head_dim; }
  else if (w == "Ks") { *dptr = b.Ks; *bytes = n * b.kv_rows * c.kv_heads * 2; }
  else if (w == "Vs") { *dptr = b.Vs; *bytes = n * b.kv_rows * c.kv_heads * 2; }
  else if (w == "router_bias") { *dptr = b.ep.Bias; *bytes = (uint64_t)c.experts * 4; }
  else return set_err(2, "unknown buffer: " + w);
  return 0;
}
int ainfer_batch_step(ainfer_batch_t h) {
  if (!h) return 2;
  int r = h->b.step();
  return set_err(r, h->b.err);
}

int ainfer_apply_rep_penalty(float *logits, int V, const int *seen, int nseen, float penalty) {
  if (!logits || V <= 0) return 2;
  std::vector<float> l(logits, logits + V);
  apply_rep_penalty(l, seen, nseen, penalty);
  std::memcpy(logits, l.data(), (size_t)V * 4);
  return 0;
}
int ainfer_sample_token(const float *logits, int V, const ainfer_sample_params *p, uint64_t *rng,
                        float *probs_out) {
  if (!logits || !p || !rng || V <= 0) return -1;
  SampleParams sp;
  sp.temp = p->temp; sp.top_k = p->top_k; sp.top_p = p->top_p; sp.rep_penalty = p->rep_penalty; sp.seed = p->seed;
  std::vector<float> probs;
  int r = sample_token(logits, V, sp, *rng, probs_out ? &probs : nullptr);
  if (probs_out) std::memcpy(probs_out, probs.data(), (size_t)V * 4);
  return r;
}

}  // extern "C"
