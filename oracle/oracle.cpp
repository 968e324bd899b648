// TEST INFRASTRUCTURE ONLY (see oracle_math.h). CPU oracle of the decode token
// loop: container parse, per-layer forward, token loop, and flat C entry points
// for ctypes. Restates tools/decode/decode_l0.cpp:556-699 (layer op order and
// tail), tools/cmdlist/layerlin_replay.cpp:444-536 and
// tools/cmdlist/layerattn_replay.cpp:441-527 (host layer math) of the
// reference, with the dense MLP replaced by the MoE block and the BF16 KV cache
// by the INT8 one (both have no reference counterpart: parity unpinned there).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <string>

#include "oracle_ops.h"


namespace orc {

enum Storage { ST_BF16 = 0, ST_FP16 = 1, ST_FP32 = 2, ST_INT4 = 3, ST_INT8 = 4, ST_FP8 = 5 };

struct Tensor {
  int storage = 0;
  int ndim = 0;
  uint64_t shape[8] = {0};
  const uint8_t *data = nullptr;
  const uint16_t *scales = nullptr;
  uint64_t data_bytes = 0, scale_bytes = 0;
  size_t numel() const {
    size_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= shape[i];
    return n;
  }
};

struct Cfg {
  int hidden = 0, layers = 0, vocab = 0;
  std::string layer_types;  // 'L' linear (Gated DeltaNet), 'A' full attention
  int q_heads = 0, kv_heads = 0, head_dim = 256, rotary_dim = 64;
  double rope_theta = 1e7;
  int lin_k_heads = 0, lin_v_heads = 0, lin_head_dim = 128, conv_kernel = 4;
  int experts = 0, top_k = 0, shared_experts = 1, expert_inter = 0;
  int mtp_layers = 0;
  float rms_eps = 1e-6f;
  int conv_dim() const { return (2 * lin_k_heads + lin_v_heads) * lin_head_dim; }
  int value_dim() const { return lin_v_heads * lin_head_dim; }
};

// Minimal reader for the flat JSON object of the architecture section.
static bool json_get(const std::string &js, const char *key, std::string &out) {
  std::string pat = std::string("\"") + key + "\":";
  size_t p = js.find(pat);
  if (p == std::string::npos) return false;
  p += pat.size();
  while (p < js.size() && js[p] == ' ') ++p;
  if (js[p] == '"') {
    size_t e = js.find('"', p + 1);
    out = js.substr(p + 1, e - p - 1);
  } else {
    size_t e = p;
    while (e < js.size() && js[e] != ',' && js[e] != '}') ++e;
    out = js.substr(p, e - p);
  }
  return true;
}
static long json_int(const std::string &js, const char *key, long dflt) {
  std::string v;
  return json_get(js, key, v) ? std::strtol(v.c_str(), nullptr, 10) : dflt;
}
static double json_num(const std::string &js, const char *key, double dflt) {
  std::string v;
  return json_get(js, key, v) ? std::strtod(v.c_str(), nullptr) : dflt;
}

static Cfg parse_cfg(const std::string &js) {
  Cfg c;
  c.hidden = (int)json_int(js, "hidden", 0);
  c.layers = (int)json_int(js, "text_layers", 0);
  c.vocab = (int)json_int(js, "vocab", 0);
  json_get(js, "layer_types", c.layer_types);
  c.q_heads = (int)json_int(js, "q_heads", 0);
  c.kv_heads = (int)json_int(js, "kv_heads", 0);
  c.head_dim = (int)json_int(js, "head_dim", 256);
  c.rotary_dim = (int)json_int(js, "rotary_dim", 64);
  c.rope_theta = json_num(js, "rope_theta", 1e7);
  c.lin_k_heads = (int)json_int(js, "lin_k_heads", 0);
  c.lin_v_heads = (int)json_int(js, "lin_v_heads", 0);
  c.lin_head_dim = (int)json_int(js, "lin_head_dim", 128);
  c.conv_kernel = (int)json_int(js, "conv_kernel", 4);
  c.experts = (int)json_int(js, "experts", 0);
  c.top_k = (int)json_int(js, "top_k", 0);
  c.shared_experts = (int)json_int(js, "shared_experts", 1);
  c.expert_inter = (int)json_int(js, "expert_intermediate", 0);
  c.mtp_layers = (int)json_int(js, "mtp_layers", 0);
  c.rms_eps = (float)json_num(js, "rms_eps", 1e-6);
  if (c.layer_types.empty())
    for (int l = 0; l < c.layers; ++l) c.layer_types += (l % 4 == 3) ? 'A' : 'L';
  return c;
}

static uint32_t crc32_bytes(const uint8_t *p, size_t n, uint32_t crc = 0) {
  static uint32_t table[256];
  static bool init = false;
  if (!init) {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
      table[i] = c;
    }
    init = true;
  }
  crc = ~crc;
  for (size_t i = 0; i < n; ++i) crc = table[(crc ^ p[i]) & 0xFF] ^ (crc >> 8);
  return ~crc;
}

// How a tensor of a lazily generated synthetic model is filled: N(0, std^2)
// draws from (seed, FNV-1a(name), index), or a constant when std == 0.
struct SynthRule {
  float std_ = 0.02f, constant = 0.0f;
};

struct Model {
  Cfg cfg;
  std::string arch_json;
  mutable std::map<std::string, Tensor> tensors;
  const uint8_t *map = nullptr;
  size_t map_bytes = 0;
  int fd = -1;
  // lazily generated synthetic model: values are produced on first use by the
  // oracle's own generator and quantiser, so that no product code is involved
  bool lazy = false;
  uint64_t seed = 0;
  std::map<std::string, SynthRule> rules;
  mutable std::map<std::string, std::pair<std::vector<uint8_t>, std::vector<uint16_t>>> store;
  mutable std::mutex mu;
  ~Model() {
    if (map) munmap((void *)map, map_bytes);
    if (fd >= 0) close(fd);
  }
  void materialise(const std::string &n, Tensor &t) const {
    const SynthRule &r = rules.at(n);
    uint64_t stream = fnv1a64(n.c_str());
    size_t numel = t.numel();
    auto &slot = store[n];
    if (t.storage == ST_INT4) {
      size_t ng = (numel + 127) / 128;
      slot.first.resize(ng * 64);
      slot.second.resize(ng);
      uint8_t *pk = slot.first.data();
      uint16_t *sc = slot.second.data();
      const uint64_t sd = seed;
      const float sdv = r.std_;
      parallel_for((int64_t)ng, [&](int64_t g) {
        float v[128];
        for (int j = 0; j < 128; ++j) {
          size_t i = (size_t)g * 128 + j;
          v[j] = i < numel ? sdv * normal_from_u32(draw_u32(sd, stream, i)) : 0.0f;
        }
        quantize_int4_g128(v, 128, pk + (size_t)g * 64, sc + g);
      });
      t.scales = slot.second.data();
      t.scale_bytes = ng * 2;
    } else {
      slot.first.resize(numel * 2);
      uint16_t *o = (uint16_t *)slot.first.data();
      const SynthRule rr = r;
      const uint64_t sd = seed;
      parallel_for((int64_t)numel, [&](int64_t i) {
        o[i] = f32_to_bf16(rr.std_ == 0.0f ? rr.constant
                                           : rr.std_ * normal_from_u32(draw_u32(sd, stream, (uint64_t)i)));
      });
    }
    t.data = slot.first.data();
    t.data_bytes = slot.first.size();
  }
  const Tensor &get(const std::string &n) const {
    std::lock_guard<std::mutex> lk(mu);
    auto it = tensors.find(n);
    if (it == tensors.end()) {
      std::fprintf(stderr, "oracle: missing %s\n", n.c_str());
      std::abort();
    }
    if (lazy && !it->second.data) materialise(n, it->second);
    return it->second;
  }
  bool has(const std::string &n) const { return tensors.count(n) != 0; }
};

// Tensor list of a synthetic model of the given shape (names as the container
// convention of the runtime: HF-style names under model.language_model.*, the
// shared expert abbreviated to mlp.shared.* to fit the 63-byte name field).
static void synth_plan(Model &M) {
  const Cfg &c = M.cfg;
  auto add = [&](const std::string &name, std::vector<uint64_t> shape, bool int4, SynthRule r) {
    Tensor t;
    t.storage = int4 ? ST_INT4 : ST_BF16;
    t.ndim = (int)shape.size();
    for (size_t i = 0; i < shape.size(); ++i) t.shape[i] = shape[i];
    M.tensors[name] = t;
    M.rules[name] = r;
  };
  const uint64_t H = c.hidden, V = c.vocab, I = c.expert_inter, D = c.head_dim;
  SynthRule w{0.02f, 0.0f}, zero{0.0f, 0.0f}, one{0.0f, 1.0f};
  auto layer = [&](const std::string &p, bool attn) {
    add(p + "input_layernorm.weight", {H}, false, zero);
    add(p + "post_attention_layernorm.weight", {H}, false, zero);
    if (attn) {
      add(p + "self_attn.q_proj.weight", {(uint64_t)c.q_heads * 2 * D, H}, true, w);
      add(p + "self_attn.k_proj.weight", {(uint64_t)c.kv_heads * D, H}, true, w);
      add(p + "self_attn.v_proj.weight", {(uint64_t)c.kv_heads * D, H}, true, w);
      add(p + "self_attn.o_proj.weight", {H, (uint64_t)c.q_heads * D}, true, w);
      add(p + "self_attn.q_norm.weight", {D}, false, zero);
      add(p + "self_attn.k_norm.weight", {D}, false, zero);
    } else {
      const uint64_t C = c.conv_dim(), VD = c.value_dim(), NV = c.lin_v_heads;
      add(p + "linear_attn.in_proj_qkv.weight", {C, H}, true, w);
      add(p + "linear_attn.in_proj_z.weight", {VD, H}, true, w);
      add(p + "linear_attn.in_proj_b.weight", {NV, H}, true, w);
      add(p + "linear_attn.in_proj_a.weight", {NV, H}, true, w);
      add(p + "linear_attn.conv1d.weight", {C, 1, 4}, false, SynthRule{0.5f, 0.0f});
      add(p + "linear_attn.A_log", {NV}, false, SynthRule{0.05f, 0.0f});
      add(p + "linear_attn.dt_bias", {NV}, false, SynthRule{0.05f, 0.0f});
      add(p + "linear_attn.norm.weight", {(uint64_t)c.lin_head_dim}, false, one);
      add(p + "linear_attn.out_proj.weight", {H, VD}, true, w);
    }
    add(p + "mlp.gate.weight", {(uint64_t)c.experts, H}, false, w);
    for (int e = 0; e <= c.experts; ++e) {
      if (e == c.experts && !c.shared_experts) break;
      std::string ep = e < c.experts ? p + "mlp.experts." + std::to_string(e) + "." : p + "mlp.shared.";
      add(ep + "gate_proj.weight", {I, H}, true, w);
      add(ep + "up_proj.weight", {I, H}, true, w);
      add(ep + "down_proj.weight", {H, I}, true, w);
    }
    if (c.shared_experts) add(p + "mlp.shared_expert_gate.weight", {1, H}, false, w);
  };
  add("lm_head.weight", {V, H}, true, w);
  add("model.language_model.embed_tokens.weight", {V, H}, false, w);
  for (int L = 0; L < c.layers; ++L)
    layer("model.language_model.layers." + std::to_string(L) + ".", c.layer_types[L] == 'A');
  add("model.language_model.norm.weight", {H}, false, zero);
  if (c.mtp_layers) {
    add("mtp.fc.weight", {H, 2 * H}, true, w);
    layer("mtp.layers.0.", true);
    add("mtp.norm.weight", {H}, false, zero);
    add("mtp.pre_fc_norm_embedding.weight", {H}, false, zero);
    add("mtp.pre_fc_norm_hidden.weight", {H}, false, zero);
  }
}

template <typename T>
static T rd(const uint8_t *p) {
  T v;
  std::memcpy(&v, p, sizeof(T));
  return v;
}

// Container parse per docs/binfer_spec.md sections 3, 8, 11 (magic, section
// table with CRCs, 192-byte directory entries, span checks against
// total-32); mirrors the checks of tools/decode/decode_l0.cpp:127-189 and
// tools/binfer.py:397-470. check_payload_crc enables the per-tensor CRC pass.
static Model *model_open(const char *path, int check_payload_crc, std::string &err) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) { err = "cannot open file"; return nullptr; }
  struct stat st;
  fstat(fd, &st);
  size_t size = (size_t)st.st_size;
  if (size < 128 + 32) { close(fd); err = "truncated (shorter than header)"; return nullptr; }
  const uint8_t *m = (const uint8_t *)mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
  if (m == MAP_FAILED) { close(fd); err = "mmap failed"; return nullptr; }
  Model *M = new Model;
  M->map = m; M->map_bytes = size; M->fd = fd;
  auto bail = [&](const std::string &e) { err = e; delete M; return (Model *)nullptr; };
  if (std::memcmp(m, "BINFER\x00\x01", 8) != 0) return bail("bad magic (not a .binfer file)");
  if (rd<uint32_t>(m + 8) != 1) return bail("bad version");
  if (rd<uint32_t>(m + 12) & ~1u) return bail("reserved flags set");
  uint64_t n = rd<uint64_t>(m + 16), table_off = rd<uint64_t>(m + 24);
  uint32_t scount = rd<uint32_t>(m + 32);
  if (rd<uint32_t>(m + 36) != 64) return bail("bad alignment field");
  if (rd<uint64_t>(m + 40) != size) return bail("total mismatch");
  if (table_off + (uint64_t)scount * 32 > size) return bail("section table out of range");
  uint64_t dir_off = 0, dir_bytes = 0;
  bool have_dir = false;
  for (uint32_t i = 0; i < scount; ++i) {
    const uint8_t *e = m + table_off + i * 32;
    uint32_t sid = rd<uint32_t>(e);
    uint64_t off = rd<uint64_t>(e + 4), nb = rd<uint64_t>(e + 12);
    uint32_t crc = rd<uint32_t>(e + 20);
    if (off + nb > size - 32) return bail("section out of range");
    if (sid == 5) {
      if (crc32_bytes(m + off, nb) != crc) return bail("section 5 (dir) CRC mismatch");
      dir_off = off; dir_bytes = nb; have_dir = true;
    } else {
      uint64_t ln = rd<uint64_t>(m + off);
      if (ln + 8 > nb) return bail("section length implausible");
      if (crc32_bytes(m + off, 8 + ln) != crc) return bail("section CRC mismatch");
      if (sid == 2) M->arch_json.assign((const char *)m + off + 8, ln);
    }
  }
  if (!have_dir) return bail("missing section 5");
  if (dir_bytes != n * 192) return bail("dir size mismatch");
  for (uint64_t i = 0; i < n; ++i) {
    const uint8_t *e = m + dir_off + i * 192;
    char name[65];
    std::memcpy(name, e, 64);
    name[64] = 0;
    Tensor t;
    t.ndim = e[64];
    for (int d = 0; d < 8; ++d) t.shape[d] = rd<uint64_t>(e + 72 + 8 * d);
    t.storage = e[137];
    uint16_t layout = rd<uint16_t>(e + 138);
    uint64_t sc_off = rd<uint64_t>(e + 144), sc_bytes = rd<uint64_t>(e + 152);
    uint64_t d_off = rd<uint64_t>(e + 160), d_bytes = rd<uint64_t>(e + 168);
    uint32_t crc = rd<uint32_t>(e + 176);
    if (layout != 0) return bail(std::string("unsupported layout_id: ") + name);
    if (d_bytes == 0 || d_off + d_bytes > size - 32)
      return bail(std::string("payload span out of range: ") + name);
    if (sc_bytes && sc_off + sc_bytes > size - 32)
      return bail(std::string("scale span out of range: ") + name);
    if (check_payload_crc && crc32_bytes(m + d_off, d_bytes) != crc)
      return bail(std::string("payload CRC ") + name);
    t.data = m + d_off; t.data_bytes = d_bytes;
    t.scales = sc_bytes ? (const uint16_t *)(m + sc_off) : nullptr;
    t.scale_bytes = sc_bytes;
    M->tensors[name] = t;
  }
  M->cfg = parse_cfg(M->arch_json);
  return M;
}

// ------------------------------------------------------------- session ---
struct Session {
  const Model *M;
  int max_ctx;
  int n_lin = 0, n_attn = 0;
  std::vector<int> slot;               // per layer: index within its type
  std::vector<float> conv;             // [n_lin][conv_dim][3]
  std::vector<float> S;                // [n_lin][nV][D][D]
  std::vector<int8_t> Kc, Vc;          // [n_attn(+mtp)][max_ctx][nKV][hd]
  std::vector<uint16_t> Ks, Vs;        // [n_attn(+mtp)][max_ctx][nKV]
  std::vector<float> x;                // residual stream
  std::vector<float> hidden_prenorm;   // residual stream after the last layer
  std::vector<float> logits;
  // per-step diagnostics
  std::vector<int> routed;             // [layers][top_k]
  std::vector<float> near_gap;         // [layers]
  std::vector<float> layer_out;        // [layers][hidden]
};

static Session *session_new(const Model *M, int max_ctx) {
  const Cfg &c = M->cfg;
  Session *s = new Session;
  s->M = M;
  s->max_ctx = max_ctx;
  s->slot.resize(c.layers);
  for (int l = 0; l < c.layers; ++l)
    s->slot[l] = c.layer_types[l] == 'A' ? s->n_attn++ : s->n_lin++;
  int n_kv_layers = s->n_attn + c.mtp_layers;
  s->conv.assign((size_t)s->n_lin * c.conv_dim() * 3, 0.0f);
  s->S.assign((size_t)s->n_lin * c.lin_v_heads * c.lin_head_dim * c.lin_head_dim, 0.0f);
  size_t kvn = (size_t)n_kv_layers * max_ctx * c.kv_heads * c.head_dim;
  s->Kc.assign(kvn, 0); s->Vc.assign(kvn, 0);
  s->Ks.assign((size_t)n_kv_layers * max_ctx * c.kv_heads, 0);
  s->Vs.assign((size_t)n_kv_layers * max_ctx * c.kv_heads, 0);
  s->x.assign(c.hidden, 0.0f);
  s->hidden_prenorm.assign(c.hidden, 0.0f);
  s->logits.assign(c.vocab, 0.0f);
  s->routed.assign((size_t)c.layers * c.top_k, -1);
  s->near_gap.assign(c.layers, 1.0f);
  s->layer_out.assign((size_t)c.layers * c.hidden, 0.0f);
  return s;
}

static std::vector<float> small_f32(const Tensor &t) {
  size_t n = t.numel();
  std::vector<float> out(n);
  if (t.storage == ST_BF16) {
    const uint16_t *p = (const uint16_t *)t.data;
    for (size_t i = 0; i < n; ++i) out[i] = bf16_to_f32(p[i]);
  } else if (t.storage == ST_FP32) {
    std::memcpy(out.data(), t.data, n * 4);
  } else {
    std::fprintf(stderr, "oracle: small tensor with storage %d\n", t.storage);
    std::abort();
  }
  return out;
}

struct Quant {  // A-quantised activation vector
  std::vector<int8_t> q;
  std::vector<float> s;
  void run(const float *x, int n) {
    q.resize(n); s.resize(n / 128);
    aquant_g128(x, n, q.data(), s.data());
  }
};

static void gemv_t(const Tensor &t, const Quant &a, float *y) {
  int N = (int)t.shape[0], K = (int)t.shape[1];
  gemv_a8(t.data, t.scales, N, K, a.q.data(), a.s.data(), y);
}

// MoE block (contract stated in oracle_ops.h): router on the fp32 normalised
// activations, top-k, each selected expert = gate/up GEMV, silu(g)*u, A-quant,
// down GEMV; combine in rank order, then the shared expert scaled by
// sigmoid(shared_gate . h). Expert MLP follows tools/decode/decode_l0.cpp:666-674.
static void moe_block(const Model &M, const std::string &pfx, const float *hn, const Quant &hq,
                      float *out, int *routed, float *near_gap) {
  const Cfg &c = M.cfg;
  int H = c.hidden, E = c.experts, k = c.top_k, I = c.expert_inter;
  const Tensor &router = M.get(pfx + "mlp.gate.weight");
  std::vector<float> logits(E);
  parallel_for((int64_t)(E), [&](int64_t e_) {
    int e = (int)e_;
    logits[e] = dot_bf16_row((const uint16_t *)router.data + (size_t)e * H, hn, H);
  });
  std::vector<int> idx(k);
  std::vector<float> wt(k);
  router_topk(logits.data(), E, k, idx.data(), wt.data(), near_gap);
  for (int j = 0; j < k; ++j) routed[j] = idx[j];
  int slots = k + (c.shared_experts ? 1 : 0);
  std::vector<float> y((size_t)slots * H);
  // the slots' tensors once, then every (slot, row) as its own work item
  std::vector<const Tensor *> wg(slots), wu(slots), wd(slots);
  for (int s = 0; s < slots; ++s) {
    std::string ep = s < k ? pfx + "mlp.experts." + std::to_string(idx[s]) + "."
                           : pfx + "mlp.shared.";
    wg[s] = &M.get(ep + "gate_proj.weight");
    wu[s] = &M.get(ep + "up_proj.weight");
    wd[s] = &M.get(ep + "down_proj.weight");
  }
  std::vector<float> act((size_t)slots * I);
  parallel_for((int64_t)slots * I, [&](int64_t i_) {
    int s = (int)(i_ / I), n = (int)(i_ % I);
    float g = gemv_a8_row(wg[s]->data, wg[s]->scales, n, H, hq.q.data(), hq.s.data());
    float u = gemv_a8_row(wu[s]->data, wu[s]->scales, n, H, hq.q.data(), hq.s.data());
    act[(size_t)s * I + n] = (g / (1.0f + det_expf(-g))) * u;
  });
  std::vector<Quant> aq(slots);
  for (int s = 0; s < slots; ++s) aq[s].run(&act[(size_t)s * I], I);
  parallel_for((int64_t)slots * H, [&](int64_t i_) {
    int s = (int)(i_ / H), n = (int)(i_ % H);
    y[i_] = gemv_a8_row(wd[s]->data, wd[s]->scales, n, I, aq[s].q.data(), aq[s].s.data());
  });
  float sg = 0.0f;
  if (c.shared_experts) {
    const Tensor &sgw = M.get(pfx + "mlp.shared_expert_gate.weight");
    sg = 1.0f / (1.0f + det_expf(-dot_bf16_row((const uint16_t *)sgw.data, hn, H)));
  }
  for (int n = 0; n < H; ++n) {
    float acc = 0.0f;
    for (int s = 0; s < k; ++s) acc = acc + wt[s] * y[(size_t)s * H + n];
    if (c.shared_experts) acc = acc + sg * y[(size_t)k * H + n];
    out[n] = acc;
  }
}

// Full-attention mixer (q|gate split, QK-norm, RoPE, INT8 KV append, split
// attention, A-quant, o_proj). Order: tools/decode/decode_l0.cpp:562-608.
static void attn_mixer(const Model &M, Session &s, const std::string &pfx, int kv_slot,
                       const Quant &hq, int pos, float *mix) {
  const Cfg &c = M.cfg;
  int nQ = c.q_heads, nKV = c.kv_heads, D = c.head_dim, H = c.hidden;
  std::vector<float> q16((size_t)nQ * 2 * D), k16((size_t)nKV * D), v16((size_t)nKV * D);
  gemv_t(M.get(pfx + "self_attn.q_proj.weight"), hq, q16.data());
  gemv_t(M.get(pfx + "self_attn.k_proj.weight"), hq, k16.data());
  gemv_t(M.get(pfx + "self_attn.v_proj.weight"), hq, v16.data());
  std::vector<float> qn((size_t)nQ * D), gate((size_t)nQ * D), kn((size_t)nKV * D);
  for (int h = 0; h < nQ; ++h)
    for (int d = 0; d < D; ++d) {
      qn[(size_t)h * D + d] = q16[(size_t)h * 2 * D + d];
      gate[(size_t)h * D + d] = q16[(size_t)h * 2 * D + D + d];
    }
  std::vector<float> qnw = small_f32(M.get(pfx + "self_attn.q_norm.weight"));
  std::vector<float> knw = small_f32(M.get(pfx + "self_attn.k_norm.weight"));
  std::vector<float> cs(c.rotary_dim), sn(c.rotary_dim);
  rope_table(pos, c.rotary_dim, c.rope_theta, cs.data(), sn.data());
  for (int h = 0; h < nQ; ++h) {
    headnorm_1pw(&qn[(size_t)h * D], qnw.data(), D, c.rms_eps, &qn[(size_t)h * D]);
    rope_apply(&qn[(size_t)h * D], c.rotary_dim, cs.data(), sn.data());
  }
  for (int h = 0; h < nKV; ++h) {
    headnorm_1pw(&k16[(size_t)h * D], knw.data(), D, c.rms_eps, &kn[(size_t)h * D]);
    rope_apply(&kn[(size_t)h * D], c.rotary_dim, cs.data(), sn.data());
  }
  int p = pos < s.max_ctx ? pos : s.max_ctx - 1;  // clamp as KvAppend (kernels.cpp:456)
  size_t base = (size_t)kv_slot * s.max_ctx;
  for (int h = 0; h < nKV; ++h) {
    size_t row = (base + p) * nKV + h;
    kv_quant_row(&kn[(size_t)h * D], D, &s.Kc[row * D], &s.Ks[row]);
    kv_quant_row(&v16[(size_t)h * D], D, &s.Vc[row * D], &s.Vs[row]);
  }
  int T = pos + 1 < s.max_ctx ? pos + 1 : s.max_ctx;
  std::vector<float> att((size_t)nQ * D);
  attn_decode_int8kv(qn.data(), &s.Kc[base * nKV * D], &s.Ks[base * nKV], &s.Vc[base * nKV * D],
                     &s.Vs[base * nKV], gate.data(), nQ, nKV, D, T, att.data());
  Quant aq;
  aq.run(att.data(), nQ * D);
  gemv_t(M.get(pfx + "self_attn.o_proj.weight"), aq, mix);
  (void)H;
}

// Gated DeltaNet mixer. Order: tools/decode/decode_l0.cpp:610-661.
static void linear_mixer(const Model &M, Session &s, const std::string &pfx, int slot,
                         const Quant &hq, float *mix) {
  const Cfg &c = M.cfg;
  int nK = c.lin_k_heads, nV = c.lin_v_heads, D = c.lin_head_dim, C = c.conv_dim();
  int ratio = nV / nK;
  std::vector<float> qkv(C), z((size_t)nV * D), b(nV), a(nV), mx(C);
  gemv_t(M.get(pfx + "linear_attn.in_proj_qkv.weight"), hq, qkv.data());
  gemv_t(M.get(pfx + "linear_attn.in_proj_z.weight"), hq, z.data());
  gemv_t(M.get(pfx + "linear_attn.in_proj_b.weight"), hq, b.data());
  gemv_t(M.get(pfx + "linear_attn.in_proj_a.weight"), hq, a.data());
  std::vector<float> cw = small_f32(M.get(pfx + "linear_attn.conv1d.weight"));
  std::vector<float> al = small_f32(M.get(pfx + "linear_attn.A_log"));
  std::vector<float> dt = small_f32(M.get(pfx + "linear_attn.dt_bias"));
  std::vector<float> ng = small_f32(M.get(pfx + "linear_attn.norm.weight"));
  conv_silu_step(qkv.data(), &s.conv[(size_t)slot * C * 3], cw.data(), C, mx.data());
  std::vector<float> att((size_t)nV * D);
  float qmul = 1.0f / sqrtf((float)D);
  parallel_for((int64_t)(nV), [&](int64_t h_) {
    int h = (int)h_;
    int kh = h / ratio;
    std::vector<float> qh(D), kk(D), o(D);
    l2norm_head(&mx[(size_t)kh * D], D, qmul, qh.data());
    l2norm_head(&mx[(size_t)nK * D + (size_t)kh * D], D, 1.0f, kk.data());
    const float *vh = &mx[(size_t)2 * nK * D + (size_t)h * D];
    float beta = dn_beta(b[h]);
    float g = dn_gdecay(a[h], al[h], dt[h]);
    float *S = &s.S[((size_t)slot * nV + h) * D * D];
    deltanet_head_step(S, qh.data(), kk.data(), vh, beta, g, D, o.data());
    gated_norm_head(o.data(), &z[(size_t)h * D], ng.data(), D, &att[(size_t)h * D]);
  });
  Quant aq;
  aq.run(att.data(), nV * D);
  gemv_t(M.get(pfx + "linear_attn.out_proj.weight"), aq, mix);
}

// One decoder layer on the residual stream x (in place).
static void decoder_layer(const Model &M, Session &s, const std::string &pfx, bool is_attn,
                          int slot, int pos, float *x, int *routed, float *near_gap) {
  const Cfg &c = M.cfg;
  int H = c.hidden;
  std::vector<float> h(H), mix(H), tmp(H), moe(H);
  std::vector<float> w_in = small_f32(M.get(pfx + "input_layernorm.weight"));
  std::vector<float> w_post = small_f32(M.get(pfx + "post_attention_layernorm.weight"));
  rmsnorm_1pw(x, w_in.data(), H, c.rms_eps, h.data());
  Quant hq;
  hq.run(h.data(), H);
  if (is_attn) attn_mixer(M, s, pfx, slot, hq, pos, mix.data());
  else linear_mixer(M, s, pfx, slot, hq, mix.data());
  for (int j = 0; j < H; ++j) tmp[j] = x[j] + mix[j];
  rmsnorm_1pw(tmp.data(), w_post.data(), H, c.rms_eps, h.data());
  hq.run(h.data(), H);
  moe_block(M, pfx, h.data(), hq, moe.data(), routed, near_gap);
  for (int j = 0; j < H; ++j) x[j] = tmp[j] + moe[j];
}

static void embed_row(const Model &M, int token, float *x) {
  const Tensor &emb = M.get("model.language_model.embed_tokens.weight");
  int H = M.cfg.hidden;
  const uint16_t *row = (const uint16_t *)emb.data + (size_t)token * H;
  for (int j = 0; j < H; ++j) x[j] = bf16_to_f32(row[j]);
}

static int lm_head_argmax(const Model &M, const float *x_prenorm, const char *norm_name,
                          float *logits) {
  const Cfg &c = M.cfg;
  int H = c.hidden;
  std::vector<float> h(H);
  std::vector<float> wf = small_f32(M.get(norm_name));
  rmsnorm_1pw(x_prenorm, wf.data(), H, c.rms_eps, h.data());
  Quant hq;
  hq.run(h.data(), H);
  gemv_t(M.get("lm_head.weight"), hq, logits);
  return argmax_first(logits, c.vocab);
}

// One trunk token: embed -> layers -> (optionally) final norm + lm_head + argmax.
// (tools/decode/decode_l0.cpp:753-775.)
static int step(Session &s, int token, int pos, bool want_logits) {
  const Model &M = *s.M;
  const Cfg &c = M.cfg;
  int H = c.hidden;
  embed_row(M, token, s.x.data());
  for (int L = 0; L < c.layers; ++L) {
    std::string pfx = "model.language_model.layers." + std::to_string(L) + ".";
    decoder_layer(M, s, pfx, c.layer_types[L] == 'A', s.slot[L], pos, s.x.data(),
                  &s.routed[(size_t)L * c.top_k], &s.near_gap[L]);
    std::memcpy(&s.layer_out[(size_t)L * H], s.x.data(), (size_t)H * 4);
  }
  s.hidden_prenorm = s.x;
  if (!want_logits) return -1;
  return lm_head_argmax(M, s.x.data(), "model.language_model.norm.weight", s.logits.data());
}

// MTP draft step: x = fc . [rms1w(embed(next_token)) ; rms1w(h_prev)], one full
// attention decoder layer with its own KV slot, mtp.norm, shared lm_head.
// (tools/t72/mtp_accept.py:11-16,66-94,142-159.) h_io: in = hidden feeding the
// draft, out = the MTP layer's output hidden (feeds the next chained draft).
static int mtp_step(Session &s, int next_token, int pos, float *h_io, float *logits) {
  const Model &M = *s.M;
  const Cfg &c = M.cfg;
  int H = c.hidden;
  std::vector<float> e(H), en(H), hn(H), cat((size_t)2 * H), x(H);
  embed_row(M, next_token, e.data());
  std::vector<float> we = small_f32(M.get("mtp.pre_fc_norm_embedding.weight"));
  std::vector<float> wh = small_f32(M.get("mtp.pre_fc_norm_hidden.weight"));
  rmsnorm_1pw(e.data(), we.data(), H, c.rms_eps, en.data());
  rmsnorm_1pw(h_io, wh.data(), H, c.rms_eps, hn.data());
  std::memcpy(cat.data(), en.data(), (size_t)H * 4);
  std::memcpy(cat.data() + H, hn.data(), (size_t)H * 4);
  Quant cq;
  cq.run(cat.data(), 2 * H);
  gemv_t(M.get("mtp.fc.weight"), cq, x.data());
  std::vector<int> routed(c.top_k);
  float gap;
  decoder_layer(M, s, "mtp.layers.0.", true, s.n_attn, pos, x.data(), routed.data(), &gap);
  std::memcpy(h_io, x.data(), (size_t)H * 4);
  return lm_head_argmax(M, x.data(), "mtp.norm.weight", logits);
}

}  // namespace orc

// ============================================================== C entry ===
using namespace orc;
extern "C" {

void *orc_model_open(const char *path, int check_crc, char *err, int errlen) {
  std::string e;
  Model *m = model_open(path, check_crc, e);
  if (!m && err && errlen > 0) std::snprintf(err, errlen, "%s", e.c_str());
  return m;
}
// In-memory model: tensors are registered with borrowed host pointers.
void *orc_model_new(const char *arch_json) {
  Model *m = new Model;
  m->arch_json = arch_json;
  m->cfg = parse_cfg(m->arch_json);
  return m;
}
void orc_model_add_tensor(void *model, const char *name, int storage, int ndim,
                          const uint64_t *shape, const void *data, uint64_t data_bytes,
                          const void *scales, uint64_t scale_bytes) {
  Tensor t;
  t.storage = storage; t.ndim = ndim;
  for (int i = 0; i < ndim; ++i) t.shape[i] = shape[i];
  t.data = (const uint8_t *)data; t.data_bytes = data_bytes;
  t.scales = (const uint16_t *)scales; t.scale_bytes = scale_bytes;
  ((Model *)model)->tensors[name] = t;
}
// Lazily generated synthetic model of the shape given by arch_json.
void *orc_model_synth(const char *arch_json, uint64_t seed) {
  Model *m = new Model;
  m->arch_json = arch_json;
  m->cfg = parse_cfg(m->arch_json);
  m->lazy = true;
  m->seed = seed;
  synth_plan(*m);
  return m;
}
void orc_model_close(void *model) { delete (Model *)model; }
const char *orc_model_arch_json(void *model) { return ((Model *)model)->arch_json.c_str(); }
int orc_model_tensor_count(void *model) { return (int)((Model *)model)->tensors.size(); }
int orc_model_tensor_info(void *model, const char *name, int *storage, int *ndim, uint64_t *shape,
                          const void **data, uint64_t *data_bytes, const void **scales,
                          uint64_t *scale_bytes) {
  Model *m = (Model *)model;
  if (!m->has(name)) return -1;
  const Tensor &t = m->get(name);
  *storage = t.storage; *ndim = t.ndim;
  for (int i = 0; i < 8; ++i) shape[i] = t.shape[i];
  *data = t.data; *data_bytes = t.data_bytes; *scales = t.scales; *scale_bytes = t.scale_bytes;
  return 0;
}

void *orc_session_new(void *model, int max_ctx) { return session_new((Model *)model, max_ctx); }
void orc_session_free(void *sess) { delete (Session *)sess; }
// Raw state access (numpy views): which = 0 conv, 1 S, 2 Kc, 3 Vc, 4 Ks, 5 Vs,
// 6 logits, 7 routed, 8 near_gap, 9 layer_out, 10 hidden_prenorm.
void *orc_session_buf(void *sess, int which, uint64_t *bytes) {
  Session *s = (Session *)sess;
  switch (which) {
    case 0: *bytes = s->conv.size() * 4; return s->conv.data();
    case 1: *bytes = s->S.size() * 4; return s->S.data();
    case 2: *bytes = s->Kc.size(); return s->Kc.data();
    case 3: *bytes = s->Vc.size(); return s->Vc.data();
    case 4: *bytes = s->Ks.size() * 2; return s->Ks.data();
    case 5: *bytes = s->Vs.size() * 2; return s->Vs.data();
    case 6: *bytes = s->logits.size() * 4; return s->logits.data();
    case 7: *bytes = s->routed.size() * 4; return s->routed.data();
    case 8: *bytes = s->near_gap.size() * 4; return s->near_gap.data();
    case 9: *bytes = s->layer_out.size() * 4; return s->layer_out.data();
    case 10: *bytes = s->hidden_prenorm.size() * 4; return s->hidden_prenorm.data();
  }
  *bytes = 0;
  return nullptr;
}
int orc_step(void *sess, int token, int pos, int want_logits) {
  return step(*(Session *)sess, token, pos, want_logits != 0);
}
int orc_mtp_step(void *sess, int next_token, int pos, float *h_io, float *logits) {
  return mtp_step(*(Session *)sess, next_token, pos, h_io, logits);
}
// The MoE block of one layer on its own (for cross-checks against third-party
// implementations): hn = the normalised fp32 activations, which are also quantised here the way
// decoder_layer does before calling the block. out[H], routed[top_k], near_gap[1].
void orc_moe_block(void *model, const char *prefix, const float *hn, float *out, int *routed,
                   float *near_gap) {
  const Model &M = *(Model *)model;
  Quant hq;
  hq.run(hn, M.cfg.hidden);
  moe_block(M, prefix, hn, hq, out, routed, near_gap);
}
// Greedy token loop: prompt of P ids, then G generated tokens; as
// tools/decode/decode_l0.cpp:742-825 (logits only from step P-1 on).
// Returns seconds spent in the generation phase (steps >= P-1... P+G-1).
double orc_decode_loop(void *sess, const int *prompt, int P, int G, int start_pos, int *out_tokens) {
  Session &s = *(Session *)sess;
  int tok = -1;
  auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < P + G - 1 + (G == 0 ? 0 : 0); ++i) {
    int in = i < P ? prompt[i] : tok;
    bool want = i >= P - 1;
    if (i == P - 1) t0 = std::chrono::steady_clock::now();
    int r = step(s, in, start_pos + i, want);
    if (want) {
      tok = r;
      out_tokens[i - (P - 1)] = r;
    }
  }
  return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}
int orc_threads(void) {
  return Pool::get().threads();
}

// ------------------------------------------------------ operator entry ---
void orc_quantize_int4(const float *w, uint64_t numel, uint8_t *packed, uint16_t *scales) {
  quantize_int4_g128(w, numel, packed, scales);
}
void orc_aquant(const float *x, int n, int8_t *q8, float *sq) { aquant_g128(x, n, q8, sq); }
void orc_gemv_a8(const uint8_t *P, const uint16_t *S, int N, int K, const int8_t *xq,
                 const float *sq, float *y) {
  gemv_a8(P, S, N, K, xq, sq, y);
}
void orc_gemv_a16(const uint8_t *P, const uint16_t *S, int N, int K, const float *x, int M,
                  float *y) {
  gemv_a16(P, S, N, K, x, M, y);
}
void orc_rmsnorm(const float *x, const float *w, int n, float eps, float *y) {
  rmsnorm_1pw(x, w, n, eps, y);
}
void orc_headnorm(const float *x, const float *w, int n, float eps, float *y) {
  headnorm_1pw(x, w, n, eps, y);
}
void orc_rope_table(int pos, int rot, double theta, float *cs, float *sn) {
  rope_table(pos, rot, theta, cs, sn);
}
void orc_rope_apply(float *x, int rot, const float *cs, const float *sn) {
  rope_apply(x, rot, cs, sn);
}
void orc_kv_quant_row(const float *x, int D, int8_t *q, uint16_t *s16) {
  kv_quant_row(x, D, q, s16);
}
void orc_attn_bf16kv(const float *q, const uint16_t *Kc, const uint16_t *Vc, const float *gate,
                     int nQ, int nKV, int D, int T, float *out, float *wts) {
  attn_decode_bf16kv(q, Kc, Vc, gate, nQ, nKV, D, T, out, wts);
}
void orc_attn_int8kv(const float *q, const int8_t *Kc, const uint16_t *Ks, const int8_t *Vc,
                     const uint16_t *Vs, const float *gate, int nQ, int nKV, int D, int T,
                     float *out) {
  attn_decode_int8kv(q, Kc, Ks, Vc, Vs, gate, nQ, nKV, D, T, out);
}
void orc_conv_silu(const float *x, float *cs, const float *cw, int C, float *mx) {
  conv_silu_step(x, cs, cw, C, mx);
}
void orc_l2norm(const float *x, int n, float mul, float *y) { l2norm_head(x, n, mul, y); }
float orc_dn_beta(float b) { return dn_beta(b); }
float orc_dn_gdecay(float a, float al, float dt) { return dn_gdecay(a, al, dt); }
void orc_deltanet_head(float *S, const float *q, const float *k, const float *v, float beta,
                       float g, int D, float *o) {
  deltanet_head_step(S, q, k, v, beta, g, D, o);
}
void orc_gated_norm(const float *o, const float *z, const float *w, int D, float *y) {
  gated_norm_head(o, z, w, D, y);
}
float orc_dot_bf16(const uint16_t *w, const float *x, int K) { return dot_bf16_row(w, x, K); }
void orc_router_topk(const float *logits, int E, int k, int *idx, float *wt, float *gap) {
  router_topk(logits, E, k, idx, wt, gap);
}
int orc_argmax(const float *x, int n) { return argmax_first(x, n); }
float orc_expf(float x) { return det_expf(x); }
float orc_logf(float x) { return det_logf(x); }
uint16_t orc_f32_to_f16(float x) { return f32_to_f16(x); }
float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
uint16_t orc_f32_to_bf16(float x) { return f32_to_bf16(x); }
uint32_t orc_crc32(const uint8_t *p, uint64_t n) { return crc32_bytes(p, n); }
// Synthetic inputs: value(i) = std * N(0,1) drawn from (seed, fnv1a(name), i).
void orc_synth_normal(const char *name, uint64_t seed, uint64_t first, uint64_t count, float std_,
                      float *out) {
  uint64_t stream = fnv1a64(name);
  parallel_for((int64_t)(count), [&](int64_t i_) {
    uint64_t i = (uint64_t)i_;
    out[i] = std_ * normal_from_u32(draw_u32(seed, stream, first + i));
  });
}
uint32_t orc_draw_u32(const char *name, uint64_t seed, uint64_t idx) {
  return draw_u32(seed, fnv1a64(name), idx);
}
float orc_normal_from_u32(uint32_t r) { return normal_from_u32(r); }

}  // extern "C"
