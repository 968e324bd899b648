#include "model.h"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <thread>

#include "../common/detmath.h"
#include "../common/tables.h"
#include "rt_util.h"

namespace ainfer {

std::string layer_prefix(int L) { return "model.language_model.layers." + std::to_string(L) + "."; }

// ------------------------------------------------------------- config ---
std::string ModelConfig::to_json() const {
  char b[1024];
  std::snprintf(
      b, sizeof b,
      "{\"arch\":\"%s\",\"text_layers\":%d,\"layer_types\":\"%s\",\"hidden\":%d,\"vocab\":%d,"
      "\"q_heads\":%d,\"kv_heads\":%d,\"head_dim\":%d,\"rotary_dim\":%d,\"rope_theta\":%.1f,"
      "\"lin_k_heads\":%d,\"lin_v_heads\":%d,\"lin_head_dim\":%d,\"conv_kernel\":%d,"
      "\"experts\":%d,\"top_k\":%d,\"shared_experts\":%d,\"expert_intermediate\":%d,"
      "\"mtp_layers\":%d,\"rms_eps\":%.9g,\"kv_cache\":\"int8_per_token_head_fp16_scale\","
      "\"attn_output_gate\":true,\"mlp_act\":\"silu\",\"vision\":\"absent\"}",
      arch.c_str(), layers, layer_types.c_str(), hidden, vocab, q_heads, kv_heads, head_dim,
      rotary_dim, rope_theta, lin_k_heads, lin_v_heads, lin_head_dim, conv_kernel, experts, top_k,
      shared_experts, expert_inter, mtp_layers, rms_eps);
  return b;
}

static bool json_raw(const std::string &js, const char *key, std::string &out) {
  std::string pat = std::string("\"") + key + "\":";
  size_t p = js.find(pat);
  if (p == std::string::npos) return false;
  p += pat.size();
  while (p < js.size() && js[p] == ' ') ++p;
  if (p < js.size() && js[p] == '"') {
    size_t e = js.find('"', p + 1);
    if (e == std::string::npos) return false;
    out = js.substr(p + 1, e - p - 1);
  } else {
    size_t e = p;
    while (e < js.size() && js[e] != ',' && js[e] != '}') ++e;
    out = js.substr(p, e - p);
  }
  return true;
}
static long jint(const std::string &js, const char *k, long d) {
  std::string v;
  return json_raw(js, k, v) ? std::strtol(v.c_str(), nullptr, 10) : d;
}
static double jnum(const std::string &js, const char *k, double d) {
  std::string v;
  return json_raw(js, k, v) ? std::strtod(v.c_str(), nullptr) : d;
}

bool ModelConfig::from_json(const std::string &js, ModelConfig &c, std::string &err) {
  c = ModelConfig();
  json_raw(js, "arch", c.arch);
  c.hidden = (int)jint(js, "hidden", 0);
  c.layers = (int)jint(js, "text_layers", 0);
  c.vocab = (int)jint(js, "vocab", 0);
  json_raw(js, "layer_types", c.layer_types);
  c.q_heads = (int)jint(js, "q_heads", 0);
  c.kv_heads = (int)jint(js, "kv_heads", 0);
  c.head_dim = (int)jint(js, "head_dim", 256);
  c.rotary_dim = (int)jint(js, "rotary_dim", 64);
  c.rope_theta = jnum(js, "rope_theta", 1e7);
  c.lin_k_heads = (int)jint(js, "lin_k_heads", 0);
  c.lin_v_heads = (int)jint(js, "lin_v_heads", 0);
  c.lin_head_dim = (int)jint(js, "lin_head_dim", 128);
  c.conv_kernel = (int)jint(js, "conv_kernel", 4);
  c.experts = (int)jint(js, "experts", 0);
  c.top_k = (int)jint(js, "top_k", 0);
  c.shared_experts = (int)jint(js, "shared_experts", 1);
  c.expert_inter = (int)jint(js, "expert_intermediate", 0);
  c.mtp_layers = (int)jint(js, "mtp_layers", 0);
  c.rms_eps = jnum(js, "rms_eps", 1e-6);
  if (c.layer_types.empty())  // the reference's fixed 3:1 pattern (decode_l0.cpp:297)
    for (int l = 0; l < c.layers; ++l) c.layer_types += (l % 4 == 3) ? 'A' : 'L';
  return c.check(err);
}

static bool pow2_between(int v, int lo, int hi) { return v >= lo && v <= hi && (v & (v - 1)) == 0; }

bool ModelConfig::check(std::string &err) const {
  auto bad = [&](const std::string &m) { err = "unsupported architecture: " + m; return false; };
  if (layers <= 0 || (int)layer_types.size() != layers) return bad("layer_types/text_layers mismatch");
  for (char c : layer_types)
    if (c != 'L' && c != 'A') return bad("layer_types may hold only L and A");
  if (!pow2_between(hidden, 256, 4096)) return bad("hidden must be a power of two in [256, 4096]");
  if (vocab <= 0) return bad("vocab");
  if (head_dim != 256) return bad("head_dim must be 256");
  if (rotary_dim != 64) return bad("rotary_dim must be 64");
  if (n_attn() || mtp_layers) {
    if (kv_heads <= 0 || q_heads % kv_heads) return bad("q_heads must be a multiple of kv_heads");
    int g = q_heads / kv_heads;
    if (g != 1 && g != 2 && g != 4 && g != 6 && g != 8) return bad("q_heads/kv_heads must be 1, 2, 4, 6 or 8");
    if (!pow2_between(q_heads * head_dim, 128, 4096)) return bad("q_heads*head_dim must be a power of two <= 4096");
  }
  if (n_lin()) {
    if (lin_head_dim != 128) return bad("lin_head_dim must be 128");
    if (conv_kernel != 4) return bad("conv_kernel must be 4");
    if (lin_k_heads <= 0 || lin_v_heads % lin_k_heads) return bad("lin_v_heads must be a multiple of lin_k_heads");
    if (!pow2_between(value_dim(), 128, 4096)) return bad("lin_v_heads*128 must be a power of two <= 4096");
  }
  if (experts < 32 || experts > 1024 || experts % 32) return bad("experts must be a multiple of 32 in [32, 1024]");
  if (top_k <= 0 || top_k > 11 || top_k > experts) return bad("top_k must be in [1, 11]");
  if (shared_experts != 0 && shared_experts != 1) return bad("shared_experts must be 0 or 1");
  if (!pow2_between(expert_inter, 128, 1024)) return bad("expert_intermediate must be a power of two in [128, 1024]");
  if (mtp_layers != 0 && mtp_layers != 1) return bad("mtp_layers must be 0 or 1");
  return true;
}

bool preset_config(const std::string &name, ModelConfig &c) {
  c = ModelConfig();
  if (name == "tiny") {
    c.hidden = 256; c.layers = 2; c.layer_types = "LA"; c.vocab = 512;
    c.q_heads = 2; c.kv_heads = 1; c.lin_k_heads = 2; c.lin_v_heads = 4;
    c.experts = 32; c.top_k = 2; c.expert_inter = 128; c.mtp_layers = 1;
  } else if (name == "mini") {
    c.hidden = 1024; c.layers = 2; c.layer_types = "LA"; c.vocab = 32000;
    c.q_heads = 8; c.kv_heads = 2; c.lin_k_heads = 8; c.lin_v_heads = 16;
    c.experts = 64; c.top_k = 4; c.expert_inter = 256; c.mtp_layers = 0;
  } else if (name == "mini-mtp") {
    preset_config("mini", c);
    c.mtp_layers = 1;
  } else if (name == "small") {  // four full-width layers of the full shape, small vocab
    c.hidden = 2048; c.layers = 4; c.layer_types = "LLLA"; c.vocab = 32000;
    c.q_heads = 16; c.kv_heads = 2; c.lin_k_heads = 16; c.lin_v_heads = 32;
    c.experts = 512; c.top_k = 10; c.expert_inter = 512; c.mtp_layers = 1;
  } else if (name == "full") {
    c.hidden = 2048; c.layers = 48; c.vocab = 151936;
    for (int l = 0; l < 48; ++l) c.layer_types += (l % 4 == 3) ? 'A' : 'L';
    c.q_heads = 16; c.kv_heads = 2; c.lin_k_heads = 16; c.lin_v_heads = 32;
    c.experts = 512; c.top_k = 10; c.expert_inter = 512; c.mtp_layers = 1;
  } else {
    return false;
  }
  return true;
}

// --------------------------------------------------------------- plan ---
namespace {
struct PlanBuilder {
  Container &c;
  std::vector<SynthSpec> &specs;
  void add(const std::string &name, std::vector<uint64_t> shape, bool int4, SynthSpec sp) {
    TensorEntry e;
    e.name = name;
    e.ndim = (int)shape.size();
    for (size_t i = 0; i < shape.size(); ++i) e.shape[i] = shape[i];
    uint64_t n = e.numel();
    e.logical = DT_BF16;
    if (int4) {
      uint64_t ng = (n + 127) / 128;
      e.storage = DT_INT4_SYM_G128; e.group = 128; e.sc_bytes = ng * 2; e.d_bytes = ng * 64;
    } else {
      e.storage = DT_BF16; e.group = 0; e.sc_bytes = 0; e.d_bytes = n * 2;
    }
    c.entries.push_back(e);
    specs.push_back(sp);
  }
};
}  // namespace

static void plan_moe(PlanBuilder &pb, const ModelConfig &cfg, const std::string &p) {
  const uint64_t H = cfg.hidden, I = cfg.expert_inter;
  SynthSpec w{0.02f, 0.0f};
  pb.add(p + "mlp.gate.weight", {(uint64_t)cfg.experts, H}, false, w);  // router: BF16 exception
  for (int e = 0; e < cfg.experts; ++e) {
    std::string ep = p + "mlp.experts." + std::to_string(e) + ".";
    pb.add(ep + "gate_proj.weight", {I, H}, true, w);
    pb.add(ep + "up_proj.weight", {I, H}, true, w);
    pb.add(ep + "down_proj.weight", {H, I}, true, w);
  }
  if (cfg.shared_experts) {
    pb.add(p + "mlp.shared.gate_proj.weight", {I, H}, true, w);
    pb.add(p + "mlp.shared.up_proj.weight", {I, H}, true, w);
    pb.add(p + "mlp.shared.down_proj.weight", {H, I}, true, w);
    pb.add(p + "mlp.shared_expert_gate.weight", {1, H}, false, w);  // BF16 exception
  }
}
static void plan_attn(PlanBuilder &pb, const ModelConfig &cfg, const std::string &p) {
  const uint64_t H = cfg.hidden, D = cfg.head_dim;
  SynthSpec w{0.02f, 0.0f}, zero{0.0f, 0.0f};
  pb.add(p + "self_attn.q_proj.weight", {(uint64_t)cfg.q_heads * 2 * D, H}, true, w);
  pb.add(p + "self_attn.k_proj.weight", {(uint64_t)cfg.kv_heads * D, H}, true, w);
  pb.add(p + "self_attn.v_proj.weight", {(uint64_t)cfg.kv_heads * D, H}, true, w);
  pb.add(p + "self_attn.o_proj.weight", {H, (uint64_t)cfg.q_heads * D}, true, w);
  pb.add(p + "self_attn.q_norm.weight", {D}, false, zero);  // (1+w) convention: 0 = unit gain
  pb.add(p + "self_attn.k_norm.weight", {D}, false, zero);
}
static void plan_layer(PlanBuilder &pb, const ModelConfig &cfg, const std::string &p, bool attn) {
  const uint64_t H = cfg.hidden;
  SynthSpec w{0.02f, 0.0f}, zero{0.0f, 0.0f}, one{0.0f, 1.0f};
  pb.add(p + "input_layernorm.weight", {H}, false, zero);
  pb.add(p + "post_attention_layernorm.weight", {H}, false, zero);
  if (attn) {
    plan_attn(pb, cfg, p);
  } else {
    const uint64_t C = cfg.conv_dim(), VD = cfg.value_dim(), NV = cfg.lin_v_heads;
    pb.add(p + "linear_attn.in_proj_qkv.weight", {C, H}, true, w);
    pb.add(p + "linear_attn.in_proj_z.weight", {VD, H}, true, w);
    pb.add(p + "linear_attn.in_proj_b.weight", {NV, H}, true, w);
    pb.add(p + "linear_attn.in_proj_a.weight", {NV, H}, true, w);
    pb.add(p + "linear_attn.conv1d.weight", {C, 1, 4}, false, SynthSpec{0.5f, 0.0f});
    pb.add(p + "linear_attn.A_log", {NV}, false, SynthSpec{0.05f, 0.0f});
    pb.add(p + "linear_attn.dt_bias", {NV}, false, SynthSpec{0.05f, 0.0f});
    pb.add(p + "linear_attn.norm.weight", {(uint64_t)cfg.lin_head_dim}, false, one);  // plain weight
    pb.add(p + "linear_attn.out_proj.weight", {H, VD}, true, w);
  }
  plan_moe(pb, cfg, p);
}

void build_plan(const ModelConfig &cfg, Container &c, std::vector<SynthSpec> &specs) {
  c = Container();
  specs.clear();
  PlanBuilder pb{c, specs};
  const uint64_t H = cfg.hidden, V = cfg.vocab;
  SynthSpec w{0.02f, 0.0f}, zero{0.0f, 0.0f};
  pb.add("lm_head.weight", {V, H}, true, w);
  pb.add("model.language_model.embed_tokens.weight", {V, H}, false, w);
  for (int L = 0; L < cfg.layers; ++L) plan_layer(pb, cfg, layer_prefix(L), cfg.layer_types[L] == 'A');
  pb.add("model.language_model.norm.weight", {H}, false, zero);
  if (cfg.mtp_layers) {
    pb.add("mtp.fc.weight", {H, 2 * H}, true, w);
    plan_layer(pb, cfg, "mtp.layers.0.", true);
    pb.add("mtp.norm.weight", {H}, false, zero);
    pb.add("mtp.pre_fc_norm_embedding.weight", {H}, false, zero);
    pb.add("mtp.pre_fc_norm_hidden.weight", {H}, false, zero);
  }
  c.identity_json =
      "{\"converter\":\"ainfer_b200 synthetic writer\",\"converter_version\":\"1.0\","
      "\"created_date\":\"1970-01-01\",\"source_repo\":\"synthetic\",\"source_revision\":"
      "\"0000000000000000000000000000000000000000\",\"source_total_bytes\":0}";
  c.arch_json = cfg.to_json();
  c.tokenizer_json = "{\"format\":\"none\",\"vocab_size\":" + std::to_string(cfg.vocab) + "}";
  c.policy_json =
      "{\"default\":\"INT4 symmetric g128 BF16 scales\",\"exceptions\":[\"embed_tokens BF16\","
      "\"1-D norms source precision\",\"A_log/dt_bias/conv1d source precision\","
      "\"mlp.gate (router) BF16\",\"mlp.shared_expert_gate BF16\"],\"group_size\":128}";
  container_layout(c);
}

// ---------------------------------------------------- host synth writer ---
// Weight quantiser of the container (tools/binfer.py:76-91 of the reference).
static void quantize_group(const float *v, uint8_t *packed, uint16_t *scale) {
  float amax = 0.0f;
  for (int j = 0; j < 128; ++j) {
    float a = std::fabs(v[j]);
    amax = a > amax ? a : amax;
  }
  float sc = amax == 0.0f ? 1.0f : amax / 7.0f;
  *scale = f32_to_bf16(sc);
  for (int j = 0; j < 128; j += 2) {
    int q0 = (int)rintf(v[j] / sc), q1 = (int)rintf(v[j + 1] / sc);
    q0 = q0 < -8 ? -8 : (q0 > 7 ? 7 : q0);
    q1 = q1 < -8 ? -8 : (q1 > 7 ? 7 : q1);
    packed[j / 2] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
  }
}

void synth_fill_host(const TensorEntry &e, const SynthSpec &sp, uint64_t seed, uint8_t *payload,
                     uint8_t *scales) {
  uint64_t key = stream_key(seed, fnv1a64(e.name.c_str()));
  uint64_t n = e.numel();
  if (e.storage == DT_INT4_SYM_G128) {
    uint64_t ng = (n + 127) / 128;
    parallel_for(ng, [&](uint64_t g) {
      float v[128];
      for (int j = 0; j < 128; ++j) {
        uint64_t i = g * 128 + j;
        v[j] = i < n ? sp.std_ * normal_from_u32(draw_u32_key(key, i)) : 0.0f;
      }
      quantize_group(v, payload + g * 64, (uint16_t *)scales + g);
    });
  } else {
    uint16_t *out = (uint16_t *)payload;
    parallel_for(n, [&](uint64_t i) {
      float v = sp.std_ == 0.0f ? sp.constant : sp.std_ * normal_from_u32(draw_u32_key(key, i));
      out[i] = f32_to_bf16(v);
    });
  }
}

int synth_write_file(const char *path, const ModelConfig &cfg, uint64_t seed, std::string &err) {
  if (!cfg.check(err)) return 2;
  Container c;
  std::vector<SynthSpec> specs;
  build_plan(cfg, c, specs);
  struct Ctx { Container *c; std::vector<SynthSpec> *specs; uint64_t seed; } ctx{&c, &specs, seed};
  auto fill = [](void *user, const TensorEntry &e, uint8_t *payload, uint8_t *scales) {
    Ctx *x = (Ctx *)user;
    size_t idx = x->c->index[e.name];
    synth_fill_host(e, (*x->specs)[idx], x->seed, payload, scales);
  };
  return container_write(path, c, fill, &ctx, err);
}

// -------------------------------------------------------- device model ---
DeviceTensor DeviceModel::tensor(const std::string &name) const {
  DeviceTensor t;
  t.entry = dir.find(name);
  if (!t.entry) return t;
  t.data = (char *)pay_arena + (t.entry->d_off - dir.pay_lo);
  t.scales = t.entry->sc_bytes ? (char *)sc_arena + (t.entry->sc_off - dir.sc_lo) : nullptr;
  return t;
}

#define RT_CHECK(expr)                                                                     \
  do {                                                                                     \
    int _r = (expr);                                                                       \
    if (_r != AINFER_OK) {                                                                 \
      err = std::string("device error ") + std::to_string(_r) + " at " + __FILE__ + ":" + \
            std::to_string(__LINE__) + " (" + ainfer_last_error(dev) + ")";                \
      return 1;                                                                            \
    }                                                                                      \
  } while (0)

static int launch_simple(ainfer_device_t dev, const char *kname,
                         const std::vector<std::pair<const void *, size_t>> &args, uint32_t groups,
                         std::string &err) {
  ainfer_kernel_t k;
  RT_CHECK(ainfer_kernel_get(dev, kname, &k));
  for (size_t i = 0; i < args.size(); ++i) {
    int r = ainfer_kernel_set_arg(k, (uint32_t)i, args[i].second, args[i].first);
    if (r) { err = ainfer_last_error(dev); ainfer_kernel_release(k); return 1; }
  }
  int r = ainfer_kernel_launch(dev, k, groups);
  ainfer_kernel_release(k);
  if (r) { err = ainfer_last_error(dev); return 1; }
  return 0;
}

static int dev_alloc(DeviceModel *m, size_t bytes, void **out, std::string &err) {
  ainfer_device_t dev = m->dev;
  RT_CHECK(ainfer_mem_alloc(dev, bytes ? bytes : 16, 256, out));
  m->owned.push_back(*out);
  return 0;
}

// Widens one small BF16/FP32 tensor into a slot of a stacked fp32 mirror
// (load_small, tools/decode/decode_l0.cpp:301-316; here on the device).
static int mirror_small(DeviceModel *m, const std::string &name, float *dst, uint64_t count,
                        std::string &err) {
  ainfer_device_t dev = m->dev;
  DeviceTensor t = m->tensor(name);
  if (!t.entry) { err = "missing " + name; return 1; }
  if (t.entry->numel() != count) { err = "unexpected size of " + name; return 2; }
  if (t.entry->storage == DT_FP32) {
    RT_CHECK(ainfer_memcpy_d2d(dev, dst, t.data, count * 4));
    return 0;
  }
  if (t.entry->storage != DT_BF16) { err = "unsupported storage for small tensor " + name; return 2; }
  const void *in = t.data;
  uint32_t groups = (uint32_t)std::min<uint64_t>((count + 255) / 256, 1024);
  return launch_simple(dev, "WidenBf16", {{&dst, 8}, {&in, 8}, {&count, 8}}, groups, err);
}

int check_directory_shapes(const Container &dir, const ModelConfig &c, std::string &err) {
  const uint64_t H = c.hidden, D = c.head_dim, I = c.expert_inter, V = c.vocab;
  auto need = [&](const std::string &name, uint64_t rows, uint64_t cols, int storage) -> int {
    const TensorEntry *e = dir.find(name);
    if (!e) { err = "missing " + name; return 1; }
    if (e->storage != storage) { err = "unexpected storage of " + name; return 2; }
    // [rows][cols]; a leading dimension of 1 may be dropped (a [1][H] gate row stored as [H])
    const bool two = e->ndim == 2 && e->shape[0] == rows && e->shape[1] == cols;
    const bool one = rows == 1 && e->ndim == 1 && e->shape[0] == cols;
    if (!two && !one) { err = "unexpected shape of " + name; return 2; }
    return 0;
  };
  int r;
  if ((r = need("model.language_model.embed_tokens.weight", V, H, DT_BF16))) return r;
  if ((r = need("lm_head.weight", V, H, DT_INT4_SYM_G128))) return r;
  const int nl = c.layers + c.mtp_layers;
  for (int L = 0; L < nl; ++L) {
    const bool mtp = L >= c.layers;
    const bool attn = mtp || c.layer_types[L] == 'A';
    const std::string p = mtp ? "mtp.layers.0." : layer_prefix(L);
    if (attn) {
      if ((r = need(p + "self_attn.q_proj.weight", (uint64_t)c.q_heads * 2 * D, H, DT_INT4_SYM_G128))) return r;
      if ((r = need(p + "self_attn.k_proj.weight", (uint64_t)c.kv_heads * D, H, DT_INT4_SYM_G128))) return r;
      if ((r = need(p + "self_attn.v_proj.weight", (uint64_t)c.kv_heads * D, H, DT_INT4_SYM_G128))) return r;
      if ((r = need(p + "self_attn.o_proj.weight", H, (uint64_t)c.q_heads * D, DT_INT4_SYM_G128))) return r;
    } else {
      const uint64_t C = c.conv_dim(), VD = c.value_dim(), NV = c.lin_v_heads;
      if ((r = need(p + "linear_attn.in_proj_qkv.weight", C, H, DT_INT4_SYM_G128))) return r;
      if ((r = need(p + "linear_attn.in_proj_z.weight", VD, H, DT_INT4_SYM_G128))) return r;
      if ((r = need(p + "linear_attn.in_proj_b.weight", NV, H, DT_INT4_SYM_G128))) return r;
      if ((r = need(p + "linear_attn.in_proj_a.weight", NV, H, DT_INT4_SYM_G128))) return r;
      if ((r = need(p + "linear_attn.out_proj.weight", H, VD, DT_INT4_SYM_G128))) return r;
    }
    if ((r = need(p + "mlp.gate.weight", (uint64_t)c.experts, H, DT_BF16))) return r;
    if (c.shared_experts && (r = need(p + "mlp.shared_expert_gate.weight", 1, H, DT_BF16))) return r;
    for (int e = 0; e <= c.experts; ++e) {
      if (e == c.experts && !c.shared_experts) break;
      const std::string ep = e < c.experts ? p + "mlp.experts." + std::to_string(e) + "." : p + "mlp.shared.";
      if ((r = need(ep + "gate_proj.weight", I, H, DT_INT4_SYM_G128))) return r;
      if ((r = need(ep + "up_proj.weight", I, H, DT_INT4_SYM_G128))) return r;
      if ((r = need(ep + "down_proj.weight", H, I, DT_INT4_SYM_G128))) return r;
    }
  }
  if (c.mtp_layers && (r = need("mtp.fc.weight", H, 2 * H, DT_INT4_SYM_G128))) return r;
  return 0;
}

static int build_mirrors(DeviceModel *m, std::string &err) {
  const ModelConfig &c = m->cfg;
  ainfer_device_t dev = m->dev;
  const int H = c.hidden, D = c.head_dim, nl = c.layers + c.mtp_layers;
  const int n_attn = c.n_attn() + c.mtp_layers, n_lin = c.n_lin();
  const int C = c.conv_dim(), NV = c.lin_v_heads;
  int r;
  if ((r = dev_alloc(m, (size_t)nl * H * 4, (void **)&m->in_norm, err))) return r;
  if ((r = dev_alloc(m, (size_t)nl * H * 4, (void **)&m->post_norm, err))) return r;
  if ((r = dev_alloc(m, (size_t)std::max(1, n_attn) * D * 4, (void **)&m->q_norm, err))) return r;
  if ((r = dev_alloc(m, (size_t)std::max(1, n_attn) * D * 4, (void **)&m->k_norm, err))) return r;
  if ((r = dev_alloc(m, (size_t)std::max(1, n_lin) * c.lin_head_dim * 4, (void **)&m->lin_norm, err))) return r;
  if ((r = dev_alloc(m, (size_t)std::max(1, n_lin) * NV * 4, (void **)&m->a_log, err))) return r;
  if ((r = dev_alloc(m, (size_t)std::max(1, n_lin) * NV * 4, (void **)&m->dt_bias, err))) return r;
  if ((r = dev_alloc(m, (size_t)std::max(1, n_lin) * C * 4 * 4, (void **)&m->conv_w, err))) return r;
  if ((r = dev_alloc(m, (size_t)H * 4, (void **)&m->final_norm, err))) return r;
  if ((r = dev_alloc(m, (size_t)3 * H * 4, (void **)&m->mtp_norms, err))) return r;
  m->slot.assign(nl, 0);
  int ia = 0, il = 0;
  for (int L = 0; L < nl; ++L) {
    bool mtp = L >= c.layers;
    bool attn = mtp || c.layer_types[L] == 'A';
    std::string p = mtp ? "mtp.layers.0." : layer_prefix(L);
    m->slot[L] = attn ? ia++ : il++;
    int s = m->slot[L];
    if ((r = mirror_small(m, p + "input_layernorm.weight", m->in_norm + (size_t)L * H, H, err))) return r;
    if ((r = mirror_small(m, p + "post_attention_layernorm.weight", m->post_norm + (size_t)L * H, H, err))) return r;
    if (attn) {
      if ((r = mirror_small(m, p + "self_attn.q_norm.weight", m->q_norm + (size_t)s * D, D, err))) return r;
      if ((r = mirror_small(m, p + "self_attn.k_norm.weight", m->k_norm + (size_t)s * D, D, err))) return r;
    } else {
      if ((r = mirror_small(m, p + "linear_attn.norm.weight", m->lin_norm + (size_t)s * c.lin_head_dim, c.lin_head_dim, err))) return r;
      if ((r = mirror_small(m, p + "linear_attn.A_log", m->a_log + (size_t)s * NV, NV, err))) return r;
      if ((r = mirror_small(m, p + "linear_attn.dt_bias", m->dt_bias + (size_t)s * NV, NV, err))) return r;
      if ((r = mirror_small(m, p + "linear_attn.conv1d.weight", m->conv_w + (size_t)s * C * 4, (uint64_t)C * 4, err))) return r;
    }
  }
  if ((r = mirror_small(m, "model.language_model.norm.weight", m->final_norm, H, err))) return r;
  if (c.mtp_layers) {
    if ((r = mirror_small(m, "mtp.pre_fc_norm_embedding.weight", m->mtp_norms, H, err))) return r;
    if ((r = mirror_small(m, "mtp.pre_fc_norm_hidden.weight", m->mtp_norms + H, H, err))) return r;
    if ((r = mirror_small(m, "mtp.norm.weight", m->mtp_norms + 2 * (size_t)H, H, err))) return r;
  }
  // expert pointer tables
  const int E1 = c.experts + 1;
  std::vector<ExpertW> tab((size_t)nl * E1);
  for (int L = 0; L < nl; ++L) {
    std::string p = L >= c.layers ? "mtp.layers.0." : layer_prefix(L);
    for (int e = 0; e < E1; ++e) {
      if (e == c.experts && !c.shared_experts) { tab[(size_t)L * E1 + e] = tab[(size_t)L * E1]; continue; }
      std::string ep = e < c.experts ? p + "mlp.experts." + std::to_string(e) + "." : p + "mlp.shared.";
      DeviceTensor g = m->tensor(ep + "gate_proj.weight"), u = m->tensor(ep + "up_proj.weight"),
                   d = m->tensor(ep + "down_proj.weight");
      if (!g.entry || !u.entry || !d.entry) { err = "missing " + ep + "{gate,up,down}_proj.weight"; return 1; }
      ExpertW &w = tab[(size_t)L * E1 + e];
      w.gP = (const uint8_t *)g.data; w.gS = (const uint16_t *)g.scales;
      w.uP = (const uint8_t *)u.data; w.uS = (const uint16_t *)u.scales;
      w.dP = (const uint8_t *)d.data; w.dS = (const uint16_t *)d.scales;
    }
  }
  if ((r = dev_alloc(m, tab.size() * sizeof(ExpertW), &m->expert_tables, err))) return r;
  RT_CHECK(ainfer_memcpy_h2d(dev, m->expert_tables, tab.data(), tab.size() * sizeof(ExpertW)));
  RT_CHECK(ainfer_sync(dev, UINT64_MAX));
  return 0;
}

int model_ensure_rope(DeviceModel *m, int max_ctx, std::string &err) {
  if (max_ctx <= m->rope_ctx) return 0;
  ainfer_device_t dev = m->dev;
  const int rot = m->cfg.rotary_dim;
  // RoPE table exactly as tools/decode/decode_l0.cpp:341-349: inverse
  // frequency and angle in double, cos/sin cast to fp32, index i % (rot/2).
  std::vector<float> cs((size_t)max_ctx * rot), sn((size_t)max_ctx * rot);
  for (int t = 0; t < max_ctx; ++t)
    for (int i = 0; i < rot; ++i) {
      double inv = 1.0 / std::pow(m->cfg.rope_theta, (double)(2 * (i % (rot / 2))) / (double)rot);
      double ang = (double)t * inv;
      cs[(size_t)t * rot + i] = (float)std::cos(ang);
      sn[(size_t)t * rot + i] = (float)std::sin(ang);
    }
  void *c = nullptr, *s = nullptr;
  int r;
  if ((r = dev_alloc(m, cs.size() * 4, &c, err))) return r;
  if ((r = dev_alloc(m, sn.size() * 4, &s, err))) return r;
  RT_CHECK(ainfer_memcpy_h2d(dev, c, cs.data(), cs.size() * 4));
  RT_CHECK(ainfer_memcpy_h2d(dev, s, sn.data(), sn.size() * 4));
  m->rope_cos = (float *)c;
  m->rope_sin = (float *)s;
  m->rope_ctx = max_ctx;
  return 0;
}

static int fill_synthetic(DeviceModel *m, const std::vector<SynthSpec> &specs, std::string &err) {
  ainfer_device_t dev = m->dev;
  ainfer_device_info info;
  RT_CHECK(ainfer_device_get_info(dev, &info));
  ainfer_kernel_t k4, kb;
  RT_CHECK(ainfer_kernel_get(dev, "SynthInt4", &k4));
  RT_CHECK(ainfer_kernel_get(dev, "SynthBf16", &kb));
  for (size_t i = 0; i < m->dir.entries.size(); ++i) {
    const TensorEntry &e = m->dir.entries[i];
    DeviceTensor t = m->tensor(e.name);
    uint64_t key = stream_key(m->seed, fnv1a64(e.name.c_str()));
    if (e.storage == DT_INT4_SYM_G128) {
      uint64_t groups = (e.numel() + 127) / 128;
      float sd = specs[i].std_;
      ainfer_kernel_set_arg(k4, 0, 8, &t.data);
      ainfer_kernel_set_arg(k4, 1, 8, &t.scales);
      ainfer_kernel_set_arg(k4, 2, 8, &key);
      ainfer_kernel_set_arg(k4, 3, 8, &groups);
      ainfer_kernel_set_arg(k4, 4, 4, &sd);
      uint32_t g = (uint32_t)std::min<uint64_t>((groups + 7) / 8, (uint64_t)info.sm_count * 16);
      RT_CHECK(ainfer_kernel_launch(dev, k4, g ? g : 1));
    } else {
      uint64_t n = e.numel();
      float sd = specs[i].std_, cst = specs[i].constant;
      ainfer_kernel_set_arg(kb, 0, 8, &t.data);
      ainfer_kernel_set_arg(kb, 1, 8, &key);
      ainfer_kernel_set_arg(kb, 2, 8, &n);
      ainfer_kernel_set_arg(kb, 3, 4, &sd);
      ainfer_kernel_set_arg(kb, 4, 4, &cst);
      uint32_t g = (uint32_t)std::min<uint64_t>((n + 255) / 256, (uint64_t)info.sm_count * 16);
      RT_CHECK(ainfer_kernel_launch(dev, kb, g ? g : 1));
    }
  }
  RT_CHECK(ainfer_sync(dev, UINT64_MAX));
  ainfer_kernel_release(k4);
  ainfer_kernel_release(kb);
  return 0;
}

static int upload_file(DeviceModel *m, const char *path, std::string &err) {
  ainfer_device_t dev = m->dev;
  FILE *f = fopen(path, "rb");
  if (!f) { err = std::string("cannot open ") + path; return 2; }
  // staged upload in 256 MiB chunks through pinned memory (decode_l0.cpp:245-267)
  const size_t CH = (size_t)1 << 28;
  void *staging = nullptr;
  if (ainfer_host_alloc(dev, CH, &staging) != AINFER_OK) { fclose(f); err = "staging alloc failed"; return 1; }
  auto upspan = [&](uint64_t foff, void *arena, uint64_t len) -> int {
    uint64_t done = 0;
    while (done < len) {
      size_t c = (size_t)std::min<uint64_t>(CH, len - done);
      if (fseeko(f, (off_t)(foff + done), SEEK_SET) != 0 || fread(staging, 1, c, f) != c) {
        err = "upload failed (short read)";
        return 2;
      }
      if (ainfer_memcpy_h2d(dev, (char *)arena + done, staging, c) != AINFER_OK) {
        err = std::string("upload failed: ") + ainfer_last_error(dev);
        return 1;
      }
      done += c;
    }
    return 0;
  };
  int r = upspan(m->dir.pay_lo, m->pay_arena, m->pay_bytes);
  if (!r && m->sc_bytes) r = upspan(m->dir.sc_lo, m->sc_arena, m->sc_bytes);
  ainfer_host_free(dev, staging);
  fclose(f);
  return r;
}

int model_open(ainfer_device_t dev, const char *spec, int validate_level, DeviceModel **out,
               std::string &err) {
  *out = nullptr;
  DeviceModel *m = new DeviceModel;
  m->dev = dev;
  std::vector<SynthSpec> specs;
  std::string s = spec ? spec : "";
  int r = 0;
  if (s.rfind("synth:", 0) == 0) {
    std::string rest = s.substr(6), preset = rest;
    size_t c = rest.find(':');
    if (c != std::string::npos) {
      preset = rest.substr(0, c);
      size_t sp = rest.find("seed=");
      if (sp != std::string::npos) m->seed = std::strtoull(rest.c_str() + sp + 5, nullptr, 10);
    }
    if (!preset_config(preset, m->cfg)) { err = "unknown synthetic preset: " + preset; delete m; return 2; }
    if (!m->cfg.check(err)) { delete m; return 2; }
    build_plan(m->cfg, m->dir, specs);
    m->synthetic = true;
  } else {
    r = container_open(s.c_str(), validate_level, m->dir, err);
    if (r) { delete m; return r; }
    if (!ModelConfig::from_json(m->dir.arch_json, m->cfg, err)) { delete m; return 2; }
    // before anything is uploaded or launched: the directory must describe the model the
    // architecture section names
    r = check_directory_shapes(m->dir, m->cfg, err);
    if (r) { delete m; return r; }
  }
  m->pay_bytes = m->dir.pay_hi - m->dir.pay_lo;
  m->sc_bytes = m->dir.sc_hi - m->dir.sc_lo;
  if (ainfer_mem_alloc(dev, m->pay_bytes, 4096, &m->pay_arena) != AINFER_OK ||
      ainfer_mem_alloc(dev, m->sc_bytes ? m->sc_bytes : 16, 4096, &m->sc_arena) != AINFER_OK) {
    err = std::string("alloc failed: ") + ainfer_last_error(dev);
    model_close(m);
    return 1;
  }
  if (m->synthetic) {
    // alignment padding between payloads is defined as zero bytes
    if (ainfer_mem_fill(dev, m->pay_arena, 0, m->pay_bytes) != AINFER_OK) {
      err = ainfer_last_error(dev); model_close(m); return 1;
    }
    r = fill_synthetic(m, specs, err);
  } else {
    r = upload_file(m, s.c_str(), err);
  }
  if (!r) r = build_mirrors(m, err);
  if (r) { model_close(m); return r; }
  *out = m;
  return 0;
}

void model_close(DeviceModel *m) {
  if (!m) return;
  for (void *p : m->owned) ainfer_mem_free(m->dev, p);
  if (m->pay_arena) ainfer_mem_free(m->dev, m->pay_arena);
  if (m->sc_arena) ainfer_mem_free(m->dev, m->sc_arena);
  delete m;
}

}  // namespace ainfer
