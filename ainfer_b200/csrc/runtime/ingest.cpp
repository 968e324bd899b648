// Checkpoint ingestion: SafeTensors -> .binfer v1, the counterpart of the reference's converter
// (tools/binfer.py:60-64 policy, :76-91 quantiser, :155-353 cmd_quantize): every 2-D tensor is
// quantised to symmetric INT4 in groups of 128 with bf16 scales, except the token embedding and,
// in this runtime, the router and the shared-expert gate (kept bf16: they are read as bf16 rows by
// the router kernel); everything else keeps bf16 (fp16 / fp32 sources are rounded to bf16, the
// storage the loader widens from); tensors of the vision tower are left out, as the reference
// does. Names are kept, with the text model's Hugging Face prefixes mapped onto the container's
// ("model.layers." -> "model.language_model.layers.", "mlp.shared_expert." -> "mlp.shared.").
// The directory is checked against the architecture JSON before anything is written, so a
// checkpoint whose shapes disagree with its declared architecture is refused here and not at
// load time.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstring>

#include "../common/detmath.h"
#include "binfer.h"
#include "model.h"
#include "rt_util.h"

namespace ainfer {

namespace {

// ---- minimal JSON reader for the SafeTensors header and the shard index ----
struct JsonCursor {
  const char *p, *end;
  std::string err;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool lit(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }
  bool str(std::string &out) {
    ws();
    if (p >= end || *p != '"') { err = "expected a string"; return false; }
    ++p;
    out.clear();
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'u': out += '?'; p += 4 < end - p ? 4 : 0; break;   // names are ASCII; other code points are not needed
          default: out += *p;
        }
        ++p;
      } else {
        out += *p++;
      }
    }
    if (p >= end) { err = "unterminated string"; return false; }
    ++p;
    return true;
  }
  bool num(uint64_t &v) {
    ws();
    if (p >= end || *p < '0' || *p > '9') { err = "expected a non-negative integer"; return false; }
    v = 0;
    while (p < end && *p >= '0' && *p <= '9') v = v * 10 + (uint64_t)(*p++ - '0');
    return true;
  }
  bool skip() {   // any value
    ws();
    if (p >= end) return false;
    if (*p == '"') { std::string s; return str(s); }
    if (*p == '{' || *p == '[') {
      const char open = *p, close = open == '{' ? '}' : ']';
      ++p;
      if (lit(close)) return true;
      do {
        if (open == '{') { std::string k; if (!str(k) || !lit(':')) return false; }
        if (!skip()) return false;
      } while (lit(','));
      return lit(close);
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;
    return true;
  }
};

struct SrcTensor {
  std::string name, dtype;
  std::vector<uint64_t> shape;
  const uint8_t *data = nullptr;
  uint64_t bytes = 0;
};

struct Shard {
  int fd = -1;
  const uint8_t *map = nullptr;
  size_t size = 0;
  ~Shard() {
    if (map) munmap((void *)map, size);
    if (fd >= 0) close(fd);
  }
};

bool open_shard(const std::string &path, Shard &s, std::vector<SrcTensor> &out, std::string &err) {
  s.fd = open(path.c_str(), O_RDONLY);
  struct stat st;
  if (s.fd < 0 || fstat(s.fd, &st) != 0) { err = "cannot open " + path; return false; }
  s.size = (size_t)st.st_size;
  if (s.size < 8) { err = path + ": too short for a SafeTensors header"; return false; }
  s.map = (const uint8_t *)mmap(nullptr, s.size, PROT_READ, MAP_PRIVATE, s.fd, 0);
  if (s.map == MAP_FAILED) { s.map = nullptr; err = "cannot map " + path; return false; }
  uint64_t hl;
  std::memcpy(&hl, s.map, 8);
  if (hl > s.size - 8) { err = path + ": header length exceeds the file"; return false; }
  const uint8_t *base = s.map + 8 + hl;
  const uint64_t data_bytes = s.size - 8 - hl;
  JsonCursor c{(const char *)s.map + 8, (const char *)s.map + 8 + hl, ""};
  if (!c.lit('{')) { err = path + ": header is not a JSON object"; return false; }
  if (c.lit('}')) return true;
  do {
    std::string key;
    if (!c.str(key) || !c.lit(':')) { err = path + ": bad header (" + c.err + ")"; return false; }
    if (key == "__metadata__") { if (!c.skip()) { err = path + ": bad metadata"; return false; } continue; }
    SrcTensor t;
    t.name = key;
    uint64_t a = 0, b = 0;
    bool have_off = false;
    if (!c.lit('{')) { err = path + ": bad entry for " + key; return false; }
    do {
      std::string f;
      if (!c.str(f) || !c.lit(':')) { err = path + ": bad entry for " + key; return false; }
      if (f == "dtype") { if (!c.str(t.dtype)) { err = path + ": bad dtype of " + key; return false; } }
      else if (f == "shape") {
        if (!c.lit('[')) { err = path + ": bad shape of " + key; return false; }
        if (!c.lit(']')) {
          do { uint64_t d; if (!c.num(d)) { err = path + ": bad shape of " + key; return false; } t.shape.push_back(d); } while (c.lit(','));
          if (!c.lit(']')) { err = path + ": bad shape of " + key; return false; }
        }
      } else if (f == "data_offsets") {
        if (!c.lit('[') || !c.num(a) || !c.lit(',') || !c.num(b) || !c.lit(']')) { err = path + ": bad data_offsets of " + key; return false; }
        have_off = true;
      } else if (!c.skip()) { err = path + ": bad entry for " + key; return false; }
    } while (c.lit(','));
    if (!c.lit('}') || !have_off) { err = path + ": bad entry for " + key; return false; }
    if (a > b || b > data_bytes) { err = path + ": data_offsets of " + key + " lie outside the file"; return false; }
    t.data = base + a;
    t.bytes = b - a;
    out.push_back(t);
  } while (c.lit(','));
  if (!c.lit('}')) { err = path + ": bad header end"; return false; }
  return true;
}

int elem_bytes(const std::string &dt) { return dt == "BF16" || dt == "F16" ? 2 : (dt == "F32" ? 4 : 0); }

float load_elem(const SrcTensor &t, int eb, uint64_t i) {
  if (eb == 4) { float v; std::memcpy(&v, t.data + i * 4, 4); return v; }
  uint16_t h;
  std::memcpy(&h, t.data + i * 2, 2);
  if (t.dtype == "BF16") return bf16_to_f32(h);
  // IEEE half -> float
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
  uint32_t u;
  if (e == 0) {
    if (m == 0) u = sign;
    else { int sh = 0; uint32_t mm = m; while (!(mm & 0x400u)) { mm <<= 1; ++sh; } u = sign | ((uint32_t)(113 - sh) << 23) | ((mm & 0x3FFu) << 13); }
  } else if (e == 31) u = sign | 0x7F800000u | (m << 13);
  else u = sign | ((e + 112) << 23) | (m << 13);
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

std::string canonical_name(std::string n) {
  auto sub = [&](const char *from, const char *to) {
    size_t at = n.find(from);
    if (at != std::string::npos) n.replace(at, std::strlen(from), to);
  };
  if (n.rfind("model.layers.", 0) == 0) n = "model.language_model." + n.substr(6);
  else if (n.rfind("model.embed_tokens.", 0) == 0 || n.rfind("model.norm.", 0) == 0) n = "model.language_model." + n.substr(6);
  sub(".mlp.shared_expert.", ".mlp.shared.");
  return n;
}

bool ends_with(const std::string &s, const char *suf) {
  const size_t n = std::strlen(suf);
  return s.size() >= n && s.compare(s.size() - n, n, suf) == 0;
}

// Weight quantiser of the container (tools/binfer.py:76-91 of the reference).
void quantize_group128(const float *v, uint8_t *packed, uint16_t *scale) {
  float amax = 0.0f;
  for (int j = 0; j < 128; ++j) {
    const float a = std::fabs(v[j]);
    amax = a > amax ? a : amax;
  }
  const float sc = amax == 0.0f ? 1.0f : amax / 7.0f;
  *scale = f32_to_bf16(sc);
  for (int j = 0; j < 128; j += 2) {
    int q0 = (int)rintf(v[j] / sc), q1 = (int)rintf(v[j + 1] / sc);
    q0 = q0 < -8 ? -8 : (q0 > 7 ? 7 : q0);
    q1 = q1 < -8 ? -8 : (q1 > 7 ? 7 : q1);
    packed[j / 2] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
  }
}

}  // namespace

int binfer_from_safetensors(const char *src, const char *arch_json, const char *out_path, std::string &err) {
  if (!src || !arch_json || !out_path) { err = "usage: source, architecture JSON and output path are required"; return 2; }
  // ---- the shards ----
  std::vector<std::string> files;
  struct stat st;
  if (stat(src, &st) != 0) { err = std::string("cannot open ") + src; return 2; }
  if (S_ISDIR(st.st_mode)) {
    const std::string dir = src, idx = dir + "/model.safetensors.index.json";
    FILE *f = std::fopen(idx.c_str(), "rb");
    if (f) {
      std::string js;
      char buf[65536];
      size_t n;
      while ((n = std::fread(buf, 1, sizeof buf, f)) > 0) js.append(buf, n);
      std::fclose(f);
      // "weight_map": {"tensor": "shard file", ...}
      size_t at = js.find("\"weight_map\"");
      if (at == std::string::npos) { err = idx + ": no weight_map"; return 2; }
      JsonCursor c{js.data() + at + 12, js.data() + js.size(), ""};
      if (!c.lit(':') || !c.lit('{')) { err = idx + ": bad weight_map"; return 2; }
      if (!c.lit('}')) {
        do {
          std::string k, v;
          if (!c.str(k) || !c.lit(':') || !c.str(v)) { err = idx + ": bad weight_map"; return 2; }
          if (std::find(files.begin(), files.end(), dir + "/" + v) == files.end()) files.push_back(dir + "/" + v);
        } while (c.lit(','));
      }
    } else {
      files.push_back(dir + "/model.safetensors");
    }
  } else {
    files.push_back(src);
  }
  std::vector<Shard> shards(files.size());
  std::vector<SrcTensor> srcs;
  for (size_t i = 0; i < files.size(); ++i)
    if (!open_shard(files[i], shards[i], srcs, err)) return 2;
  // ---- the plan: names sorted, vision tower left out, policy per tensor ----
  ModelConfig cfg;
  if (!ModelConfig::from_json(arch_json, cfg, err) || !cfg.check(err)) return 2;
  std::vector<std::pair<std::string, const SrcTensor *>> plan;
  for (const SrcTensor &t : srcs) {
    if (t.name.find("visual") != std::string::npos) continue;
    plan.emplace_back(canonical_name(t.name), &t);
  }
  std::sort(plan.begin(), plan.end(), [](const auto &a, const auto &b) { return a.first < b.first; });
  Container c;
  std::vector<const SrcTensor *> by_entry;
  for (auto &pr : plan) {
    const SrcTensor &t = *pr.second;
    const int eb = elem_bytes(t.dtype);
    if (!eb) { err = "unsupported source dtype " + t.dtype + " for " + t.name; return 2; }
    if (pr.first.size() > 63) { err = "tensor name longer than 63 bytes: " + pr.first; return 2; }
    if (t.shape.empty() || t.shape.size() > 8) { err = "unsupported rank for " + t.name; return 2; }
    if (c.index.count(pr.first)) { err = "duplicate tensor " + pr.first; return 2; }
    TensorEntry e;
    e.name = pr.first;
    e.ndim = (int)t.shape.size();
    uint64_t n = 1;
    for (int i = 0; i < e.ndim; ++i) { e.shape[i] = t.shape[i]; n *= t.shape[i]; }
    if (n * (uint64_t)eb != t.bytes) { err = "payload size does not match shape: " + t.name; return 2; }
    const bool keep = e.ndim != 2 || ends_with(e.name, "embed_tokens.weight") || ends_with(e.name, "mlp.gate.weight") ||
                      ends_with(e.name, "shared_expert_gate.weight");
    e.logical = DT_BF16;
    if (keep) {
      e.storage = DT_BF16;
      e.d_bytes = n * 2;
    } else {
      if (e.shape[1] % 128) { err = "row length is not a multiple of the quantiser's group of 128: " + t.name; return 2; }
      e.storage = DT_INT4_SYM_G128;
      e.group = 128;
      e.sc_bytes = n / 128 * 2;
      e.d_bytes = n / 2;
    }
    c.index[e.name] = c.entries.size();
    c.entries.push_back(e);
    by_entry.push_back(&t);
  }
  c.identity_json = std::string("{\"converter\":\"ainfer_b200 SafeTensors converter\",\"converter_version\":\"1.0\",") +
                    "\"created_date\":\"1970-01-01\",\"source_repo\":\"local\",\"source_revision\":" +
                    "\"0000000000000000000000000000000000000000\",\"source_total_bytes\":0}";
  c.arch_json = cfg.to_json();
  c.tokenizer_json = "{\"format\":\"none\",\"vocab_size\":" + std::to_string(cfg.vocab) + "}";
  c.policy_json =
      "{\"default\":\"INT4 symmetric g128 BF16 scales\",\"exceptions\":[\"embed_tokens BF16\","
      "\"1-D norms source precision\",\"A_log/dt_bias/conv1d source precision\","
      "\"mlp.gate (router) BF16\",\"mlp.shared_expert_gate BF16\"],\"group_size\":128}";
  container_layout(c);
  int r = check_directory_shapes(c, cfg, err);   // every tensor the runtime will read, with its shape and storage
  if (r) return r;
  struct Ctx { Container *c; std::vector<const SrcTensor *> *src; } ctx{&c, &by_entry};
  auto fill = [](void *user, const TensorEntry &e, uint8_t *payload, uint8_t *scales) {
    Ctx *x = (Ctx *)user;
    const SrcTensor &t = *(*x->src)[x->c->index[e.name]];
    const int eb = elem_bytes(t.dtype);
    const uint64_t n = e.numel();
    if (e.storage == DT_INT4_SYM_G128) {
      parallel_for(n / 128, [&](uint64_t g) {
        float v[128];
        for (int j = 0; j < 128; ++j) v[j] = load_elem(t, eb, g * 128 + j);
        quantize_group128(v, payload + g * 64, (uint16_t *)scales + g);
      });
    } else if (t.dtype == "BF16") {
      std::memcpy(payload, t.data, n * 2);
    } else {
      uint16_t *out = (uint16_t *)payload;
      parallel_for(n, [&](uint64_t i) { out[i] = f32_to_bf16(load_elem(t, eb, i)); });
    }
  };
  return container_write(out_path, c, fill, &ctx, err);
}

}  // namespace ainfer
