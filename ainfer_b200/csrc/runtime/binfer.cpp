#include "binfer.h"

#include <unistd.h>

#include <algorithm>
#include <cstring>

namespace ainfer {

static const unsigned char kMagic[8] = {'B', 'I', 'N', 'F', 'E', 'R', 0, 1};

uint32_t crc32_update(uint32_t crc, const void *data, size_t n) {
  static uint32_t table[8][256];
  static bool init = false;
  if (!init) {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
      table[0][i] = c;
    }
    for (uint32_t i = 0; i < 256; ++i)
      for (int t = 1; t < 8; ++t) table[t][i] = (table[t - 1][i] >> 8) ^ table[0][table[t - 1][i] & 0xFF];
    init = true;
  }
  const uint8_t *p = (const uint8_t *)data;
  crc = ~crc;
  while (n >= 8) {  // slicing-by-8
    uint32_t a, b;
    std::memcpy(&a, p, 4);
    std::memcpy(&b, p + 4, 4);
    a ^= crc;
    crc = table[7][a & 0xFF] ^ table[6][(a >> 8) & 0xFF] ^ table[5][(a >> 16) & 0xFF] ^
          table[4][a >> 24] ^ table[3][b & 0xFF] ^ table[2][(b >> 8) & 0xFF] ^
          table[1][(b >> 16) & 0xFF] ^ table[0][b >> 24];
    p += 8;
    n -= 8;
  }
  while (n--) crc = table[0][(crc ^ *p++) & 0xFF] ^ (crc >> 8);
  return ~crc;
}

// ------------------------------------------------------------- SHA-256 ---
static const uint32_t kSha[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
static inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
static void sha_block(uint32_t h[8], const uint8_t *p) {
  uint32_t w[64];
  for (int i = 0; i < 16; ++i)
    w[i] = ((uint32_t)p[4 * i] << 24) | ((uint32_t)p[4 * i + 1] << 16) | ((uint32_t)p[4 * i + 2] << 8) |
           p[4 * i + 3];
  for (int i = 16; i < 64; ++i) {
    uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
    uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
    w[i] = w[i - 16] + s0 + w[i - 7] + s1;
  }
  uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
  for (int i = 0; i < 64; ++i) {
    uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
    uint32_t ch = (e & f) ^ (~e & g);
    uint32_t t1 = hh + S1 + ch + kSha[i] + w[i];
    uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
    uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
    uint32_t t2 = S0 + mj;
    hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
  }
  h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
}
Sha256::Sha256() {
  static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                                   0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  std::memcpy(h, init, sizeof h);
}
void Sha256::update(const void *data, size_t n) {
  const uint8_t *p = (const uint8_t *)data;
  len += n;
  if (fill) {
    size_t take = std::min(n, (size_t)64 - fill);
    std::memcpy(buf + fill, p, take);
    fill += take; p += take; n -= take;
    if (fill == 64) { sha_block(h, buf); fill = 0; }
  }
  while (n >= 64) { sha_block(h, p); p += 64; n -= 64; }
  if (n) { std::memcpy(buf, p, n); fill = n; }
}
void Sha256::final(uint8_t out[32]) {
  uint64_t bits = len * 8;
  uint8_t pad = 0x80;
  update(&pad, 1);
  uint8_t z = 0;
  while (fill != 56) update(&z, 1);
  uint8_t lb[8];
  for (int i = 0; i < 8; ++i) lb[i] = (uint8_t)(bits >> (56 - 8 * i));
  update(lb, 8);
  for (int i = 0; i < 8; ++i) {
    out[4 * i] = (uint8_t)(h[i] >> 24); out[4 * i + 1] = (uint8_t)(h[i] >> 16);
    out[4 * i + 2] = (uint8_t)(h[i] >> 8); out[4 * i + 3] = (uint8_t)h[i];
  }
}

// -------------------------------------------------------------- reader ---
template <typename T>
static T rd(const uint8_t *p) { T v; std::memcpy(&v, p, sizeof v); return v; }
template <typename T>
static void wr(std::vector<uint8_t> &b, T v) {
  const uint8_t *p = (const uint8_t *)&v;
  b.insert(b.end(), p, p + sizeof v);
}

static bool read_at(FILE *f, uint64_t off, void *dst, size_t n) {
  if (fseeko(f, (off_t)off, SEEK_SET) != 0) return false;
  return fread(dst, 1, n, f) == n;
}

static void compute_spans(Container &c) {
  c.pay_lo = c.sc_lo = UINT64_MAX;
  c.pay_hi = c.sc_hi = 0;
  for (auto &e : c.entries) {
    c.pay_lo = std::min(c.pay_lo, e.d_off);
    c.pay_hi = std::max(c.pay_hi, e.d_off + e.d_bytes);
    if (e.sc_bytes) {
      c.sc_lo = std::min(c.sc_lo, e.sc_off);
      c.sc_hi = std::max(c.sc_hi, e.sc_off + e.sc_bytes);
    }
  }
  if (c.sc_hi == 0) c.sc_lo = 0;
  if (c.pay_hi == 0) c.pay_lo = 0;
}

int container_open(const char *path, int level, Container &c, std::string &err) {
  FILE *f = fopen(path, "rb");
  if (!f) { err = std::string("cannot open ") + path; return 2; }
  struct Closer { FILE *f; ~Closer() { fclose(f); } } closer{f};
  fseeko(f, 0, SEEK_END);
  uint64_t size = (uint64_t)ftello(f);
  c = Container();
  c.file_bytes = size;
  uint8_t hdr[128];
  if (size < 128 + 32 || !read_at(f, 0, hdr, 128)) { err = "unparseable/truncated: shorter than the header"; return 2; }
  if (std::memcmp(hdr, kMagic, 8) != 0) { err = "bad magic (not a .binfer file)"; return 2; }
  if (rd<uint32_t>(hdr + 8) != 1) { err = "bad version"; return 2; }
  if (rd<uint32_t>(hdr + 12) & ~1u) { err = "reserved flags set"; return 2; }
  uint64_t n = rd<uint64_t>(hdr + 16), table_off = rd<uint64_t>(hdr + 24);
  uint32_t scount = rd<uint32_t>(hdr + 32);
  if (rd<uint32_t>(hdr + 36) != 64) { err = "bad alignment field"; return 2; }
  uint64_t total = rd<uint64_t>(hdr + 40);
  if (total != size) {
    err = "total mismatch header=" + std::to_string(total) + " actual=" + std::to_string(size);
    return 2;
  }
  if (scount > 64 || table_off + (uint64_t)scount * 32 > size - 32) { err = "section table out of range"; return 2; }
  std::vector<uint8_t> table((size_t)scount * 32);
  if (!read_at(f, table_off, table.data(), table.size())) { err = "unparseable/truncated: section table"; return 2; }
  uint64_t dir_off = 0, dir_bytes = 0;
  uint32_t dir_crc = 0;
  bool seen[6] = {false, false, false, false, false, false};
  for (uint32_t i = 0; i < scount; ++i) {
    const uint8_t *e = table.data() + i * 32;
    uint32_t sid = rd<uint32_t>(e);
    uint64_t off = rd<uint64_t>(e + 4), nb = rd<uint64_t>(e + 12);
    uint32_t crc = rd<uint32_t>(e + 20);
    if (off > size - 32 || nb > size - 32 - off) { err = "section " + std::to_string(sid) + " out of range"; return 2; }
    if (sid >= 1 && sid <= 5) seen[sid] = true;
    if (sid == 5) { dir_off = off; dir_bytes = nb; dir_crc = crc; continue; }
    if (nb < 8) { err = "section " + std::to_string(sid) + " length implausible"; return 2; }
    std::vector<uint8_t> body(nb);
    if (!read_at(f, off, body.data(), nb)) { err = "unparseable/truncated: section body"; return 2; }
    uint64_t ln = rd<uint64_t>(body.data());
    if (ln > nb - 8) { err = "section " + std::to_string(sid) + " length implausible"; return 2; }
    if (level >= VALIDATE_SECTIONS && crc32_of(body.data(), 8 + ln) != crc) {
      err = "section " + std::to_string(sid) + " CRC mismatch";
      return 2;
    }
    std::string s((const char *)body.data() + 8, ln);
    if (sid == 1) c.identity_json = s;
    else if (sid == 2) c.arch_json = s;
    else if (sid == 3) c.tokenizer_json = s;
    else if (sid == 4) c.policy_json = s;
  }
  for (int sid = 1; sid <= 5; ++sid)
    if (!seen[sid]) { err = "missing section " + std::to_string(sid); return 2; }
  if (dir_bytes != n * 192) { err = "dir size mismatch"; return 2; }
  std::vector<uint8_t> dir(dir_bytes);
  if (!read_at(f, dir_off, dir.data(), dir_bytes)) { err = "truncated dir"; return 2; }
  if (level >= VALIDATE_SECTIONS && crc32_of(dir.data(), dir_bytes) != dir_crc) {
    err = "section 5 (dir) CRC mismatch";
    return 2;
  }
  c.entries.resize(n);
  for (uint64_t i = 0; i < n; ++i) {
    const uint8_t *e = dir.data() + i * 192;
    TensorEntry &t = c.entries[i];
    char name[65];
    std::memcpy(name, e, 64);
    name[64] = 0;
    t.name = name;
    t.ndim = e[64];
    if (t.ndim > 8) { err = "bad ndim: " + t.name; return 2; }
    for (int d = 0; d < 8; ++d) t.shape[d] = rd<uint64_t>(e + 72 + 8 * d);
    t.logical = e[136];
    t.storage = e[137];
    t.layout = rd<uint16_t>(e + 138);
    t.group = rd<uint32_t>(e + 140);
    t.sc_off = rd<uint64_t>(e + 144);
    t.sc_bytes = rd<uint64_t>(e + 152);
    t.d_off = rd<uint64_t>(e + 160);
    t.d_bytes = rd<uint64_t>(e + 168);
    t.crc = rd<uint32_t>(e + 176);
    if (c.index.count(t.name)) { err = "duplicate names: " + t.name; return 2; }
    c.index[t.name] = i;
    if (t.layout != 0) { err = "unsupported layout_id: " + t.name; return 2; }
    if (t.storage > DT_FP8_E4M3) { err = "unsupported dtype enum: " + t.name; return 2; }
    if (t.d_bytes == 0 || t.d_off > size - 32 || t.d_bytes > size - 32 - t.d_off) {
      err = "payload span out of range: " + t.name;
      return 2;
    }
    if (t.sc_bytes && (t.sc_off > size - 32 || t.sc_bytes > size - 32 - t.sc_off)) {
      err = "scale span out of range: " + t.name;
      return 2;
    }
    if (t.name.find(".visual.") != std::string::npos || t.name.find(".merger.") != std::string::npos ||
        t.name.find("patch_embed") != std::string::npos || t.name.find("pos_embed") != std::string::npos) {
      err = "visual tensor present: " + t.name;
      return 2;
    }
    if (t.storage == DT_INT4_SYM_G128) {
      uint64_t ng = (t.numel() + 127) / 128;
      if (t.group != 128 || t.sc_bytes != ng * 2) { err = "bad quant params " + t.name; return 2; }
      if (t.d_bytes != ng * 64) { err = "bad packed size " + t.name; return 2; }
    } else if (t.storage == DT_BF16 || t.storage == DT_FP16 || t.storage == DT_FP32) {
      // a payload shorter than its shape would make every reader of the tensor run past it
      const uint64_t elem = t.storage == DT_FP32 ? 4 : 2;
      if (t.d_bytes != t.numel() * elem) { err = "payload size does not match shape: " + t.name; return 2; }
    }
  }
  compute_spans(c);
  if (level >= VALIDATE_SECTIONS) {
    struct Span { uint64_t a, b; const std::string *n; };
    std::vector<Span> spans;
    for (auto &e : c.entries) {
      spans.push_back({e.d_off, e.d_off + e.d_bytes, &e.name});
      if (e.sc_bytes) spans.push_back({e.sc_off, e.sc_off + e.sc_bytes, &e.name});
    }
    std::sort(spans.begin(), spans.end(), [](const Span &x, const Span &y) { return x.a < y.a; });
    for (size_t i = 1; i < spans.size(); ++i)
      if (spans[i].a < spans[i - 1].b) {
        err = "overlap " + *spans[i - 1].n + " vs " + *spans[i].n;
        return 2;
      }
  }
  if (level >= VALIDATE_FULL) {
    std::vector<uint8_t> buf(1 << 22);
    for (auto &e : c.entries) {
      uint32_t crc = 0;
      uint64_t left = e.d_bytes, off = e.d_off;
      while (left) {
        size_t ch = (size_t)std::min<uint64_t>(left, buf.size());
        if (!read_at(f, off, buf.data(), ch)) { err = "payload CRC " + e.name; return 2; }
        crc = crc32_update(crc, buf.data(), ch);
        left -= ch; off += ch;
      }
      if (crc != e.crc) { err = "payload CRC " + e.name; return 2; }
    }
    Sha256 sha;
    uint64_t left = size - 32, off = 0;
    while (left) {
      size_t ch = (size_t)std::min<uint64_t>(left, buf.size());
      if (!read_at(f, off, buf.data(), ch)) { err = "unparseable/truncated: body"; return 2; }
      sha.update(buf.data(), ch);
      left -= ch; off += ch;
    }
    uint8_t dg[32], tail[32];
    sha.final(dg);
    if (!read_at(f, size - 32, tail, 32) || std::memcmp(dg, tail, 32) != 0) {
      err = "trailing sha256 mismatch";
      return 2;
    }
  }
  return 0;
}

// -------------------------------------------------------------- writer ---
static uint64_t align_up(uint64_t n) { return (n + 63) / 64 * 64; }

void container_layout(Container &c) {
  const std::string *blobs[4] = {&c.identity_json, &c.arch_json, &c.tokenizer_json, &c.policy_json};
  uint64_t off = align_up(128 + 5 * 32);
  for (int i = 0; i < 4; ++i) off = align_up(off + 8 + blobs[i]->size());
  off = align_up(off + c.entries.size() * 192);  // directory
  uint64_t scale_off = off, scale_total = 0;
  for (auto &e : c.entries) scale_total += e.sc_bytes;
  off = align_up(off + scale_total);
  uint64_t data_off = off;
  c.index.clear();
  for (size_t i = 0; i < c.entries.size(); ++i) {
    TensorEntry &e = c.entries[i];
    e.sc_off = e.sc_bytes ? scale_off : 0;
    scale_off += e.sc_bytes;
    e.d_off = data_off;
    data_off = align_up(data_off + e.d_bytes);
    c.index[e.name] = i;
  }
  c.file_bytes = data_off + 32;
  compute_spans(c);
}

static void put_entry(std::vector<uint8_t> &b, const TensorEntry &e) {
  size_t start = b.size();
  b.resize(start + 192, 0);
  uint8_t *p = b.data() + start;
  std::memcpy(p, e.name.c_str(), std::min<size_t>(e.name.size(), 63));
  p[64] = (uint8_t)e.ndim;
  for (int d = 0; d < 8; ++d) std::memcpy(p + 72 + 8 * d, &e.shape[d], 8);
  p[136] = e.logical;
  p[137] = e.storage;
  std::memcpy(p + 138, &e.layout, 2);
  std::memcpy(p + 140, &e.group, 4);
  std::memcpy(p + 144, &e.sc_off, 8);
  std::memcpy(p + 152, &e.sc_bytes, 8);
  std::memcpy(p + 160, &e.d_off, 8);
  std::memcpy(p + 168, &e.d_bytes, 8);
  std::memcpy(p + 176, &e.crc, 4);
}

int container_write(const char *path, Container &c, FillFn fill, void *user, std::string &err) {
  for (auto &e : c.entries)
    if (e.name.size() > 63) { err = "tensor name longer than 63 bytes: " + e.name; return 2; }
  container_layout(c);
  FILE *f = fopen(path, "wb+");
  if (!f) { err = std::string("cannot create ") + path; return 2; }
  const std::string *blobs[4] = {&c.identity_json, &c.arch_json, &c.tokenizer_json, &c.policy_json};
  // header
  std::vector<uint8_t> head;
  head.insert(head.end(), kMagic, kMagic + 8);
  wr<uint32_t>(head, 1); wr<uint32_t>(head, 1);
  wr<uint64_t>(head, c.entries.size()); wr<uint64_t>(head, 128);
  wr<uint32_t>(head, 5); wr<uint32_t>(head, 64);
  wr<uint64_t>(head, c.file_bytes);
  head.resize(128, 0);
  // section table
  uint64_t off = align_up(128 + 5 * 32);
  uint64_t sec_off[5], sec_bytes[5];
  for (int i = 0; i < 4; ++i) {
    sec_off[i] = off; sec_bytes[i] = 8 + blobs[i]->size();
    off = align_up(off + sec_bytes[i]);
  }
  sec_off[4] = off; sec_bytes[4] = c.entries.size() * 192;
  for (int i = 0; i < 4; ++i) {
    std::vector<uint8_t> body;
    wr<uint64_t>(body, blobs[i]->size());
    body.insert(body.end(), blobs[i]->begin(), blobs[i]->end());
    wr<uint32_t>(head, i + 1); wr<uint64_t>(head, sec_off[i]); wr<uint64_t>(head, sec_bytes[i]);
    wr<uint32_t>(head, crc32_of(body.data(), body.size())); wr<uint32_t>(head, 0); wr<uint32_t>(head, 0);
  }
  wr<uint32_t>(head, 5); wr<uint64_t>(head, sec_off[4]); wr<uint64_t>(head, sec_bytes[4]);
  wr<uint32_t>(head, 0); wr<uint32_t>(head, 0); wr<uint32_t>(head, 0);
  head.resize(align_up(head.size()), 0);
  for (int i = 0; i < 4; ++i) {
    if (head.size() != sec_off[i]) { err = "internal: section offset"; fclose(f); return 3; }
    wr<uint64_t>(head, blobs[i]->size());
    head.insert(head.end(), blobs[i]->begin(), blobs[i]->end());
    head.resize(align_up(head.size()), 0);
  }
  fwrite(head.data(), 1, head.size(), f);
  // zero-fill the directory, the scale pool and everything up to the end
  // (sparse-friendly: payloads are written at their offsets below)
  if (ftruncate(fileno(f), (off_t)(c.file_bytes - 32)) != 0) { err = "ftruncate failed"; fclose(f); return 2; }
  // payloads + scales
  std::vector<uint8_t> pay, sc;
  for (auto &e : c.entries) {
    pay.assign(e.d_bytes, 0);
    sc.assign(e.sc_bytes, 0);
    fill(user, e, pay.data(), sc.data());
    e.crc = crc32_of(pay.data(), pay.size());
    fseeko(f, (off_t)e.d_off, SEEK_SET);
    fwrite(pay.data(), 1, pay.size(), f);
    if (e.sc_bytes) {
      fseeko(f, (off_t)e.sc_off, SEEK_SET);
      fwrite(sc.data(), 1, sc.size(), f);
    }
  }
  // directory + its CRC
  std::vector<uint8_t> dir;
  dir.reserve(c.entries.size() * 192);
  for (auto &e : c.entries) put_entry(dir, e);
  fseeko(f, (off_t)sec_off[4], SEEK_SET);
  fwrite(dir.data(), 1, dir.size(), f);
  uint32_t dcrc = crc32_of(dir.data(), dir.size());
  fseeko(f, 128 + 4 * 32 + 20, SEEK_SET);
  fwrite(&dcrc, 4, 1, f);
  // trailing SHA-256 over everything before it
  fflush(f);
  fseeko(f, 0, SEEK_SET);
  Sha256 sha;
  std::vector<uint8_t> buf(1 << 22);
  uint64_t left = c.file_bytes - 32;
  while (left) {
    size_t ch = (size_t)std::min<uint64_t>(left, buf.size());
    if (fread(buf.data(), 1, ch, f) != ch) { err = "read-back failed"; fclose(f); return 2; }
    sha.update(buf.data(), ch);
    left -= ch;
  }
  uint8_t dg[32];
  sha.final(dg);
  fseeko(f, (off_t)(c.file_bytes - 32), SEEK_SET);
  fwrite(dg, 1, 32, f);
  bool bad = ferror(f) != 0;
  fclose(f);
  if (bad) { err = "write failed"; return 2; }
  return 0;
}

}  // namespace ainfer
