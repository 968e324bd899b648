// .binfer v1 container: reader, validator and writer.
// Format: docs/binfer_spec.md of the reference (128-byte header, section table
// of 32-byte entries with CRC-32, sections 1-4 as length-prefixed JSON blobs,
// section 5 = raw 192-byte directory entries, scale pool, 64-byte aligned
// payloads, trailing SHA-256). Writer layout follows tools/binfer.py:155-353,
// validation follows tools/binfer.py:397-499 and the span checks of
// tools/decode/decode_l0.cpp:127-189.
#pragma once
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

namespace ainfer {

enum StorageDtype : uint8_t {
  DT_BF16 = 0, DT_FP16 = 1, DT_FP32 = 2, DT_INT4_SYM_G128 = 3, DT_INT8 = 4, DT_FP8_E4M3 = 5
};

struct TensorEntry {
  std::string name;
  int ndim = 0;
  uint64_t shape[8] = {0};
  uint8_t logical = DT_BF16, storage = DT_BF16;
  uint16_t layout = 0;
  uint32_t group = 0;
  uint64_t sc_off = 0, sc_bytes = 0, d_off = 0, d_bytes = 0;
  uint32_t crc = 0;
  uint64_t numel() const {
    uint64_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= shape[i];
    return n;
  }
};

struct Container {
  uint64_t file_bytes = 0;
  std::string identity_json, arch_json, tokenizer_json, policy_json;
  std::vector<TensorEntry> entries;
  std::map<std::string, size_t> index;
  uint64_t pay_lo = 0, pay_hi = 0, sc_lo = 0, sc_hi = 0;  // spans over all entries
  const TensorEntry *find(const std::string &name) const {
    auto it = index.find(name);
    return it == index.end() ? nullptr : &entries[it->second];
  }
};

uint32_t crc32_update(uint32_t crc, const void *data, size_t n);
inline uint32_t crc32_of(const void *data, size_t n) { return crc32_update(0, data, n); }

struct Sha256 {
  uint32_t h[8];
  uint64_t len = 0;
  uint8_t buf[64];
  size_t fill = 0;
  Sha256();
  void update(const void *data, size_t n);
  void final(uint8_t out[32]);
};

enum ValidateLevel {
  VALIDATE_SPANS = 0,     // header, section table, directory, span checks (the runtime loader's checks)
  VALIDATE_SECTIONS = 1,  // + section CRCs, quant-parameter consistency, overlap
  VALIDATE_FULL = 2       // + payload CRCs and trailing SHA-256 (spec section 11)
};

// Parses and validates. Returns 0 on success; on failure returns 2 (the
// reference's exit code for a bad container) and fills err with the first
// failure, worded as the reference words it where it has a message.
int container_open(const char *path, int level, Container &out, std::string &err);

// Directory + layout computation shared by the file writer and the in-memory
// synthetic loader: assigns scale-pool and payload offsets exactly as the
// reference writer does (header 128 B, 5 table entries, sections 64-aligned,
// directory, scale pool in entry order, payloads in entry order each
// 64-aligned, 32-byte trailer).
void container_layout(Container &c);

// Streaming writer: header/sections/directory are written first with
// placeholder CRCs; payloads and scales are supplied tensor by tensor in entry
// order through the callback; directory CRCs, section-5 CRC and the trailing
// SHA-256 are patched at the end.
typedef void (*FillFn)(void *user, const TensorEntry &e, uint8_t *payload, uint8_t *scales);
int container_write(const char *path, Container &c, FillFn fill, void *user, std::string &err);

}  // namespace ainfer
