// Problem lists that cover the rows of one row-batched GEMM in slabs of eight rows, for
// Int4GemvA8MultiGrouped (the dp4a kernel that streams a tile of weights once for up to eight
// rows). With 9 rows or more the tensor-core GEMM (Int4GemmA8Tc, at most 64 rows a launch) spends about 2 us per group of 128
// input columns whatever the number of its output rows, so a matrix of few output rows is one or a
// few tiles of pure latency (35 us at K = 2048); the slabs re-read such a matrix from L2 once per
// eight rows and finish in a fraction of that (measured at 64 rows: 14 us against 35 us for 32 or
// 512 output rows, 27 against 35 for 4096, 41 against 64 for 2048 x 4096; 8192 x 2048 stays on the
// tensor cores, 36 against 43). Every row's arithmetic is the one-row GEMV's either way.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "../../../include/ainfer_cuda.h"
#include "model.h"

namespace ainfer {

struct RowSlabs {
  void *groups = nullptr;       // device: ceil(rows / 8) problem records of the grouped kernels' layout
  int32_t *count = nullptr;     // device: their number
};
struct RowSlabCache {
  std::map<std::pair<const void *, int>, RowSlabs> lists;   // by (packed weights, rows)
};

// True when a GEMM of `rows` rows over this matrix should take the slabs.
inline bool row_slabs_pay(int N, int K, int rows) {
  const int G = K / 128;
  return rows > 8 && N <= 4096 && G <= 256 && 256 % G == 0;
}

// The list for (matrix, rows), built on first use (two small synchronous uploads); the device
// blocks are appended to `owned` for the caller to free. Returns 0 or 1 with err set.
inline int row_slabs_get(ainfer_device_t dev, RowSlabCache &cache, std::vector<void *> &owned, const DeviceTensor &t, int rows,
                         RowSlabs *out, std::string &err) {
  const auto key = std::make_pair((const void *)t.data, rows);
  auto it = cache.lists.find(key);
  if (it != cache.lists.end()) { *out = it->second; return 0; }
  struct Rec { uint64_t P, S; int32_t x_row0, M, y_col, pad; };
  static_assert(sizeof(Rec) == 32, "problem record of the grouped kernels");
  const int ng = (rows + 7) / 8;
  std::vector<Rec> recs((size_t)ng);
  for (int j = 0; j < ng; ++j)
    recs[(size_t)j] = Rec{(uint64_t)(uintptr_t)t.data, (uint64_t)(uintptr_t)t.scales, 8 * j, rows - 8 * j < 8 ? rows - 8 * j : 8, 0, 0};
  RowSlabs r;
  void *g = nullptr, *c = nullptr;
  const int32_t n = ng;
  if (ainfer_mem_alloc(dev, recs.size() * sizeof(Rec), 256, &g) != AINFER_OK || ainfer_mem_alloc(dev, 16, 256, &c) != AINFER_OK ||
      ainfer_memcpy_h2d(dev, g, recs.data(), recs.size() * sizeof(Rec)) != AINFER_OK || ainfer_memcpy_h2d(dev, c, &n, 4) != AINFER_OK) {
    err = std::string("row slabs: ") + ainfer_last_error(dev);
    if (g) ainfer_mem_free(dev, g);
    if (c) ainfer_mem_free(dev, c);
    return 1;
  }
  owned.push_back(g);
  owned.push_back(c);
  r.groups = g;
  r.count = (int32_t *)c;
  cache.lists[key] = r;
  *out = r;
  return 0;
}

}  // namespace ainfer
