// Batched decode over sequences owned by this rank: see batch.cpp.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "ep.h"
#include "model.h"
#include "row_slabs.h"

namespace ainfer {

struct BatchDecode {
  DeviceModel *m = nullptr;
  ainfer_device_t dev = nullptr;
  std::string err;
  EpMoe ep;
  bool ep_ready = false;
  int n = 0, max_ctx = 0, max_chunks = 0, sm_count = 0;
  // rows
  int32_t *Ctrl = nullptr, *OutT = nullptr;     // [n][4], [n]
  int8_t *Q8 = nullptr; float *SQ = nullptr;
  float *Pq = nullptr, *Mx = nullptr, *Z = nullptr, *Br = nullptr, *Ar = nullptr, *Bt = nullptr, *Gt = nullptr, *O = nullptr;
  float *Q16 = nullptr, *K16 = nullptr, *V16 = nullptr, *Qn = nullptr, *Pm = nullptr, *Pse = nullptr, *Pacc = nullptr;
  float *Logits = nullptr;                      // [n][V]
  // per-sequence state
  float *conv = nullptr, *S = nullptr;
  int8_t *Kc = nullptr, *Vc = nullptr;
  uint16_t *Ks = nullptr, *Vs = nullptr;
  size_t conv_stride = 0, s_stride = 0, kv_rows = 0;
  std::vector<ainfer_list_t> lists, layer_lists;
  ainfer_list_t embed_list = nullptr, tail_list = nullptr;
  std::map<std::string, ainfer_kernel_t> kernels;
  std::vector<void *> owned;
  RowSlabCache slabs;   // problem lists of the GEMMs with few output rows (row_slabs.h)

  // Returns 0, 1 (device / NCCL error) or 2 (usage); err holds the message.
  int create(DeviceModel *model, const void *id128, int rank, int world, int batch, int max_ctx, int flags);
  // One token for every owned sequence: reads each sequence's control block {token, position,
  // length, -}, writes its greedy token to OutT and advances the block. Asynchronous.
  int step();
  void destroy();

  template <typename T>
  int alloc(T **p, size_t count);
  int record();
};

}  // namespace ainfer
