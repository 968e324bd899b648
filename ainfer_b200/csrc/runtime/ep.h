// Expert-parallel mixture-of-experts block for a decode batch: see ep.cpp.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "../common/tables.h"
#include "model.h"

namespace ainfer {

enum EpFlags {
  EP_ROUTER_BIAS = 1,  // add the "router_bias" buffer to the routed experts' logits (load generators)
  EP_RES_ADD = 2       // the block's residual input is "res" + "add" (the mixer's output not yet added)
};

// Fills 128 bytes with a fresh NCCL id (rank 0 calls, the caller hands it to every rank).
int ep_unique_id(void *out128, std::string &err);

struct EpMoe {
  struct Impl;
  DeviceModel *m = nullptr;
  ainfer_device_t dev = nullptr;
  Impl *impl = nullptr;
  void *stream = nullptr;
  std::string err;
  int rank = 0, world = 1, batch = 0, flags = 0;
  int n = 0;        // rows this rank owns
  int H = 0, E = 0, k = 0, I = 0, epr = 0, cap = 0, sm_count = 0;
  bool shared = false;
  uint32_t slot_d = 0, slot_r = 0;   // bytes of one peer's slot in the dispatch / return buffers
  // owner side
  float *Add = nullptr, *ResSum = nullptr;   // EP_RES_ADD: second addend, and the sum the block works on
  float *Res = nullptr, *X = nullptr, *Hn = nullptr, *SQ = nullptr, *Logits = nullptr, *Bias = nullptr;
  int8_t *Q8 = nullptr;
  int32_t *SelIdx = nullptr, *ItemDest = nullptr;
  float *SelW = nullptr, *NearGap = nullptr;
  unsigned char *Send = nullptr, *Recv = nullptr, *Ret = nullptr, *Back = nullptr;
  // expert side
  int32_t *Sorted = nullptr, *Counts = nullptr;
  void *GroupsGU = nullptr, *GroupsD = nullptr, *GroupsGUL = nullptr, *GroupsDL = nullptr;   // problem lists: few rows / many rows
  int8_t *XQs = nullptr, *AQ = nullptr;
  float *SQs = nullptr, *GU = nullptr, *ASQ = nullptr, *Y2 = nullptr;
  float *Ysh = nullptr;   // shared expert's outputs of the owned rows (tail of Y2)
  std::vector<int> layer_lists;   // per layer: index of its first list, -1 = not recorded yet

  // Returns 0, 1 (device / NCCL error) or 2 (usage); err holds the message.
  int create(DeviceModel *model, const void *id128, int rank, int world, int batch, int flags);
  // X = Res + MoE(norm_L(Res)) for the owned rows, and Res <- X afterwards (layers chain). seg_ms (optional,
  // 5 floats, accumulated): device time of route+pack, dispatch, experts, return, shared+combine;
  // asking for it synchronises after the layer.
  int run_layer(int L, bool chain, float *seg_ms);
  int run_stack(int first, int count, float *seg_ms);
  void destroy();

  template <typename T>
  int alloc(T **p, size_t bytes);
  int record_layer(int L);
  int ensure_layer(int L);
  int exchange(void *send, void *recv, uint32_t slot);
};

}  // namespace ainfer
