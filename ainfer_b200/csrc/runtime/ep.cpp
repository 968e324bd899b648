// Expert-parallel mixture-of-experts block for a decode batch (the one place the decode path
// shards across GPUs). Experts are split evenly over the ranks (contiguous ids, E / R per rank);
// the router and the shared expert are replicated; rank r owns batch rows [r * B / R, (r + 1) * B / R).
// Per layer, on the device's stream:
//   A  owner:   post-attention RMSNorm + quantiser, router logits, top-k, dispatch plan, permute
//      exchange of the dispatch buffer (one fixed-size slot per peer; NCCL send/recv in one group)
//   B  experts: group received items by expert, gather, grouped tensor-core GEMM gate/up,
//               SiLU-multiply + quantiser, grouped GEMM down, un-permute into the return buffer;
//               the shared expert of the owned rows is one more problem of the same launches
//      exchange of the return buffer
//   C  owner:   slot-ordered combine with the residual
// Every piece keeps the single-token kernels' arithmetic, so each token's row is bit-identical
// to the one-GPU decode kernels' whatever the batch and the number of ranks. The reference
// decodes one token on one device (tools/decode/decode_l0.cpp:666-674 is its dense MLP) and has
// no counterpart for the exchange.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the library the process already uses if any);
// a world of one rank needs none and replaces the exchanges by device copies inside the list.
#include "ep.h"

#include <dlfcn.h>

#include <cstring>

namespace ainfer {

namespace {

// ---- the few NCCL entry points used, declared here so that the runtime builds without CUDA headers ----
struct NcclUniqueId { char internal[128]; };
typedef struct ncclComm *NcclComm;
struct Nccl {
  void *lib = nullptr;
  int (*GetUniqueId)(NcclUniqueId *) = nullptr;
  int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*Send)(const void *, size_t, int, int, NcclComm, void *) = nullptr;
  int (*Recv)(void *, size_t, int, int, NcclComm, void *) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  std::string err;
  bool load() {
    if (lib) return true;
    lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) { err = std::string("cannot load libnccl.so.2: ") + dlerror(); return false; }
    auto sym = [&](const char *n) { void *p = dlsym(lib, n); if (!p) err = std::string("libnccl.so.2 lacks ") + n; return p; };
    GetUniqueId = (decltype(GetUniqueId))sym("ncclGetUniqueId");
    CommInitRank = (decltype(CommInitRank))sym("ncclCommInitRank");
    CommDestroy = (decltype(CommDestroy))sym("ncclCommDestroy");
    Send = (decltype(Send))sym("ncclSend");
    Recv = (decltype(Recv))sym("ncclRecv");
    GroupStart = (decltype(GroupStart))sym("ncclGroupStart");
    GroupEnd = (decltype(GroupEnd))sym("ncclGroupEnd");
    GetErrorString = (decltype(GetErrorString))sym("ncclGetErrorString");
    if (!err.empty()) { lib = nullptr; return false; }
    return true;
  }
};
Nccl g_nccl;
constexpr int kNcclUint8 = 1;

int item_bytes(int H) { return H + ((H / 128 * 4 + 15) & ~15); }

}  // namespace

struct EpMoe::Impl {
  NcclComm comm = nullptr;
  std::map<std::string, ainfer_kernel_t> kernels;
  std::vector<void *> owned;
  std::vector<ainfer_list_t> lists;   // per layer: A, B, C (world > 1) or one list (world == 1)
  std::vector<ainfer_event_t> events;
};

#define EP_CHECK(call)                                        \
  do {                                                        \
    if ((call) != AINFER_OK) {                                \
      err = ainfer_last_error(dev);                           \
      return 1;                                               \
    }                                                         \
  } while (0)

int ep_unique_id(void *out128, std::string &err) {
  if (!g_nccl.load()) { err = g_nccl.err; return 1; }
  NcclUniqueId id;
  int r = g_nccl.GetUniqueId(&id);
  if (r) { err = std::string("ncclGetUniqueId: ") + g_nccl.GetErrorString(r); return 1; }
  std::memcpy(out128, &id, sizeof id);
  return 0;
}

template <typename T>
int EpMoe::alloc(T **p, size_t bytes) {
  void *q = nullptr;
  if (ainfer_mem_alloc(dev, bytes ? bytes : 16, 256, &q) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
  if (ainfer_mem_fill(dev, q, 0, bytes ? bytes : 16) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
  impl->owned.push_back(q);
  *p = (T *)q;
  return 0;
}

namespace {
struct Rec {   // appends launches to a list; arguments by index in member order
  EpMoe *e;
  ainfer_list_t list;
  int status = 0;
  ainfer_kernel_t kernel(const char *name) {
    auto it = e->impl->kernels.find(name);
    if (it != e->impl->kernels.end()) return it->second;
    ainfer_kernel_t k = nullptr;
    if (ainfer_kernel_get(e->dev, name, &k) != AINFER_OK) {
      e->err = std::string("entry ") + name + " not found";
      status = 1;
      return nullptr;
    }
    e->impl->kernels[name] = k;
    return k;
  }
  template <typename T>
  void set(ainfer_kernel_t k, uint32_t &idx, const T &v) {
    if (status) return;
    if (ainfer_kernel_set_arg(k, idx, sizeof(T), &v) != AINFER_OK) { e->err = ainfer_last_error(e->dev); status = 1; }
    ++idx;
  }
  template <typename... A>
  void launch(const char *name, uint32_t groups, const A &...args) {
    if (status) return;
    ainfer_kernel_t k = kernel(name);
    if (!k) return;
    uint32_t idx = 0;
    (set(k, idx, args), ...);
    if (status) return;
    if (ainfer_list_append_launch(list, k, groups) != AINFER_OK) { e->err = ainfer_last_error(e->dev); status = 1; }
  }
  void copy(void *dst, const void *src, size_t bytes) {
    if (status) return;
    if (ainfer_list_append_memcpy(list, dst, src, bytes) != AINFER_OK) { e->err = ainfer_last_error(e->dev); status = 1; }
  }
};
}  // namespace

int EpMoe::create(DeviceModel *model, const void *id128, int rank_, int world_, int batch_, int flags_) {
  m = model;
  dev = m->dev;
  rank = rank_; world = world_; batch = batch_; flags = flags_;
  impl = new Impl;
  const ModelConfig &c = m->cfg;
  H = c.hidden; E = c.experts; k = c.top_k; I = c.expert_inter; shared = c.shared_experts != 0;
  if (world < 1 || world > 64 || rank < 0 || rank >= world) { err = "usage: 0 <= rank < world <= 64"; return 2; }
  if (batch < world || batch % world) { err = "usage: the batch must divide over the ranks"; return 2; }
  if (E % world) { err = "usage: the experts must divide evenly over the ranks"; return 2; }
  if (E > 1024 || H % 256 || I % 128) { err = "usage: unsupported shape (experts <= 1024, hidden % 256 == 0, intermediate % 128 == 0)"; return 2; }
  n = batch / world;
  epr = E / world;
  cap = n * k;
  if (cap > 2048 || batch * k > 2048) { err = "usage: batch x top-k above the planner's limit (2048 items)"; return 2; }
  // shapes the dp4a kernel does not take run every expert as one tensor-core problem, which holds at most 64 rows
  if (batch > 64 && !(256 % (H / 128) == 0 && 256 % (I / 128) == 0)) { err = "usage: more than 64 rows need hidden and intermediate sizes whose group counts divide 256"; return 2; }
  slot_d = (uint32_t)((16 + (size_t)cap * 16 + (size_t)cap * item_bytes(H) + 15) & ~(size_t)15);
  slot_r = (uint32_t)((size_t)cap * H * 4);
  ainfer_device_info info;
  EP_CHECK(ainfer_device_get_info(dev, &info));
  sm_count = info.sm_count;
  const int G = H / 128, rows = world * cap;   // rows: most items a rank can receive
  int r = 0;
  const int shn = shared ? n : 0;   // the owned rows follow the received items in the grouped layout
  r |= alloc(&Res, (size_t)n * H * 4); r |= alloc(&X, (size_t)n * H * 4); r |= alloc(&Hn, (size_t)n * H * 4);
  if (flags & EP_RES_ADD) { r |= alloc(&Add, (size_t)n * H * 4); r |= alloc(&ResSum, (size_t)n * H * 4); }
  r |= alloc(&Logits, (size_t)n * (E + 1) * 4); r |= alloc(&Bias, (size_t)E * 4);
  r |= alloc(&SelIdx, (size_t)n * (k + 1) * 4); r |= alloc(&SelW, (size_t)n * (k + 1) * 4); r |= alloc(&NearGap, (size_t)n * 4);
  r |= alloc(&ItemDest, (size_t)cap * 4);
  r |= alloc(&Send, (size_t)world * slot_d); r |= alloc(&Recv, (size_t)world * slot_d);
  r |= alloc(&Ret, (size_t)world * slot_r); r |= alloc(&Back, (size_t)world * slot_r);
  r |= alloc(&Sorted, (size_t)rows * 4); r |= alloc(&Counts, 32);
  r |= alloc(&GroupsGU, (size_t)2 * (epr + 1) * 32); r |= alloc(&GroupsD, (size_t)(epr + 1) * 32);
  const size_t nlarge = (size_t)epr + 1 + (size_t)rows / 64 + (size_t)n / 64 + 2;   // an expert with more than 64 rows is cut into 64-row problems
  r |= alloc(&GroupsGUL, 2 * nlarge * 32); r |= alloc(&GroupsDL, nlarge * 32);
  r |= alloc(&XQs, (size_t)(rows + n) * H); r |= alloc(&SQs, (size_t)(rows + n) * G * 4);
  r |= alloc(&GU, (size_t)(rows + shn) * 2 * I * 4); r |= alloc(&AQ, (size_t)(rows + shn) * I);
  r |= alloc(&ASQ, (size_t)(rows + shn) * (I / 128) * 4);
  r |= alloc(&Y2, (size_t)(rows + shn) * H * 4);
  if (r) return 1;
  // the owner's quantised rows live at the tail of the grouped layout: the shared expert reads them in place
  Q8 = XQs + (size_t)rows * H;
  SQ = SQs + (size_t)rows * G;
  Ysh = shared ? Y2 + (size_t)rows * H : nullptr;
  if (world > 1) {
    if (!id128) { err = "usage: a world of several ranks needs the shared NCCL id"; return 2; }
    if (!g_nccl.load()) { err = g_nccl.err; return 1; }
    NcclUniqueId id;
    std::memcpy(&id, id128, sizeof id);
    int nr = g_nccl.CommInitRank(&impl->comm, world, id, rank);
    if (nr) { err = std::string("ncclCommInitRank: ") + g_nccl.GetErrorString(nr); return 1; }
  }
  EP_CHECK(ainfer_device_stream(dev, &stream));
  return 0;
}

// Records the lists of one layer: [A, B, C] for several ranks, [all] for one.
int EpMoe::record_layer(int L) {
  const ModelConfig &c = m->cfg;
  const int G = H / 128, rows = world * cap;
  const std::string p = layer_prefix(L);
  DeviceTensor router = m->tensor(p + "mlp.gate.weight");
  DeviceTensor sgate = m->tensor(p + "mlp.shared_expert_gate.weight");
  if (!router.entry || (shared && !sgate.entry)) { err = "missing " + p + "mlp.gate.weight / shared_expert_gate.weight"; return 1; }
  const ExpertW *tab = (const ExpertW *)m->expert_tables + (size_t)L * (E + 1);
  const float eps = (float)c.rms_eps;
  auto new_list = [&](ainfer_list_t *l) {
    if (ainfer_list_create(dev, l) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
    impl->lists.push_back(*l);
    return 0;
  };
  auto close = [&](Rec &r) {
    if (r.status) return 1;
    if (ainfer_list_close(r.list) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
    return 0;
  };
  const uint32_t tc_blocks = (uint32_t)(2 * sm_count);
  ainfer_list_t la = nullptr;
  if (new_list(&la)) return 1;
  Rec r{this, la};
  // ---- A: route the owned rows and pack their items ----
  const float *res_in = (flags & EP_RES_ADD) ? ResSum : Res;   // what the combine adds the experts' outputs to
  r.launch("RmsNormQuant", (uint32_t)n, (const float *)Res, (const float *)((flags & EP_RES_ADD) ? Add : nullptr),
           (float *)((flags & EP_RES_ADD) ? ResSum : nullptr), (const float *)(m->post_norm + (size_t)L * H), Hn, Q8, SQ,
           (int32_t)H, eps);
  const int tpb = 4;   // tokens per block of the router: enough blocks to fill the device, weights re-read from L2
  r.launch("RouterLogitsRows", (uint32_t)(((E + 1 + 7) / 8) * ((n + tpb - 1) / tpb)), (const uint16_t *)router.data,
           (const uint16_t *)(shared ? sgate.data : nullptr), (const float *)Hn,
           (const float *)((flags & EP_ROUTER_BIAS) ? Bias : nullptr), Logits, (int32_t)E, (int32_t)H, (int32_t)n, (int32_t)tpb);
  r.launch("RouterSelectRows", (uint32_t)n, (const float *)Logits, SelIdx, SelW, NearGap, (int32_t)E, (int32_t)k, (int32_t)(shared ? 1 : 0));
  r.launch("EpPlan", 1u, (const int32_t *)SelIdx, Send, ItemDest, (int32_t)n, (int32_t)k, (int32_t)epr, (int32_t)world, (int32_t)cap, slot_d);
  r.launch("EpPack", (uint32_t)cap, (const int8_t *)Q8, (const float *)SQ, (const int32_t *)ItemDest, Send, (int32_t)k, (int32_t)H, (int32_t)cap,
           slot_d);
  if (world > 1) {
    if (close(r) || new_list(&la)) return 1;
    r.list = la;
  } else {
    r.copy(Recv, Send, slot_d);
  }
  // ---- B: the experts of this rank on everything received ----
  // experts with few rows: the dp4a kernel (weights once, a fraction of the tensor-core kernel's latency); the rest: tensor cores
  const bool multi_ok = 256 % (H / 128) == 0 && 256 % (I / 128) == 0;
  r.launch("EpGroup", 1u, (const unsigned char *)Recv, tab, Sorted, GroupsGU, GroupsD, GroupsGUL, GroupsDL, Counts, (int32_t)world, (int32_t)rank, (int32_t)epr,
           (int32_t)cap, (int32_t)I, slot_d, (int32_t)rows, (int32_t)(shared ? n : 0), (int32_t)E,
           (int32_t)(multi_ok ? 8 : (1 << 30)), (int32_t)64);
  r.launch("EpGather", (uint32_t)rows, (const unsigned char *)Recv, (const int32_t *)Sorted, (const int32_t *)Counts, XQs, SQs, (int32_t)H,
           (int32_t)cap, slot_d);
  const void *gu_tc = multi_ok ? GroupsGUL : GroupsGU, *d_tc = multi_ok ? GroupsDL : GroupsD;
  const int32_t *ngu_tc = multi_ok ? Counts + 3 : Counts + 1, *nd_tc = multi_ok ? Counts + 4 : Counts + 2;
  if (multi_ok)
    r.launch("Int4GemvA8MultiGrouped", tc_blocks, (const void *)GroupsGU, (const int32_t *)(Counts + 1), (const int8_t *)XQs, (const float *)SQs,
             GU, (int32_t)I, (int32_t)H, (int32_t)(2 * I));
  if (batch > 8 || !multi_ok)
    r.launch("Int4GemmA8TcGrouped", tc_blocks, gu_tc, ngu_tc, (const int8_t *)XQs, (const float *)SQs, GU, (int32_t)I, (int32_t)H,
             (int32_t)std::min(batch, 64), (int32_t)(2 * I));
  r.launch("SiluQuantRows", (uint32_t)(rows + (shared ? n : 0)), (const float *)GU, (const int32_t *)Counts, AQ, ASQ, (int32_t)I, (int32_t)rows);
  if (multi_ok)
    r.launch("Int4GemvA8MultiGrouped", tc_blocks, (const void *)GroupsD, (const int32_t *)(Counts + 2), (const int8_t *)AQ, (const float *)ASQ, Y2,
             (int32_t)H, (int32_t)I, (int32_t)H);
  if (batch > 8 || !multi_ok)
    r.launch("Int4GemmA8TcGrouped", tc_blocks, d_tc, nd_tc, (const int8_t *)AQ, (const float *)ASQ, Y2, (int32_t)H, (int32_t)I,
             (int32_t)std::min(batch, 64), (int32_t)H);
  r.launch("EpScatter", (uint32_t)rows, (const float *)Y2, (const int32_t *)Sorted, (const int32_t *)Counts, Ret, (int32_t)H, slot_r);
  if (world > 1) {
    if (close(r) || new_list(&la)) return 1;
    r.list = la;
  } else {
    r.copy(Back, Ret, slot_r);
  }
  // ---- C: combine ----
  r.launch("EpCombine", (uint32_t)(n * ((H + 255) / 256)), res_in, (const unsigned char *)Back, (const int32_t *)ItemDest,
           (const float *)SelW, (const float *)(shared ? Ysh : nullptr), X, (int32_t)k, (int32_t)H, slot_r);
  r.copy(Res, X, (size_t)n * H * 4);   // the next layer's input: layers chain through "res"
  (void)G;
  return close(r);
}

int EpMoe::ensure_layer(int L) {
  const int nl = m->cfg.layers + m->cfg.mtp_layers;
  if (L < 0 || L >= nl) { err = "usage: no such layer"; return 2; }
  if (layer_lists.empty()) layer_lists.assign((size_t)nl, -1);
  if (layer_lists[L] >= 0) return 0;
  const int first = (int)impl->lists.size();
  int r = record_layer(L);
  if (r) return r;
  layer_lists[L] = first;
  return 0;
}

int EpMoe::exchange(void *send, void *recv, uint32_t slot) {
  int r = g_nccl.GroupStart();
  for (int p = 0; p < world && !r; ++p) {
    r = g_nccl.Send((const char *)send + (size_t)p * slot, slot, kNcclUint8, p, impl->comm, stream);
    if (!r) r = g_nccl.Recv((char *)recv + (size_t)p * slot, slot, kNcclUint8, p, impl->comm, stream);
  }
  const int e = g_nccl.GroupEnd();
  if (!r) r = e;
  if (r) { err = std::string("NCCL exchange: ") + g_nccl.GetErrorString(r); return 1; }
  return 0;
}

int EpMoe::run_layer(int L, bool chain, float *seg_ms) {
  int r = ensure_layer(L);
  if (r) return r;
  const int i = layer_lists[L];
  auto stamp = [&](int j) {
    if (!seg_ms) return 0;
    while ((int)impl->events.size() <= j) {
      ainfer_event_t ev = nullptr;
      if (ainfer_event_create(dev, &ev) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
      impl->events.push_back(ev);
    }
    if (ainfer_event_record(impl->events[j]) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
    return 0;
  };
  if (stamp(0)) return 1;
  if (world == 1) {
    EP_CHECK(ainfer_list_execute(impl->lists[i]));
    if (stamp(1) || stamp(2) || stamp(3) || stamp(4)) return 1;
  } else {
    EP_CHECK(ainfer_list_execute(impl->lists[i]));
    if (stamp(1)) return 1;
    if (exchange(Send, Recv, slot_d)) return 1;
    if (stamp(2)) return 1;
    EP_CHECK(ainfer_list_execute(impl->lists[i + 1]));
    if (stamp(3)) return 1;
    if (exchange(Ret, Back, slot_r)) return 1;
    if (stamp(4)) return 1;
    EP_CHECK(ainfer_list_execute(impl->lists[i + 2]));
  }
  (void)chain;   // the layer's last list already copies x to res
  if (stamp(5)) return 1;
  if (seg_ms) {
    EP_CHECK(ainfer_sync(dev, ~0ull));
    for (int j = 0; j < 5; ++j) {
      float ms = 0;
      EP_CHECK(ainfer_event_elapsed_ms(impl->events[j], impl->events[j + 1], &ms));
      seg_ms[j] += ms;
    }
  }
  return 0;
}

int EpMoe::run_stack(int first, int count, float *seg_ms) {
  for (int L = first; L < first + count; ++L) {
    int r = run_layer(L, true, seg_ms);
    if (r) return r;
  }
  return 0;
}

void EpMoe::destroy() {
  if (!impl) return;
  ainfer_sync(dev, ~0ull);
  for (ainfer_list_t l : impl->lists) ainfer_list_destroy(l);
  for (auto &kv : impl->kernels) ainfer_kernel_release(kv.second);
  for (ainfer_event_t e : impl->events) ainfer_event_destroy(e);
  for (void *p : impl->owned) ainfer_mem_free(dev, p);
  if (impl->comm) g_nccl.CommDestroy(impl->comm);
  delete impl;
  impl = nullptr;
}

}  // namespace ainfer
