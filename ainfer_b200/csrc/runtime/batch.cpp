// Batched decode: every sequence of a batch advances one token per step. The batch is split
// over the ranks by sequence: rank r owns sequences [r B/R, (r+1) B/R) with their DeltaNet state,
// conv history and INT8 KV cache; attention, DeltaNet, the dense projections and the LM head run
// on the owner alone (their weights are replicated), and only the MoE block exchanges tokens with
// the ranks that hold the routed experts (ep.cpp). A step is, per layer, one recorded list of
// row-batched launches for the mixer (RMSNorm + quantiser of the rows, tensor-core GEMMs for the
// projections, per-sequence conv / recurrence / attention kernels) followed by the MoE block of
// the rows, then the final norm, the LM head as one batched GEMM and a per-sequence argmax that
// also advances each sequence's control block on the device: a greedy loop needs no host work
// between steps. The reference decodes one sequence at a time (its token loop is
// tools/decode/decode_l0.cpp:742-825); each sequence's arithmetic here is that loop's, so a
// sequence decodes to the same tokens in a batch as alone.
#include <cstring>

#include "batch.h"

namespace ainfer {

namespace {
struct Rec {   // appends launches to a list; arguments by index in member order
  BatchDecode *b;
  ainfer_list_t list;
  int status = 0;
  template <typename T>
  void set(ainfer_kernel_t k, uint32_t &idx, const T &v) {
    if (status) return;
    if (ainfer_kernel_set_arg(k, idx, sizeof(T), &v) != AINFER_OK) { b->err = ainfer_last_error(b->dev); status = 1; }
    ++idx;
  }
  template <typename... A>
  void launch(const char *name, uint32_t groups, const A &...args) {
    if (status) return;
    ainfer_kernel_t k = nullptr;
    auto it = b->kernels.find(name);
    if (it != b->kernels.end()) k = it->second;
    else {
      if (ainfer_kernel_get(b->dev, name, &k) != AINFER_OK) { b->err = std::string("entry ") + name + " not found"; status = 1; return; }
      b->kernels[name] = k;
    }
    uint32_t idx = 0;
    (set(k, idx, args), ...);
    if (status) return;
    if (ainfer_list_append_launch(list, k, groups ? groups : 1) != AINFER_OK) { b->err = ainfer_last_error(b->dev); status = 1; }
  }
  void gemm(const DeviceTensor &t, const int8_t *XQ, const float *SQ, float *Y, int K, int rows) {
    if (status) return;
    if (!t.entry || (int)t.entry->shape[1] != K || t.entry->storage != DT_INT4_SYM_G128) {
      b->err = "batch: missing tensor or unexpected shape/storage" + (t.entry ? " of " + t.entry->name : std::string());
      status = 2;
      return;
    }
    const int N = (int)t.entry->shape[0];
    const int G = K / 128;
    if (rows <= 8 && G <= 256 && 256 % G == 0) {
      // few rows: the dp4a kernel streams the weights once and has a fraction of the tensor-core kernel's latency
      const uint32_t tiles = (uint32_t)((N + 256 / G - 1) / (256 / G));
      launch("Int4GemvA8Multi", std::min<uint32_t>(tiles, 2u * (uint32_t)b->sm_count), (const uint8_t *)t.data, (const uint16_t *)t.scales, XQ, SQ,
             Y, (int32_t)N, (int32_t)K, (int32_t)rows, (int32_t)N);
      return;
    }
    if (row_slabs_pay(N, K, rows)) {
      // few output rows: slabs of eight rows through the dp4a kernel beat the tensor-core kernel's latency (row_slabs.h)
      RowSlabs sl;
      if (row_slabs_get(b->dev, b->slabs, b->owned, t, rows, &sl, b->err)) { status = 1; return; }
      launch("Int4GemvA8MultiGrouped", 2u * (uint32_t)b->sm_count, (const void *)sl.groups, (const int32_t *)sl.count, XQ, SQ, Y, (int32_t)N,
             (int32_t)K, (int32_t)N);
      return;
    }
    const uint32_t tiles = (uint32_t)((N + 127) / 128);
    launch("Int4GemmA8Tc", std::min<uint32_t>(tiles, 2u * (uint32_t)b->sm_count), (const uint8_t *)t.data, (const uint16_t *)t.scales, XQ, SQ, Y,
           (int32_t)N, (int32_t)K, (int32_t)rows, (int32_t)N);
  }
};
}  // namespace

template <typename T>
int BatchDecode::alloc(T **p, size_t count) {
  void *q = nullptr;
  const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
  if (ainfer_mem_alloc(dev, bytes, 256, &q) != AINFER_OK || ainfer_mem_fill(dev, q, 0, bytes) != AINFER_OK) {
    err = std::string("batch: alloc of ") + std::to_string(bytes) + " bytes failed: " + ainfer_last_error(dev);
    return 1;
  }
  owned.push_back(q);
  *p = (T *)q;
  return 0;
}

int BatchDecode::create(DeviceModel *model, const void *id128, int rank, int world, int batch, int max_ctx_, int flags) {
  m = model;
  dev = m->dev;
  max_ctx = max_ctx_;
  const ModelConfig &c = m->cfg;
  if (batch < world || batch % world || max_ctx < 1) { err = "usage: the batch must divide over the ranks"; return 2; }
  const int ratio = c.kv_heads ? c.q_heads / c.kv_heads : 0;
  if (c.head_dim != 256 || !(ratio == 1 || ratio == 2 || ratio == 4 || ratio == 6 || ratio == 8)) { err = "usage: unsupported attention shape"; return 2; }
  n = batch / world;
  ainfer_device_info info;
  if (ainfer_device_get_info(dev, &info) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
  sm_count = info.sm_count;
  std::string e2;
  if (model_ensure_rope(m, max_ctx, e2)) { err = e2; return 1; }
  int r = ep.create(m, id128, rank, world, batch, EP_RES_ADD | (flags & EP_ROUTER_BIAS));
  if (r) { err = ep.err; return r; }
  ep_ready = true;
  const int H = c.hidden, C = c.conv_dim(), VD = c.value_dim(), nV = c.lin_v_heads, nQ = c.q_heads, nKV = c.kv_heads, D = c.head_dim;
  const int QN = nQ * 2 * D, KN = nKV * D, AK = nQ * D, maxK = std::max(H, std::max(VD, AK));
  max_chunks = (max_ctx + 63) / 64;
  r = 0;
  r |= alloc(&Ctrl, (size_t)n * 4); r |= alloc(&OutT, (size_t)n);
  r |= alloc(&Q8, (size_t)n * maxK); r |= alloc(&SQ, (size_t)n * (maxK / 128));
  r |= alloc(&Pq, (size_t)n * C); r |= alloc(&Mx, (size_t)n * C); r |= alloc(&Z, (size_t)n * VD);
  r |= alloc(&Br, (size_t)n * nV); r |= alloc(&Ar, (size_t)n * nV); r |= alloc(&Bt, (size_t)n * nV); r |= alloc(&Gt, (size_t)n * nV);
  r |= alloc(&O, (size_t)n * VD);
  r |= alloc(&Q16, (size_t)n * QN); r |= alloc(&K16, (size_t)n * KN); r |= alloc(&V16, (size_t)n * KN); r |= alloc(&Qn, (size_t)n * AK);
  r |= alloc(&Pm, (size_t)n * nQ * max_chunks); r |= alloc(&Pse, (size_t)n * nQ * max_chunks);
  r |= alloc(&Pacc, (size_t)n * nQ * max_chunks * D);
  r |= alloc(&Logits, (size_t)n * c.vocab);
  // per-sequence state: [sequence][layer of its kind][...]
  conv_stride = (size_t)c.n_lin() * C * 3;
  s_stride = (size_t)c.n_lin() * nV * 128 * 128;
  kv_rows = (size_t)c.n_attn() * max_ctx;   // cache rows of one sequence (all its attention layers)
  r |= alloc(&conv, (size_t)n * conv_stride); r |= alloc(&S, (size_t)n * s_stride);
  r |= alloc(&Kc, (size_t)n * kv_rows * nKV * D); r |= alloc(&Vc, (size_t)n * kv_rows * nKV * D);
  r |= alloc(&Ks, (size_t)n * kv_rows * nKV); r |= alloc(&Vs, (size_t)n * kv_rows * nKV);
  if (r) return 1;
  return record();
}

int BatchDecode::record() {
  const ModelConfig &c = m->cfg;
  const int H = c.hidden, C = c.conv_dim(), VD = c.value_dim(), nK = c.lin_k_heads, nV = c.lin_v_heads;
  const int nQ = c.q_heads, nKV = c.kv_heads, D = c.head_dim, AK = nQ * D;
  const float eps = (float)c.rms_eps;
  DeviceTensor emb = m->tensor("model.language_model.embed_tokens.weight");
  if (!emb.entry) { err = "missing model.language_model.embed_tokens.weight"; return 1; }
  auto new_list = [&](ainfer_list_t *l) {
    if (ainfer_list_create(dev, l) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
    lists.push_back(*l);
    return 0;
  };
  auto close = [&](Rec &r) {
    if (r.status) return r.status;
    if (ainfer_list_close(r.list) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
    return 0;
  };
  float *X = ep.Res;   // the rows' residual stream lives in the MoE block's input buffer
  ainfer_list_t l = nullptr;
  if (new_list(&l)) return 1;
  embed_list = l;
  {
    Rec r{this, l};
    r.launch("EmbedRow", (uint32_t)n, X, (const uint16_t *)emb.data, (const int32_t *)Ctrl, (int32_t)H, (int32_t)c.vocab, (int32_t)4);
    if (int e = close(r)) return e;
  }
  for (int L = 0; L < c.layers; ++L) {
    if (new_list(&l)) return 1;
    layer_lists.push_back(l);
    Rec r{this, l};
    const std::string pf = layer_prefix(L);
    const int slot = m->slot[L];
    r.launch("RmsNormQuant", (uint32_t)n, (const float *)X, (const float *)nullptr, (float *)nullptr,
             (const float *)(m->in_norm + (size_t)L * H), (float *)nullptr, Q8, SQ, (int32_t)H, eps);
    if (c.layer_types[L] == 'A') {
      r.gemm(m->tensor(pf + "self_attn.q_proj.weight"), Q8, SQ, Q16, H, n);
      r.gemm(m->tensor(pf + "self_attn.k_proj.weight"), Q8, SQ, K16, H, n);
      r.gemm(m->tensor(pf + "self_attn.v_proj.weight"), Q8, SQ, V16, H, n);
      const size_t off = (size_t)slot * max_ctx * nKV;   // this layer's rows inside a sequence's cache
      auto attn = [&](const char *name, int groups) {
        r.launch(name, (uint32_t)(n * groups), (const float *)Q16, (const float *)K16, (const float *)V16,
                 (const float *)(m->q_norm + (size_t)slot * D), (const float *)(m->k_norm + (size_t)slot * D), (const float *)m->rope_cos,
                 (const float *)m->rope_sin, (const int32_t *)Ctrl, Qn, Kc + off * D, Vc + off * D, Ks + off, Vs + off, Pm, Pse, Pacc, Q8, SQ,
                 (int32_t)nQ, (int32_t)nKV, (int32_t)c.rotary_dim, (int32_t)max_ctx, (int32_t)max_chunks, (int32_t)n, (int32_t)groups, eps,
                 (int64_t)kv_rows);
      };
      attn("BatchAttnPrep", (nQ + 2 * nKV + 7) / 8);
      attn("BatchAttnSplit", std::max(1, std::min(max_chunks * nKV, (sm_count * 8 + n - 1) / n)));
      attn("BatchAttnCombine", nQ);
      r.gemm(m->tensor(pf + "self_attn.o_proj.weight"), Q8, SQ, ep.Add, AK, n);
    } else {
      r.gemm(m->tensor(pf + "linear_attn.in_proj_qkv.weight"), Q8, SQ, Pq, H, n);
      r.gemm(m->tensor(pf + "linear_attn.in_proj_z.weight"), Q8, SQ, Z, H, n);
      r.gemm(m->tensor(pf + "linear_attn.in_proj_b.weight"), Q8, SQ, Br, H, n);
      r.gemm(m->tensor(pf + "linear_attn.in_proj_a.weight"), Q8, SQ, Ar, H, n);
      r.launch("BatchConvSilu", (uint32_t)(((size_t)n * C + 255) / 256), Mx, (const float *)Pq, conv + (size_t)slot * C * 3,
               (const float *)(m->conv_w + (size_t)slot * C * 4), (int32_t)C, (int32_t)n, (int64_t)conv_stride);
      r.launch("ChunkBetaDecay", (uint32_t)((n * nV + 255) / 256), (const float *)Br, (const float *)Ar,
               (const float *)(m->a_log + (size_t)slot * nV), (const float *)(m->dt_bias + (size_t)slot * nV), Bt, Gt, (int32_t)nV,
               (int32_t)(n * nV));
      r.launch("BatchDeltaNetStep", (uint32_t)(n * nV * 4), O, (const float *)Mx, S + (size_t)slot * nV * 128 * 128, (const float *)Bt,
               (const float *)Gt, (int32_t)nK, (int32_t)nV, (int32_t)n, (int64_t)s_stride);
      r.launch("GatedNormQuant", (uint32_t)((n * nV + 3) / 4), (const float *)O, (const float *)Z,
               (const float *)(m->lin_norm + (size_t)slot * c.lin_head_dim), Q8, SQ, (float *)nullptr, (int32_t)(n * nV), eps);
      r.gemm(m->tensor(pf + "linear_attn.out_proj.weight"), Q8, SQ, ep.Add, VD, n);
    }
    if (int e = close(r)) return e;
  }
  if (new_list(&l)) return 1;
  tail_list = l;
  {
    Rec r{this, l};
    r.launch("RmsNormQuant", (uint32_t)n, (const float *)X, (const float *)nullptr, (float *)nullptr, (const float *)m->final_norm,
             (float *)nullptr, Q8, SQ, (int32_t)H, eps);
    r.gemm(m->tensor("lm_head.weight"), Q8, SQ, Logits, H, n);
    r.launch("BatchArgmax", (uint32_t)n, (const float *)Logits, OutT, Ctrl, (int32_t)c.vocab, (int32_t)1);
    if (int e = close(r)) return e;
  }
  return 0;
}

int BatchDecode::step() {
  if (ainfer_list_execute(embed_list) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
  for (int L = 0; L < m->cfg.layers; ++L) {
    if (ainfer_list_execute(layer_lists[L]) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
    // x = (x + mixer) + MoE(norm(x + mixer)) for the rows, experts wherever they live
    int e = ep.run_layer(L, true, nullptr);
    if (e) { err = ep.err; return e; }
  }
  if (ainfer_list_execute(tail_list) != AINFER_OK) { err = ainfer_last_error(dev); return 1; }
  return 0;
}

void BatchDecode::destroy() {
  if (dev) ainfer_sync(dev, UINT64_MAX);
  for (ainfer_list_t l : lists) ainfer_list_destroy(l);
  lists.clear();
  if (ep_ready || ep.impl) ep.destroy();
  ep_ready = false;
  for (auto &kv : kernels) ainfer_kernel_release(kv.second);
  kernels.clear();
  for (void *q : owned) ainfer_mem_free(dev, q);
  owned.clear();
}

}  // namespace ainfer
