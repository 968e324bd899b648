// Chunked prefill: advances a session's state (DeltaNet state, conv history, INT8 KV cache) over a
// run of prompt tokens, up to 64 rows at a time, instead of one decode step per token. The chunk
// orchestration of the reference (tools/cmdlist/chunklayer_replay.cpp:366-443: ChunkGemm,
// ChunkSsmConv, ChunkSsmRecur, ChunkAttn per layer, state persisting across chunk replays) with
// this library's row-batched kernels:
//   rows' RMSNorm + quantiser -> batched W4A8 GEMM on the tensor cores for every projection
//   (weights cross HBM once per chunk, not once per token) -> DeltaNet: conv + SiLU over the rows,
//   beta / decay, the recurrence with the state on the chip for the whole chunk, gated norm ->
//   attention: the decode kernels' bodies for all rows at once (head norm + RoPE + INT8 append of
//   every row, then every row's chunked attention over the cache up to its own position, then the
//   merges) -> output projection -> the MoE block of the rows (router,
//   device permute by expert, grouped tensor-core expert GEMMs, slot-ordered combine; ep.cpp with
//   one rank), which also performs the residual add.
// Every row's arithmetic is the decode path's, so a prefilled session is bit-identical to one that
// decoded the same tokens one by one (tests/test_prefill_gpu.py). Launches are immediate (no
// recorded list): the number of rows of the last chunk varies.
//
// The same pass verifies speculative rows (the MTP loop's batched verification): it can return
// every row's greedy prediction (final norm, LM head as one GEMM over the rows, argmax per row)
// and keep a snapshot of the DeltaNet state and conv history after every row, so that the caller
// rolls back to the last accepted row (the INT8 cache needs no rollback: rows beyond the accepted
// ones are overwritten before any later position reads them).
#include <cstring>

#include "ep.h"
#include "executor.h"
#include "row_slabs.h"

namespace ainfer {

struct Prefill {
  Session *s = nullptr;
  EpMoe ep;
  bool ep_ready = false;
  int rows_cap = 64;
  std::vector<void *> owned;
  // row buffers
  int32_t *Ctrl = nullptr, *OutT = nullptr;      // [rows][4], [rows]
  float *Logits = nullptr;                       // [rows][V] (verification only)
  float *SnapS = nullptr, *SnapC = nullptr;      // [rows][all DeltaNet layers' state / conv history] (verification only)
  size_t snap_s_stride = 0, snap_c_stride = 0;
  int last_rows = 0;
  // a full verification pass recorded once: vlists[L] = everything between the MoE blocks of layers
  // L - 1 and L (vlists[0] starts with the embedding), vlists[layers] = the rows' predictions
  std::vector<ainfer_list_t> vlists;
  int8_t *Q8 = nullptr; float *SQ = nullptr;     // [rows][maxK], [rows][maxK/128]
  float *Pq = nullptr, *Mx = nullptr, *Z = nullptr, *Br = nullptr, *Ar = nullptr, *Bt = nullptr, *Gt = nullptr, *O = nullptr;
  float *Q16 = nullptr, *K16 = nullptr, *V16 = nullptr;
  float *Qn = nullptr, *Pm = nullptr, *Pse = nullptr, *Pacc = nullptr;   // per-row attention scratch
  std::map<std::string, ainfer_kernel_t> kernels;
  RowSlabCache slabs;   // problem lists of the GEMMs with few output rows (row_slabs.h)
};

namespace {

template <typename T>
int palloc(Prefill *p, size_t count, T **out) {
  Session *s = p->s;
  void *q = nullptr;
  const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
  if (ainfer_mem_alloc(s->dev, bytes, 256, &q) != AINFER_OK || ainfer_mem_fill(s->dev, q, 0, bytes) != AINFER_OK) {
    s->err = std::string("prefill: alloc failed: ") + ainfer_last_error(s->dev);
    return 1;
  }
  p->owned.push_back(q);
  *out = (T *)q;
  return 0;
}

struct Launcher {   // immediate launches, or appended to recorded lists; arguments by index in member order
  Prefill *p;
  int status = 0;
  bool recording = false;
  ainfer_list_t list = nullptr;
  // recording: closes the current list (if any) into p->vlists and opens the next one
  void cut(bool open_next) {
    if (status) return;
    Session *s = p->s;
    if (list) {
      if (ainfer_list_close(list) != AINFER_OK) { s->err = ainfer_last_error(s->dev); status = 1; return; }
      p->vlists.push_back(list);
      list = nullptr;
    }
    if (open_next && ainfer_list_create(s->dev, &list) != AINFER_OK) { s->err = ainfer_last_error(s->dev); status = 1; }
  }
  template <typename T>
  void set(ainfer_kernel_t k, uint32_t &idx, const T &v) {
    if (status) return;
    if (ainfer_kernel_set_arg(k, idx, sizeof(T), &v) != AINFER_OK) { p->s->err = ainfer_last_error(p->s->dev); status = 1; }
    ++idx;
  }
  template <typename... A>
  void launch(const char *name, uint32_t groups, const A &...args) {
    if (status) return;
    Session *s = p->s;
    auto it = p->kernels.find(name);
    ainfer_kernel_t k = nullptr;
    if (it != p->kernels.end()) k = it->second;
    else {
      if (ainfer_kernel_get(s->dev, name, &k) != AINFER_OK) { s->err = std::string("entry ") + name + " not found"; status = 1; return; }
      p->kernels[name] = k;
    }
    uint32_t idx = 0;
    (set(k, idx, args), ...);
    if (status) return;
    const int rc = recording ? ainfer_list_append_launch(list, k, groups ? groups : 1) : ainfer_kernel_launch(s->dev, k, groups ? groups : 1);
    if (rc != AINFER_OK) { s->err = std::string(name) + ": " + ainfer_last_error(s->dev); status = 1; }
  }
  // Y[rows][N] = X[rows][K] . W^T on the tensor cores
  void gemm(const DeviceTensor &t, const int8_t *XQ, const float *SQ, float *Y, int K, int rows) {
    if (status) return;
    Session *s = p->s;
    if (!t.entry || (int)t.entry->shape[1] != K || t.entry->storage != DT_INT4_SYM_G128) {
      s->err = "prefill: missing tensor or unexpected shape/storage" + (t.entry ? " of " + t.entry->name : std::string());
      status = 2;
      return;
    }
    const int N = (int)t.entry->shape[0];
    const int G = K / 128;
    if (rows <= 8 && G <= 256 && 256 % G == 0) {
      // few rows: the dp4a kernel streams the weights once and has a fraction of the tensor-core kernel's latency
      const uint32_t tiles = (uint32_t)((N + 256 / G - 1) / (256 / G));
      launch("Int4GemvA8Multi", std::min<uint32_t>(tiles, 2u * (uint32_t)s->sm_count), (const uint8_t *)t.data, (const uint16_t *)t.scales, XQ, SQ,
             Y, (int32_t)N, (int32_t)K, (int32_t)rows, (int32_t)N);
      return;
    }
    if (row_slabs_pay(N, K, rows)) {
      // few output rows: slabs of eight rows through the dp4a kernel beat the tensor-core kernel's latency (row_slabs.h)
      RowSlabs sl;
      if (row_slabs_get(s->dev, p->slabs, p->owned, t, rows, &sl, s->err)) { status = 1; return; }
      launch("Int4GemvA8MultiGrouped", 2u * (uint32_t)s->sm_count, (const void *)sl.groups, (const int32_t *)sl.count, XQ, SQ, Y, (int32_t)N,
             (int32_t)K, (int32_t)N);
      return;
    }
    const uint32_t tiles = (uint32_t)((N + 127) / 128);
    for (int r0 = 0; r0 < rows; r0 += 64)   // the tensor-core kernel takes 64 rows a launch
      launch("Int4GemmA8Tc", std::min<uint32_t>(tiles, 2u * (uint32_t)s->sm_count), (const uint8_t *)t.data, (const uint16_t *)t.scales,
             XQ + (size_t)r0 * K, SQ + (size_t)r0 * G, Y + (size_t)r0 * N, (int32_t)N, (int32_t)K, (int32_t)std::min(64, rows - r0), (int32_t)N);
  }
};

}  // namespace

int prefill_create(Session *s, int rows_cap, bool verify, Prefill **out, int ep_rank, int ep_world, const void *id128) {
  const ModelConfig &c = s->m->cfg;
  Prefill *p = new Prefill;
  p->s = s;
  p->rows_cap = rows_cap;
  const int R = p->rows_cap, H = c.hidden, C = c.conv_dim(), VD = c.value_dim(), nV = c.lin_v_heads;
  const int QN = c.q_heads * 2 * c.head_dim, KN = c.kv_heads * c.head_dim, AK = c.q_heads * c.head_dim;
  const int maxK = std::max(H, std::max(VD, AK));
  int r = 0;
  r |= palloc(p, (size_t)R * 4, &p->Ctrl);
  r |= palloc(p, (size_t)R * maxK, &p->Q8); r |= palloc(p, (size_t)R * (maxK / 128), &p->SQ);
  r |= palloc(p, (size_t)R * C, &p->Pq); r |= palloc(p, (size_t)R * C, &p->Mx); r |= palloc(p, (size_t)R * VD, &p->Z);
  r |= palloc(p, (size_t)R * nV, &p->Br); r |= palloc(p, (size_t)R * nV, &p->Ar);
  r |= palloc(p, (size_t)R * nV, &p->Bt); r |= palloc(p, (size_t)R * nV, &p->Gt);
  r |= palloc(p, (size_t)R * VD, &p->O);
  r |= palloc(p, (size_t)R * QN, &p->Q16); r |= palloc(p, (size_t)R * KN, &p->K16); r |= palloc(p, (size_t)R * KN, &p->V16);
  r |= palloc(p, (size_t)R * AK, &p->Qn); r |= palloc(p, (size_t)R * c.q_heads * s->max_chunks, &p->Pm);
  r |= palloc(p, (size_t)R * c.q_heads * s->max_chunks, &p->Pse); r |= palloc(p, (size_t)R * c.q_heads * s->max_chunks * c.head_dim, &p->Pacc);
  if (verify) {
    p->snap_s_stride = (size_t)c.n_lin() * nV * 128 * 128;
    p->snap_c_stride = (size_t)c.n_lin() * C * 3;
    r |= palloc(p, (size_t)R, &p->OutT); r |= palloc(p, (size_t)R * c.vocab, &p->Logits);
    r |= palloc(p, (size_t)R * p->snap_s_stride, &p->SnapS); r |= palloc(p, (size_t)R * p->snap_c_stride, &p->SnapC);
  }
  if (!r) {
    // the expert-parallel block counts rows over all ranks: every rank brings R of them
    int e = p->ep.create(s->m, ep_world > 1 ? id128 : nullptr, ep_rank, ep_world, R * ep_world, EP_RES_ADD);
    if (e) { s->err = "prefill: " + p->ep.err; r = e; }
    else p->ep_ready = true;
  }
  if (r) { prefill_destroy(p); return r; }
  *out = p;
  return 0;
}

int prefill_rows_cap(const Prefill *p) { return p->rows_cap; }

void prefill_destroy(Prefill *p) {
  if (!p) return;
  ainfer_sync(p->s->dev, UINT64_MAX);
  if (p->ep_ready || p->ep.impl) p->ep.destroy();
  for (ainfer_list_t l : p->vlists) ainfer_list_destroy(l);
  for (auto &kv : p->kernels) ainfer_kernel_release(kv.second);
  for (void *q : p->owned) ainfer_mem_free(p->s->dev, q);
  delete p;
}

// Advances the session over tokens[0..n) at positions start_pos... predictions (optional, needs a
// verification object and n <= its rows): every row's greedy next token; the state after every
// row is then also kept for prefill_rollback.
int prefill_run(Prefill *p, const int *tokens, int n, int start_pos, int *predictions) {
  Session *s = p->s;
  DeviceModel *m = s->m;
  const ModelConfig &c = m->cfg;
  if (n < 0 || start_pos < 0 || start_pos + n > s->max_ctx) {
    s->err = "context overflow: pos " + std::to_string(start_pos + n) + " >= MAXCTX " + std::to_string(s->max_ctx);
    return 3;
  }
  const int H = c.hidden, C = c.conv_dim(), VD = c.value_dim(), nK = c.lin_k_heads, nV = c.lin_v_heads;
  const int nQ = c.q_heads, nKV = c.kv_heads, D = c.head_dim;
  const int QN = nQ * 2 * D, KN = nKV * D, AK = nQ * D;
  const float eps = (float)c.rms_eps;
  DeviceTensor emb = m->tensor("model.language_model.embed_tokens.weight");
  if (!emb.entry) { s->err = "missing model.language_model.embed_tokens.weight"; return 1; }
  EpMoe &ep = p->ep;
  const bool verify = predictions != nullptr;
  if (verify && (!p->SnapS || n > p->rows_cap)) { s->err = "usage: predictions need a verification object and at most its rows"; return 2; }
  p->last_rows = verify ? n : 0;
  // One pass over `rows` rows whose control blocks are in p->Ctrl: immediate, or recorded into p->vlists.
  auto pass = [&](Launcher &l, int rows) -> int {
    float *X = ep.Res;   // the rows' residual stream lives in the MoE block's input buffer
    l.launch("EmbedRow", (uint32_t)rows, X, (const uint16_t *)emb.data, (const int32_t *)p->Ctrl, (int32_t)H, (int32_t)c.vocab, (int32_t)4);
    for (int L = 0; L < c.layers && !l.status; ++L) {
      const std::string pf = layer_prefix(L);
      const int slot = m->slot[L];
      l.launch("RmsNormQuant", (uint32_t)rows, (const float *)X, (const float *)nullptr, (float *)nullptr,
               (const float *)(m->in_norm + (size_t)L * H), (float *)nullptr, p->Q8, p->SQ, (int32_t)H, eps);
      if (c.layer_types[L] == 'A') {
        l.gemm(m->tensor(pf + "self_attn.q_proj.weight"), p->Q8, p->SQ, p->Q16, H, rows);
        l.gemm(m->tensor(pf + "self_attn.k_proj.weight"), p->Q8, p->SQ, p->K16, H, rows);
        l.gemm(m->tensor(pf + "self_attn.v_proj.weight"), p->Q8, p->SQ, p->V16, H, rows);
        const size_t kv_off = (size_t)slot * s->max_ctx * nKV;
        int8_t *Kc = s->Kc + kv_off * D, *Vc = s->Vc + kv_off * D;
        uint16_t *Ks = s->Ks + kv_off, *Vs = s->Vs + kv_off;
        // all rows at once, three launches: every row appends its K / V (its own cache position), then
        // every row attends to the cache up to its own position (rows before it included: the appends of
        // the whole pass are complete), then the merges. Per row the arithmetic is the decode kernels'.
        auto attn = [&](const char *name, int groups) {
          l.launch(name, (uint32_t)(rows * groups), (const float *)p->Q16, (const float *)p->K16, (const float *)p->V16,
                   (const float *)(m->q_norm + (size_t)slot * D), (const float *)(m->k_norm + (size_t)slot * D), (const float *)m->rope_cos,
                   (const float *)m->rope_sin, (const int32_t *)p->Ctrl, p->Qn, Kc, Vc, Ks, Vs, p->Pm, p->Pse, p->Pacc, p->Q8, p->SQ, (int32_t)nQ,
                   (int32_t)nKV, (int32_t)c.rotary_dim, (int32_t)s->max_ctx, (int32_t)s->max_chunks, (int32_t)rows, (int32_t)groups, eps,
                   (int64_t)0);
        };
        attn("BatchAttnPrep", (nQ + 2 * nKV + 7) / 8);
        attn("BatchAttnSplit", std::max(1, std::min(s->max_chunks * nKV, (s->sm_count * 8 + rows - 1) / rows)));
        attn("BatchAttnCombine", nQ);
        l.gemm(m->tensor(pf + "self_attn.o_proj.weight"), p->Q8, p->SQ, ep.Add, AK, rows);
      } else {
        l.gemm(m->tensor(pf + "linear_attn.in_proj_qkv.weight"), p->Q8, p->SQ, p->Pq, H, rows);
        l.gemm(m->tensor(pf + "linear_attn.in_proj_z.weight"), p->Q8, p->SQ, p->Z, H, rows);
        l.gemm(m->tensor(pf + "linear_attn.in_proj_b.weight"), p->Q8, p->SQ, p->Br, H, rows);
        l.gemm(m->tensor(pf + "linear_attn.in_proj_a.weight"), p->Q8, p->SQ, p->Ar, H, rows);
        l.launch("ChunkConvSilu", (uint32_t)((C + 255) / 256), p->Mx, (const float *)p->Pq, s->conv + (size_t)slot * C * 3,
                 (const float *)(m->conv_w + (size_t)slot * C * 4), (int32_t)C, (int32_t)rows,
                 (float *)(verify ? p->SnapC + (size_t)slot * C * 3 : nullptr), (int64_t)p->snap_c_stride);
        l.launch("ChunkBetaDecay", (uint32_t)((rows * nV + 255) / 256), (const float *)p->Br, (const float *)p->Ar,
                 (const float *)(m->a_log + (size_t)slot * nV), (const float *)(m->dt_bias + (size_t)slot * nV), p->Bt, p->Gt, (int32_t)nV,
                 (int32_t)(rows * nV));
        l.launch("ChunkDeltaNet", (uint32_t)(nV * 4), p->O, (const float *)p->Mx, s->S + (size_t)slot * nV * 128 * 128, (const float *)p->Bt,
                 (const float *)p->Gt, (int32_t)nK, (int32_t)nV, (int32_t)rows,
                 (float *)(verify ? p->SnapS + (size_t)slot * nV * 128 * 128 : nullptr), (int64_t)p->snap_s_stride);
        l.launch("GatedNormQuant", (uint32_t)((rows * nV + 3) / 4), (const float *)p->O, (const float *)p->Z,
                 (const float *)(m->lin_norm + (size_t)slot * c.lin_head_dim), p->Q8, p->SQ, (float *)nullptr, (int32_t)(rows * nV), eps);
        l.gemm(m->tensor(pf + "linear_attn.out_proj.weight"), p->Q8, p->SQ, ep.Add, VD, rows);
      }
      if (l.status) break;
      if (l.recording) {
        l.cut(true);
      } else {
        // x = (x + mixer) + MoE(norm(x + mixer)) for the rows; rows past `rows` hold stale values and are ignored
        int e = ep.run_layer(L, true, nullptr);
        if (e) { s->err = "prefill: " + ep.err; return e; }
      }
    }
    if (verify && !l.status) {
      // every row's greedy prediction: final norm, LM head over the rows, argmax per row (no control advance)
      l.launch("RmsNormQuant", (uint32_t)rows, (const float *)ep.Res, (const float *)nullptr, (float *)nullptr,
               (const float *)m->final_norm, (float *)nullptr, p->Q8, p->SQ, (int32_t)H, eps);
      l.gemm(m->tensor("lm_head.weight"), p->Q8, p->SQ, p->Logits, H, rows);
      l.launch("BatchArgmax", (uint32_t)rows, (const float *)p->Logits, p->OutT, p->Ctrl, (int32_t)c.vocab, (int32_t)0);
    }
    if (l.recording) l.cut(false);
    return l.status;
  };
  std::vector<int32_t> ctrl((size_t)p->rows_cap * 4);
  const bool use_lists = verify && n == p->rows_cap;
  if (use_lists && p->vlists.empty()) {
    Launcher rec{p};
    rec.recording = true;
    rec.cut(true);
    int e = pass(rec, n);
    if (e || (int)p->vlists.size() != c.layers + 1) {
      if (!e) { s->err = "internal: verification lists"; e = 3; }
      for (ainfer_list_t q : p->vlists) ainfer_list_destroy(q);
      p->vlists.clear();
      return e;
    }
  }
  for (int t0 = 0; t0 < n; t0 += p->rows_cap) {
    const int rows = std::min(p->rows_cap, n - t0);
    for (int i = 0; i < rows; ++i) {
      ctrl[4 * i] = tokens[t0 + i];
      ctrl[4 * i + 1] = start_pos + t0 + i;
      ctrl[4 * i + 2] = start_pos + t0 + i + 1;
      ctrl[4 * i + 3] = -1;
    }
    if (ainfer_memcpy_h2d(s->dev, p->Ctrl, ctrl.data(), (size_t)rows * 16) != AINFER_OK) { s->err = ainfer_last_error(s->dev); return 1; }
    if (use_lists) {
      for (int L = 0; L < c.layers; ++L) {
        if (ainfer_list_execute(p->vlists[L]) != AINFER_OK) { s->err = ainfer_last_error(s->dev); return 1; }
        int e = ep.run_layer(L, true, nullptr);
        if (e) { s->err = "prefill: " + ep.err; return e; }
      }
      if (ainfer_list_execute(p->vlists[c.layers]) != AINFER_OK) { s->err = ainfer_last_error(s->dev); return 1; }
    } else {
      Launcher l{p};
      int e = pass(l, rows);
      if (e) return e;
    }
  }
  if (verify) {
    if (ainfer_memcpy_d2h(s->dev, predictions, p->OutT, (size_t)n * 4) != AINFER_OK) { s->err = ainfer_last_error(s->dev); return 1; }
  } else if (ainfer_sync(s->dev, UINT64_MAX) != AINFER_OK) { s->err = ainfer_last_error(s->dev); return 1; }
  return 0;
}

// Copies row `row`'s final residual of the last verifying pass to dst (H floats, device).
int prefill_row_hidden(Prefill *p, int row, float *dst) {
  Session *s = p->s;
  const int H = s->m->cfg.hidden;
  if (row < 0 || row >= p->last_rows) { s->err = "usage: no such row"; return 2; }
  if (ainfer_memcpy_d2d(s->dev, dst, p->ep.Res + (size_t)row * H, (size_t)H * 4) != AINFER_OK) { s->err = ainfer_last_error(s->dev); return 1; }
  return 0;
}

// After a verifying prefill_run of r rows: makes the session's DeltaNet state and conv history those
// after the first `keep` rows (1 <= keep <= r).
int prefill_rollback(Prefill *p, int keep) {
  Session *s = p->s;
  if (!p->SnapS || keep < 1 || keep > p->last_rows) { s->err = "usage: nothing to roll back to"; return 2; }
  if (keep < p->last_rows) {
    if (ainfer_memcpy_d2d(s->dev, s->S, p->SnapS + (size_t)(keep - 1) * p->snap_s_stride, p->snap_s_stride * 4) != AINFER_OK ||
        ainfer_memcpy_d2d(s->dev, s->conv, p->SnapC + (size_t)(keep - 1) * p->snap_c_stride, p->snap_c_stride * 4) != AINFER_OK) {
      s->err = ainfer_last_error(s->dev);
      return 1;
    }
  }
  return 0;
}

}  // namespace ainfer
