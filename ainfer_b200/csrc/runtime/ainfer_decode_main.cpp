// ainfer_decode: the decode CLI. Keeps the process contract of the reference's
// decode_l0 (tools/decode/decode_l0.cpp:66-123 argv/env, :742-825 token loop
// and stdout lines, :827-869 JSON report, :870-893 profile and dump, exit codes
// 0/1/2/3) so that its process-level callers (tools/http/ainfer_http.py,
// tools/e2e/run_e2e.py, tools/stress/run_stress.py, tools/sweep/run_sweep.py)
// can point at this binary instead.
//
//   ainfer_decode <model|synth:preset[:seed=N]> <P> <G> [kernel-dir] [report]
//                 [--ids=a,b,..] [--max-new=N] [--temp=T] [--top-k=K] [--top-p=P]
//                 [--seed=S] [--rep-penalty=R] [--eos=a,b] [--device=N]
//   env: AINFER_MAXCTX, AINFER_PROFILE, AINFER_TOP5, AINFER_DUMP0
// The fourth positional (the reference's SPIR-V directory) is accepted and
// ignored: kernels are linked into the library.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "executor.h"
#include "host_sampler.h"
#include "model.h"

using namespace ainfer;

static std::vector<int> parse_ids(const char *q) {
  std::vector<int> v;
  while (*q) {
    v.push_back(atoi(q));
    while (*q && *q != ',') ++q;
    if (*q == ',') ++q;
  }
  return v;
}

int main(int argc, char **argv) {
  std::vector<int> opt_ids, eos = {248046, 248044};  // the reference's EOS pair, configurable
  int opt_max_new = -1, device = 0;
  SampleParams samp;
  std::vector<const char *> pos;
  for (int i = 1; i < argc; ++i) {
    const char *a = argv[i];
    if (!std::strncmp(a, "--ids=", 6)) opt_ids = parse_ids(a + 6);
    else if (!std::strncmp(a, "--max-new=", 10)) opt_max_new = atoi(a + 10);
    else if (!std::strncmp(a, "--temp=", 7)) samp.temp = (float)atof(a + 7);
    else if (!std::strncmp(a, "--top-k=", 8)) samp.top_k = atoi(a + 8);
    else if (!std::strncmp(a, "--top-p=", 8)) samp.top_p = (float)atof(a + 8);
    else if (!std::strncmp(a, "--seed=", 7)) samp.seed = (uint64_t)atoll(a + 7);
    else if (!std::strncmp(a, "--rep-penalty=", 14)) samp.rep_penalty = (float)atof(a + 14);
    else if (!std::strncmp(a, "--eos=", 6)) eos = parse_ids(a + 6);
    else if (!std::strncmp(a, "--device=", 9)) device = atoi(a + 9);
    else if (!std::strncmp(a, "--spvdir=", 9)) { /* accepted for compatibility */ }
    else pos.push_back(a);
  }
  if (pos.size() < 3) {
    std::fprintf(stderr, "usage: ainfer_decode <model> <P> <G> [kernel-dir] [report] [--ids=..] [--max-new=..]\n");
    return 2;
  }
  const char *path = pos[0];
  int P = atoi(pos[1]), G = atoi(pos[2]);
  if (!opt_ids.empty()) P = (int)opt_ids.size();
  if (opt_max_new >= 0) G = opt_max_new;
  if (P < 1) { std::fprintf(stderr, "usage: P must be >= 1\n"); return 2; }
  int MAXCTX = P + G + 8;  // grow-only override, decode_l0.cpp:118-123
  if (const char *mx = std::getenv("AINFER_MAXCTX")) MAXCTX = std::max(MAXCTX, std::atoi(mx));

  const bool prof = std::getenv("AINFER_PROFILE") != nullptr;
  const char *top5e = std::getenv("AINFER_TOP5");
  const bool wantTop5 = !(top5e && top5e[0] == '0');
  const bool needLogits = wantTop5 || samp.temp > 0;
  const char *dump0 = std::getenv("AINFER_DUMP0");

  ainfer_device_t dev = nullptr;
  int rc = ainfer_device_open(device, &dev);
  if (rc != AINFER_OK) {
    std::fprintf(stderr, "device error %d (%s)\n", rc, ainfer_last_error(nullptr));
    return rc == AINFER_ERR_NO_DEVICE ? 2 : 1;
  }
  std::string err;
  DeviceModel *model = nullptr;
  rc = model_open(dev, path, VALIDATE_SPANS, &model, err);
  if (rc) { std::fprintf(stderr, "%s\n", err.c_str()); return rc; }
  const ModelConfig &cfg = model->cfg;
  const int V = cfg.vocab, H = cfg.hidden;

  int flags = 0;
  if (dump0) flags |= SESSION_DIAG;
  if (prof) flags |= SESSION_PER_LAYER_LISTS;
  Session *s = nullptr;
  rc = session_create(model, MAXCTX, flags, &s, err);
  if (rc) { std::fprintf(stderr, "%s\n", err.c_str()); return rc; }
  s->profile = prof;
  std::fprintf(stderr, "[cuda] recorded %d layers, %llu launches per token\n", cfg.layers,
               (unsigned long long)s->launches_per_token);

  // default prompt: the reference's 24-token template clipped to the vocabulary
  std::vector<int> ids = {248045, 846, 198, 3710, 369, 220, 23, 19, 348, 220, 18, 593,
                          220, 17, 30, 248046, 198, 248045, 74455, 198, 248068, 271, 248069, 271};
  if (!opt_ids.empty()) ids = opt_ids;
  else if ((int)ids.size() > P) ids.resize(P);
  else while ((int)ids.size() < P) ids.push_back(198);
  for (int &t : ids) t = ((t % V) + V) % V;
  ids.reserve((size_t)P + (size_t)G + 1);

  std::vector<int> generated;
  std::vector<std::vector<int>> tops5;
  std::vector<std::vector<float>> tops5v;
  std::vector<float> lg((size_t)V), lgS, dump;
  std::vector<int> lidx((size_t)V);
  uint64_t samp_rng = samp.seed;
  bool stopped_eos = false;
  auto is_eos = [&](int t) { return std::find(eos.begin(), eos.end(), t) != eos.end(); };

  // prompt steps 0..P-2 need no logits (decode_l0.cpp:771)
  if (P > 1) {
    rc = session_generate(s, ids.data(), P, 0, 0, nullptr, nullptr);
    if (rc) { std::fprintf(stderr, "%s\n", s->err.c_str()); return rc; }
  }
  if (!needLogits && !prof && !dump0) {
    // token-only steady state: device-advanced control block, tokens read back in blocks
    int step = P - 1, last = ids[(size_t)P - 1];
    const int BLK = 16;
    std::vector<int> out((size_t)BLK);
    while (step < P + G && !stopped_eos) {
      int n = std::min(BLK, P + G - step);
      rc = session_generate(s, &last, 1, n, step, out.data(), nullptr);
      if (rc) { std::fprintf(stderr, "%s\n", s->err.c_str()); return rc; }
      for (int i = 0; i < n; ++i) {
        generated.push_back(out[(size_t)i]);
        if (step + i < P + G - 1) ids.push_back(out[(size_t)i]);
        std::printf("step %d pos %d -> token %d\n", step + i, step + i, out[(size_t)i]);
        if (is_eos(out[(size_t)i])) { stopped_eos = true; break; }
      }
      step += n;
      last = out[(size_t)n - 1];
    }
  } else {
    for (int step = P - 1; step < P + G; ++step) {
      if (step >= MAXCTX) {
        std::fprintf(stderr, "context overflow: pos %d >= MAXCTX %d\n", step, MAXCTX);
        return 3;
      }
      if ((int)ids.size() <= step) { std::fprintf(stderr, "internal: missing id at step %d\n", step); return 3; }
      int tok = -1;
      rc = session_step(s, ids[(size_t)step], step, &tok);
      if (rc) { std::fprintf(stderr, "%s\n", s->err.c_str()); return rc; }
      if (dump0 && dump.empty() && s->layer_out) {
        dump.resize((size_t)cfg.layers * H);
        ainfer_memcpy_d2h(dev, dump.data(), s->layer_out, dump.size() * 4);
      }
      if (needLogits) {
        if (ainfer_memcpy_d2h(dev, lg.data(), s->Logits, (size_t)V * 4) != AINFER_OK) {
          std::fprintf(stderr, "device error (%s)\n", ainfer_last_error(dev));
          return 1;
        }
      }
      if (wantTop5) {
        for (int i = 0; i < V; ++i) lidx[(size_t)i] = i;
        int n5 = std::min(5, V);
        std::partial_sort(lidx.begin(), lidx.begin() + n5, lidx.end(),
                          [&](int a, int b) { return lg[(size_t)a] > lg[(size_t)b]; });
        double mn = 0, sd = 0;
        for (float v : lg) mn += v;
        mn /= (double)lg.size();
        for (float v : lg) sd += (v - mn) * (v - mn);
        sd = std::sqrt(sd / (double)lg.size());
        std::printf("TOP5@s%d: ", step);
        for (int i = 0; i < n5; ++i) std::printf("%d(%.3f) ", lidx[(size_t)i], lg[(size_t)lidx[(size_t)i]]);
        std::printf("| mean %.3f std %.3f\n", mn, sd);
        tops5.emplace_back(lidx.begin(), lidx.begin() + n5);
        tops5v.emplace_back();
        for (int i = 0; i < n5; ++i) tops5v.back().push_back(lg[(size_t)lidx[(size_t)i]]);
      }
      if (samp.temp > 0) {
        lgS = lg;
        apply_rep_penalty(lgS, ids.data(), (int)ids.size(), samp.rep_penalty);
        tok = sample_token(lgS.data(), V, samp, samp_rng);
        std::printf("sampled (t=%.2f,k=%d,p=%.2f,rep=%.2f,seed=%llu)\n", samp.temp, samp.top_k,
                    samp.top_p, samp.rep_penalty, (unsigned long long)samp.seed);
      }
      generated.push_back(tok);
      if (step < P + G - 1) ids.push_back(tok);
      std::printf("step %d pos %d -> token %d\n", step, step, tok);
      if (is_eos(tok)) { stopped_eos = true; break; }
    }
  }

  char sbuf[256];
  std::snprintf(sbuf, sizeof sbuf,
                "{\"device\":\"B200\",\"backend\":\"cuda-graph\",\"sampling\":{\"temp\":%.3f,\"top_k\":%d,"
                "\"top_p\":%.3f,\"rep_penalty\":%.3f,\"seed\":%llu},\"prompt\":[",
                samp.temp, samp.top_k, samp.top_p, samp.rep_penalty, (unsigned long long)samp.seed);
  std::string json = sbuf;
  for (size_t i = 0; i < ids.size() && i < (size_t)P; ++i) json += (i ? "," : "") + std::to_string(ids[i]);
  json += "],\"generated\":[";
  for (size_t i = 0; i < generated.size(); ++i) json += (i ? "," : "") + std::to_string(generated[i]);
  json += "],\"stopped_eos\":";
  json += stopped_eos ? "true" : "false";
  json += ",\"top5_per_step\":[";
  for (size_t k = 0; k < tops5.size(); ++k) {
    json += (k ? "," : "") + std::string("{\"step\":") + std::to_string(P - 1 + (int)k) + ",\"top5\":[";
    for (size_t i = 0; i < tops5[k].size(); ++i) json += (i ? "," : "") + std::to_string(tops5[k][i]);
    json += "],\"top5v\":[";
    char vb[64];
    for (size_t i = 0; i < tops5v[k].size(); ++i) {
      std::snprintf(vb, sizeof vb, "%s%.4f", i ? "," : "", tops5v[k][i]);
      json += vb;
    }
    json += "]}";
  }
  json += "]}";
  FILE *o = stdout;
  if (pos.size() > 4) {
    o = std::fopen(pos[4], "w");
    if (!o) return 1;
  }
  std::fprintf(o, "%s\n", json.c_str());
  if (o != stdout) std::fclose(o);
  std::printf("generated: ");
  for (int t : generated) std::printf("%d ", t);
  std::printf("\n");
  if (prof) {
    std::fprintf(stderr, "%-12s %6s %10s %10s %10s\n", "class", "n", "total_ms", "mean_ms", "med_ms");
    for (auto &kv : s->buckets) {
      auto &v = kv.second;
      if (v.empty()) continue;
      std::sort(v.begin(), v.end());
      double tot = 0;
      for (double x : v) tot += x;
      std::fprintf(stderr, "%-12s %6zu %10.2f %10.3f %10.3f\n", kv.first.c_str(), v.size(), tot / 1e6,
                   tot / (double)v.size() / 1e6, v[v.size() / 2] / 1e6);
    }
  }
  if (dump0 && !dump.empty()) {
    if (FILE *df = std::fopen(dump0, "wb")) {
      std::fwrite(dump.data(), 4, dump.size(), df);
      std::fclose(df);
      std::printf("dumped %zu floats -> %s\n", dump.size(), dump0);
    }
  }
  session_destroy(s);
  model_close(model);
  ainfer_device_close(dev);
  return 0;
}
