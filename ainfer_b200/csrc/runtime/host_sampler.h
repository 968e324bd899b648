// Host sampler of the decode runtime. Interface and semantics of the
// reference's tools/sample/sampler.h (SampleParams :16-22, apply_rep_penalty
// :27-45, xorshift64* :47-56, sample_token :60-158): greedy first-max-wins for
// temp <= 0; otherwise softmax in double with the maximum subtracted, top-k
// (k largest, ties to the lower index), top-p (shortest prefix of the sorted
// distribution reaching p), renormalisation after each filter with sums taken
// in index order, and an inverse-CDF draw in index order from a 53-bit uniform.
// Header-only, caller owns all buffers, not thread-safe across a shared rng.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <numeric>
#include <vector>

struct SampleParams {
  float temp = 0.0f;         // <= 0: greedy
  int top_k = 0;             // <= 0: off
  float top_p = 1.0f;        // >= 1: off
  float rep_penalty = 1.0f;  // <= 1: off
  uint64_t seed = 0;
};

// Divides positive / multiplies non-positive logits of every id seen so far.
static inline void apply_rep_penalty(std::vector<float> &logits, const int *seen, int nseen,
                                     float penalty) {
  if (!(penalty > 1.0f) || nseen <= 0) return;
  const int V = (int)logits.size();
  std::vector<unsigned char> mark((size_t)V, 0);
  for (int i = 0; i < nseen; ++i) {
    int id = seen[i];
    if (id >= 0 && id < V) mark[(size_t)id] = 1;
  }
  for (int id = 0; id < V; ++id) {
    if (!mark[(size_t)id]) continue;
    float &l = logits[(size_t)id];
    l = l > 0 ? l / penalty : l * penalty;
  }
}

static inline uint64_t xrs64(uint64_t &s) {
  s ^= s >> 12;
  s ^= s << 25;
  s ^= s >> 27;
  return s * 2685821657736338717ull;
}
static inline double xrunif(uint64_t &s) {
  return (double)(xrs64(s) >> 11) * (1.0 / 9007199254740992.0);
}

namespace ainfer_sampler_detail {
// Keeps only the ids flagged in keep and rescales so that they sum to one
// (sum accumulated in ascending id order).
inline void keep_and_renormalise(std::vector<double> &prob, const std::vector<unsigned char> &keep) {
  double total = 0;
  for (size_t i = 0; i < prob.size(); ++i) {
    if (keep[i]) total += prob[i];
    else prob[i] = 0;
  }
  for (double &p : prob) p /= total;
}
}  // namespace ainfer_sampler_detail

static inline int sample_token(const float *logits, int V, const SampleParams &p, uint64_t &rng,
                               std::vector<float> *probs_out = nullptr) {
  if (p.temp <= 0.0f) {
    int arg = 0;
    for (int i = 1; i < V; ++i)
      if (logits[i] > logits[arg]) arg = i;
    if (probs_out) {
      probs_out->assign((size_t)V, 0.0f);
      (*probs_out)[(size_t)arg] = 1.0f;
    }
    return arg;
  }
  double top = logits[0];
  for (int i = 1; i < V; ++i) top = std::max(top, (double)logits[i]);
  std::vector<double> prob((size_t)V);
  double z = 0;
  for (int i = 0; i < V; ++i) {
    prob[(size_t)i] = std::exp(((double)logits[i] - top) / p.temp);
    z += prob[(size_t)i];
  }
  for (double &q : prob) q /= z;

  auto before = [&prob](int a, int b) {
    return prob[(size_t)a] > prob[(size_t)b] || (prob[(size_t)a] == prob[(size_t)b] && a < b);
  };
  std::vector<int> order((size_t)V);
  std::iota(order.begin(), order.end(), 0);
  std::vector<unsigned char> keep;
  if (p.top_k > 0 && p.top_k < V) {
    std::nth_element(order.begin(), order.begin() + p.top_k, order.end(), before);
    keep.assign((size_t)V, 0);
    for (int i = 0; i < p.top_k; ++i) keep[(size_t)order[(size_t)i]] = 1;
    ainfer_sampler_detail::keep_and_renormalise(prob, keep);
  }
  if (p.top_p < 1.0f) {
    std::sort(order.begin(), order.end(), before);
    int cut = V;
    double mass = 0;
    for (int i = 0; i < V; ++i) {
      mass += prob[(size_t)order[(size_t)i]];
      if (mass >= p.top_p) { cut = i + 1; break; }
    }
    cut = std::max(cut, 1);
    keep.assign((size_t)V, 0);
    for (int i = 0; i < cut; ++i) keep[(size_t)order[(size_t)i]] = 1;
    ainfer_sampler_detail::keep_and_renormalise(prob, keep);
  }
  const double u = xrunif(rng);
  int chosen = V - 1;
  double acc = 0;
  for (int i = 0; i < V; ++i) {
    acc += prob[(size_t)i];
    if (u < acc) { chosen = i; break; }
  }
  if (probs_out) {
    probs_out->resize((size_t)V);
    for (int i = 0; i < V; ++i) (*probs_out)[(size_t)i] = (float)prob[(size_t)i];
  }
  return chosen;
}
