// TEST INFRASTRUCTURE ONLY. Flat C entry points over the reference's own host
// sampler header, compiled from the reference checkout where it lies (the
// header is included by path, never copied). Used to pin the runtime's sampler
// and to generate the committed sampler fixtures.
#include <cstdint>
#include <vector>

#include "sampler.h"  // <reference>/tools/sample/sampler.h via -I

extern "C" {
int ref_sample_token(const float *logits, int V, float temp, int top_k, float top_p,
                     float rep_penalty, uint64_t seed, uint64_t *rng, float *probs_out) {
  SampleParams p;
  p.temp = temp; p.top_k = top_k; p.top_p = top_p; p.rep_penalty = rep_penalty; p.seed = seed;
  std::vector<float> probs;
  int r = sample_token(logits, V, p, *rng, probs_out ? &probs : nullptr);
  if (probs_out)
    for (int i = 0; i < V; ++i) probs_out[i] = probs[i];
  return r;
}
void ref_apply_rep_penalty(float *logits, int V, const int *seen, int nseen, float penalty) {
  std::vector<float> l(logits, logits + V);
  apply_rep_penalty(l, seen, nseen, penalty);
  for (int i = 0; i < V; ++i) logits[i] = l[i];
}
uint64_t ref_xrs64(uint64_t *s) { return xrs64(*s); }
double ref_xrunif(uint64_t *s) { return xrunif(*s); }
}
