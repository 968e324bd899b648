// Device-side token sampler with the semantics of the reference's host sampler
// (tools/sample/sampler.h:16-62 parameters, :27-45 repetition penalty, :47-56 xorshift64* stream,
// :60-158 sample_token): greedy first-max-wins for temp <= 0; otherwise softmax in double with the
// maximum subtracted, top-k (k most probable, ties to the lower index), top-p (shortest prefix of
// the sorted distribution whose mass reaches p, ties to the lower index), renormalisation after
// each filter, and an inverse-CDF draw in index order from the same 53-bit uniform stream. The
// logits never leave the device: 4 bytes come back instead of 4 V.
//
// One block of 1024 threads. Selection by rank is a radix select over the probabilities' bit
// patterns (non-negative doubles order like unsigned integers): eight passes of 256-bin
// histograms, which for top-p also carry each bin's mass as a 62-bit fixed-point integer (integer
// sums do not depend on the order of the additions, so the cut is the same on every run). Other sums are block-tree sums, not the host's
// index-order sums, so a draw that lands within rounding of a CDF step may pick the neighbouring
// token; everything else (support of top-k / top-p, tie rules, the stream of uniforms) is identical.
#include "tail_core.cuh"

namespace ainfer {

struct SampleTokenArgs {
  const float *Logits;    // [V]
  const int32_t *Seen;    // [nseen] ids for the repetition penalty (may be null when nseen == 0)
  double *Work;           // [V] scratch: probabilities
  unsigned char *Mark;    // [V] scratch
  unsigned long long *Rng;// [1] xorshift64* state, advanced by one draw when temp > 0
  int32_t *OutT;          // [1] selected token
  float *Probs;           // optional [V]: the final distribution
  int32_t *Ctrl;          // optional control block: {token, position + 1, length + 1, token}
  int32_t V, nseen;
  float temp;
  int32_t top_k;
  float top_p, rep_penalty;
};

constexpr int kSampThreads = 1024;
constexpr double kFix = 4611686018427387904.0;   // 2^62

__device__ __forceinline__ double block_sum(double v, double *sh) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(kFull, v, off);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  double t = 0.0;
  for (int w = 0; w < kSampThreads / 32; ++w) t += sh[w];   // same order in every thread
  return t;
}
// Exclusive scan over the threads (thread order = index order for contiguous chunks); total in *tot.
template <typename T>
__device__ __forceinline__ T block_excl_scan(T v, T *sh, T *tot) {
  __syncthreads();
  sh[threadIdx.x] = v;
  __syncthreads();
  T acc = 0;
  // 1024 values: serial per warp leader, then broadcast; simple and exact in thread order
  if (threadIdx.x < 32) {
    T run = 0;
    for (int i = 0; i < 32; ++i) run += sh[threadIdx.x * 32 + i];
    sh[kSampThreads + threadIdx.x] = run;
  }
  __syncthreads();
  const int w = threadIdx.x >> 5;
  for (int i = 0; i < w; ++i) acc += sh[kSampThreads + i];
  for (int i = w * 32; i < (int)threadIdx.x; ++i) acc += sh[i];
  if (tot) {
    T t = 0;
    for (int i = 0; i < 32; ++i) t += sh[kSampThreads + i];
    *tot = t;
  }
  return acc;
}

__global__ void __launch_bounds__(kSampThreads) SampleToken(const SampleTokenArgs a) {
  __shared__ double shd[kSampThreads + 32];
  __shared__ unsigned long long shu[kSampThreads + 32];
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ unsigned int hist[256];
  __shared__ unsigned long long hmass[256];   // bin mass in units of 2^-62
  __shared__ unsigned long long s_prefix;
  __shared__ long long s_need;
  __shared__ unsigned long long s_cum;         // mass above the threshold, same units
  __shared__ int s_flag, s_chosen;
  __shared__ double s_u;
  const int tid = threadIdx.x, V = a.V;
  const int chunk = (V + kSampThreads - 1) / kSampThreads, lo = tid * chunk, hi = lo + chunk < V ? lo + chunk : V;
  const bool penal = a.rep_penalty > 1.0f && a.nseen > 0;
  // ---- repetition penalty: every seen id once ----
  if (penal) {
    for (int i = tid; i < V; i += kSampThreads) a.Mark[i] = 0;
    __syncthreads();
    for (int i = tid; i < a.nseen; i += kSampThreads) {
      const int id = a.Seen[i];
      if (id >= 0 && id < V) a.Mark[id] = 1;
    }
    __syncthreads();
  }
  auto logit = [&](int i) {
    float l = a.Logits[i];
    if (penal && a.Mark[i]) l = l > 0 ? l / a.rep_penalty : l * a.rep_penalty;
    return l;
  };
  // ---- maximum (and the greedy answer) ----
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  for (int i = tid; i < V; i += kSampThreads) argmax_merge(bv, bi, logit(i), i);
  block_argmax(bv, bi, sv, si);
  if (tid == 0) { sv[0] = bv; si[0] = bi; }
  __syncthreads();
  const float top = sv[0];
  int chosen = si[0];
  if (a.temp <= 0.0f) {
    if (a.Probs) for (int i = tid; i < V; i += kSampThreads) a.Probs[i] = i == chosen ? 1.0f : 0.0f;
  } else {
    // ---- softmax in double ----
    double part = 0.0;
    for (int i = lo; i < hi; ++i) {
      const double p = exp(((double)logit(i) - (double)top) / (double)a.temp);
      a.Work[i] = p;
      part += p;
    }
    double z = block_sum(part, shd);
    for (int i = lo; i < hi; ++i) a.Work[i] = a.Work[i] / z;
    __syncthreads();
    // ---- filters: keep the `need_count` most probable (top-k), or the shortest prefix of mass >= top_p ----
    for (int filter = 0; filter < 2; ++filter) {
      const bool by_count = filter == 0;
      if (by_count ? !(a.top_k > 0 && a.top_k < V) : !(a.top_p < 1.0f)) continue;
      if (tid == 0) { s_prefix = 0ull; s_need = by_count ? a.top_k : 0; s_cum = 0ull; s_flag = 0; }
      __syncthreads();
      // radix select, most significant byte first: after the loop s_prefix is the threshold key T,
      // s_need (top-k) the number of entries equal to T to keep, s_cum (top-p) the mass above T
      for (int pass = 7; pass >= 0 && !s_flag; --pass) {
        for (int b = tid; b < 256; b += kSampThreads) { hist[b] = 0u; hmass[b] = 0ull; }
        __syncthreads();
        const unsigned long long prefix = s_prefix;
        const unsigned long long himask = pass == 7 ? 0ull : ~0ull << (8 * (pass + 1));
        for (int i = lo; i < hi; ++i) {
          const double p = a.Work[i];
          const unsigned long long key = (unsigned long long)__double_as_longlong(p);
          if ((key & himask) == (prefix & himask)) {
            const unsigned b = (unsigned)(key >> (8 * pass)) & 0xFFu;
            atomicAdd(&hist[b], 1u);
            if (!by_count) atomicAdd(&hmass[b], (unsigned long long)(p * kFix));
          }
        }
        __syncthreads();
        if (tid == 0) {
          int b = 255;
          if (by_count) {
            long long need = s_need;
            for (; b > 0; --b) {
              if ((long long)hist[b] >= need) break;
              need -= hist[b];
            }
            s_need = need;
          } else {
            unsigned long long cum = s_cum;
            const unsigned long long want = (unsigned long long)((double)a.top_p * kFix);
            bool found = false;
            for (; b >= 0; --b) {
              if (hist[b] && cum + hmass[b] >= want) { found = true; break; }
              cum += hmass[b];
            }
            if (!found) { s_flag = 1; b = 0; }   // the whole distribution does not reach top_p (rounding): keep everything
            s_cum = cum;
          }
          s_prefix = prefix | ((unsigned long long)b << (8 * pass));
        }
        __syncthreads();
      }
      const bool keep_all = s_flag != 0;
      const unsigned long long T = s_prefix;
      long long need_eq;
      if (by_count) {
        need_eq = s_need;
      } else {
        // ties at the threshold all have probability pT: as many as it takes to reach top_p, at least one
        const double pT = __longlong_as_double((long long)T);
        const double rest = (double)a.top_p - (double)s_cum / kFix;
        need_eq = pT > 0.0 ? (long long)ceil(rest / pT) : 1;
        if (need_eq < 1) need_eq = 1;
      }
      // entries equal to T are kept in index order: rank among equals by an exclusive scan over the chunks
      long long mine = 0;
      for (int i = lo; i < hi; ++i) mine += (unsigned long long)__double_as_longlong(a.Work[i]) == T;
      long long before = (long long)block_excl_scan<unsigned long long>((unsigned long long)mine, shu, nullptr);
      double part2 = 0.0;
      for (int i = lo; i < hi; ++i) {
        const double p = a.Work[i];
        const unsigned long long key = (unsigned long long)__double_as_longlong(p);
        bool keep = keep_all || key > T;
        if (key == T) {
          if (before < need_eq) keep = true;
          ++before;
        }
        if (keep) part2 += p; else a.Work[i] = 0.0;
      }
      const double total = block_sum(part2, shd);
      for (int i = lo; i < hi; ++i) a.Work[i] = a.Work[i] / total;
      __syncthreads();
    }
    // ---- inverse-CDF draw in index order ----
    if (tid == 0) {
      unsigned long long s = *a.Rng;
      s ^= s >> 12; s ^= s << 25; s ^= s >> 27;
      *a.Rng = s;
      s_u = (double)((s * 2685821657736338717ull) >> 11) * (1.0 / 9007199254740992.0);
      s_chosen = V - 1;
    }
    double part3 = 0.0;
    for (int i = lo; i < hi; ++i) part3 += a.Work[i];
    double base = block_excl_scan<double>(part3, shd, nullptr);
    __syncthreads();
    const double u = s_u;
    int first = 0x7FFFFFFF;
    double acc = base;
    for (int i = lo; i < hi; ++i) {
      acc += a.Work[i];
      if (u < acc) { first = i; break; }
    }
    if (first != 0x7FFFFFFF) atomicMin(&s_chosen, first);
    __syncthreads();
    chosen = s_chosen;
    if (a.Probs) for (int i = tid; i < V; i += kSampThreads) a.Probs[i] = (float)a.Work[i];
  }
  if (tid == 0) {
    a.OutT[0] = chosen;
    if (a.Ctrl) {
      a.Ctrl[CTRL_SELECTED] = chosen;
      a.Ctrl[CTRL_TOKEN] = chosen;
      a.Ctrl[CTRL_POS] = a.Ctrl[CTRL_POS] + 1;
      a.Ctrl[CTRL_LEN] = a.Ctrl[CTRL_LEN] + 1;
    }
  }
}

#define F(f) AINFER_ARG(SampleTokenArgs, f)
AINFER_REGISTER(SampleToken, SampleTokenArgs, kSampThreads, 0, 0, nullptr, F(Logits), F(Seen), F(Work), F(Mark), F(Rng), F(OutT), F(Probs),
                F(Ctrl), F(V), F(nseen), F(temp), F(top_k), F(top_p), F(rep_penalty));
#undef F

}  // namespace ainfer
