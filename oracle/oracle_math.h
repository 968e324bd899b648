// TEST INFRASTRUCTURE ONLY. CPU oracle for the AInfer decode hot path.
// Nothing in the product path (the CUDA library or the C++ runtime) may
// include, link or execute this file; only tests, the smoke check and the
// bench's cpu_baseline / reference arm use it, and only as the checker.
//
// Scalar arithmetic primitives of the oracle. The reference evaluates exp/log
// through the SYCL and libm math libraries (tools/cmdlist/kernels.cpp:35,270,
// 333,612-615), whose last-ulp results differ between device and host; its own
// harnesses absorb that with tolerances (tools/cmdlist/layerlin_replay.cpp:
// 680-687). This restatement fixes every transcendental to a polynomial built
// from IEEE add/mul/fma only, so that a second implementation following the
// same operation order is bit-identical on any IEEE machine. Compile with
// -ffp-contract=off: a fused multiply-add happens only where fmaf is written.
#pragma once
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace orc {

// Small persistent thread pool (std::thread only, no OpenMP runtime needed).
// parallel_for splits [0, n) into contiguous blocks, one per worker; results
// never depend on the split because every index is computed independently.
class Pool {
 public:
  static Pool &get() {
    static Pool p;
    return p;
  }
  int threads() const { return nthreads_; }
  void run(int64_t n, const std::function<void(int64_t, int64_t)> &fn) {
    if (n <= 0) return;
    if (nthreads_ <= 1 || n == 1 || busy_.exchange(true)) {  // nested call: run inline
      fn(0, n);
      return;
    }
    {
      std::lock_guard<std::mutex> lk(mu_);
      fn_ = &fn;
      n_ = n;
      pending_ = nthreads_ - 1;
      ++epoch_;
    }
    cv_.notify_all();
    block(0);
    std::unique_lock<std::mutex> lk(mu_);
    done_cv_.wait(lk, [&] { return pending_ == 0; });
    fn_ = nullptr;
    busy_ = false;
  }

 private:
  Pool() {
    const char *e = std::getenv("ORACLE_THREADS");
    int n = e ? std::atoi(e) : (int)std::thread::hardware_concurrency();
    nthreads_ = n < 1 ? 1 : n;
    for (int i = 1; i < nthreads_; ++i) workers_.emplace_back([this, i] { loop(i); });
  }
  ~Pool() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
      ++epoch_;
    }
    cv_.notify_all();
    for (auto &t : workers_) t.join();
  }
  void block(int i) {
    int64_t per = (n_ + nthreads_ - 1) / nthreads_;
    int64_t a = per * i, b = a + per < n_ ? a + per : n_;
    if (a < b) (*fn_)(a, b);
  }
  void loop(int i) {
    uint64_t seen = 0;
    for (;;) {
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return epoch_ != seen; });
        seen = epoch_;
        if (stop_) return;
      }
      block(i);
      {
        std::lock_guard<std::mutex> lk(mu_);
        --pending_;
      }
      done_cv_.notify_one();
    }
  }
  int nthreads_ = 1;
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable cv_, done_cv_;
  const std::function<void(int64_t, int64_t)> *fn_ = nullptr;
  int64_t n_ = 0;
  int pending_ = 0;
  uint64_t epoch_ = 0;
  bool stop_ = false;
  std::atomic<bool> busy_{false};
};
template <typename F>
static inline void parallel_for(int64_t n, F &&f) {
  Pool::get().run(n, [&](int64_t a, int64_t b) {
    for (int64_t i = a; i < b; ++i) f(i);
  });
}

static inline uint32_t f2u(float x) { uint32_t u; std::memcpy(&u, &x, 4); return u; }
static inline float u2f(uint32_t u) { float x; std::memcpy(&x, &u, 4); return x; }

// BF16 round-to-nearest-even and exact widening (tools/cmdlist/kernels.cpp:17-27,
// tools/binfer.py:65-71).
static inline uint16_t f32_to_bf16(float x) {
  uint32_t u = f2u(x);
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
static inline float bf16_to_f32(uint16_t b) { return u2f((uint32_t)b << 16); }

// IEEE binary16 round-to-nearest-even (scales of the INT8 KV cache). Written
// out by hand so that it does not depend on compiler _Float16 support.
static inline uint16_t f32_to_f16(float x) {
  uint32_t u = f2u(x);
  uint32_t sign = (u >> 16) & 0x8000u;
  uint32_t a = u & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) return (uint16_t)(sign | (a > 0x7F800000u ? 0x7E00u : 0x7C00u));
  if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);  // rounds to inf
  if (a < 0x38800000u) {                                      // subnormal half
    if (a < 0x33000000u) return (uint16_t)sign;               // < 2^-25 -> 0
    int e = (int)(a >> 23);
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    int shift = 126 - e;  // 14..24
    uint32_t h = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1u))) h++;
    return (uint16_t)(sign | h);
  }
  uint32_t h = ((a - 0x38000000u) >> 13);
  uint32_t rem = a & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
  return (uint16_t)(sign | h);
}
static inline float f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
  if (e == 0) {
    if (m == 0) return u2f(sign);
    float v = (float)m * 5.9604644775390625e-8f;  // m * 2^-24, exact
    return sign ? -v : v;
  }
  if (e == 31) return u2f(sign | 0x7F800000u | (m << 13));
  return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

// exp(x): range reduction by ln2 in two pieces, degree-5 polynomial for the
// remainder, power of two applied through the exponent field.
static inline float det_expf(float x) {
  if (x > 88.0f) x = 88.0f;
  if (x < -86.0f) return 0.0f;
  float t = x * 1.44269504088896341f;
  float n = rintf(t);
  float r = fmaf(n, -0.693145751953125f, x);
  r = fmaf(n, -1.42860682030941723212e-6f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  float r2 = r * r;
  float y = fmaf(p, r2, r);
  y = y + 1.0f;
  int ni = (int)n;
  return y * u2f((uint32_t)(ni + 127) << 23);
}

// log(x) for normal positive x: mantissa in [sqrt(1/2), sqrt(2)), degree-8
// polynomial, exponent added back in two pieces.
static inline float det_logf(float x) {
  uint32_t u = f2u(x);
  int e = (int)((u >> 23) & 255u) - 126;
  float m = u2f((u & 0x007FFFFFu) | 0x3F000000u);
  if (m < 0.707106781186547524f) {
    e -= 1;
    m = (m + m) - 1.0f;
  } else {
    m = m - 1.0f;
  }
  float z = m * m;
  float p = 7.0376836292e-2f;
  p = fmaf(p, m, -1.1514610310e-1f);
  p = fmaf(p, m, 1.1676998740e-1f);
  p = fmaf(p, m, -1.2420140846e-1f);
  p = fmaf(p, m, 1.4249322787e-1f);
  p = fmaf(p, m, -1.6668057665e-1f);
  p = fmaf(p, m, 2.0000714765e-1f);
  p = fmaf(p, m, -2.4999993993e-1f);
  p = fmaf(p, m, 3.3333331174e-1f);
  float y = (m * z) * p;
  float fe = (float)e;
  y = fmaf(fe, -2.12194440e-4f, y);
  y = fmaf(-0.5f, z, y);
  float res = m + y;
  return fmaf(fe, 0.693359375f, res);
}

static inline float sigmoidf_det(float x) { return 1.0f / (1.0f + det_expf(-x)); }
// x * sigmoid(x) exactly as the reference writes it: x / (1 + exp(-x))
// (tools/cmdlist/kernels.cpp:35,333,628).
static inline float siluf_det(float x) { return x / (1.0f + det_expf(-x)); }

// Stride-halving sum tree over a power-of-two number of lanes, as the
// reference's shared-memory reduction (tools/cmdlist/kernels.cpp:104-110):
// for st = n/2 .. 1: p[l] += p[l+st] for l < st. Result in p[0].
template <typename T>
static inline T tree_sum(T *p, int n) {
  for (int st = n / 2; st > 0; st >>= 1)
    for (int l = 0; l < st; ++l) p[l] = p[l] + p[l + st];
  return p[0];
}

// 64-bit mixer used by the synthetic-input generator (SplitMix64 finaliser).
static inline uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
static inline uint64_t fnv1a64(const char *s) {
  uint64_t h = 0xCBF29CE484222325ull;
  for (; *s; ++s) { h ^= (uint8_t)*s; h *= 0x100000001B3ull; }
  return h;
}
// Counter-based 32-bit draw: (seed, stream, index) -> u32.
static inline uint32_t draw_u32(uint64_t seed, uint64_t stream, uint64_t idx) {
  uint64_t key = mix64(seed ^ mix64(stream));
  return (uint32_t)(mix64(key + idx) >> 32);
}
// Standard normal from a 32-bit draw by the inverse CDF (Acklam's rational
// approximation, evaluated in fp32 with the operation order written here).
static inline float normal_from_u32(uint32_t r) {
  uint32_t k = r >> 9;                       // 23 bits
  bool upper = k >= (1u << 22);
  uint32_t kk = upper ? ((1u << 23) - 1u - k) : k;
  float p = ((float)kk + 0.5f) * 1.1920928955078125e-7f;  // (kk+0.5) * 2^-23, in (0, 0.5)
  float x;
  if (p < 0.02425f) {
    float q = sqrtf(-2.0f * det_logf(p));
    float num = -7.784894002430293e-03f;
    num = num * q + -3.223964580411365e-01f;
    num = num * q + -2.400758277161838e+00f;
    num = num * q + -2.549732539343734e+00f;
    num = num * q + 4.374664141464968e+00f;
    num = num * q + 2.938163982698783e+00f;
    float den = 7.784695709041462e-03f;
    den = den * q + 3.224671290700398e-01f;
    den = den * q + 2.445134137142996e+00f;
    den = den * q + 3.754408661907416e+00f;
    den = den * q + 1.0f;
    x = num / den;
  } else {
    float q = p - 0.5f;
    float r2 = q * q;
    float num = -3.969683028665376e+01f;
    num = num * r2 + 2.209460984245205e+02f;
    num = num * r2 + -2.759285104469687e+02f;
    num = num * r2 + 1.383577518672690e+02f;
    num = num * r2 + -3.066479806614716e+01f;
    num = num * r2 + 2.506628277459239e+00f;
    float den = -5.447609879822406e+01f;
    den = den * r2 + 1.615858368580409e+02f;
    den = den * r2 + -1.556989798598866e+02f;
    den = den * r2 + 6.680131188771972e+01f;
    den = den * r2 + -1.328068155288572e+01f;
    den = den * r2 + 1.0f;
    x = (num * q) / den;
  }
  return upper ? -x : x;
}

}  // namespace orc
