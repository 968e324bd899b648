// Scalar arithmetic of the decode path, shared by device kernels and by the
// host-side synthetic-model writer. Every transcendental is a fixed polynomial
// over IEEE add/mul/fma, so host and device agree bit for bit. Build rules:
// nvcc -fmad=false and g++ -ffp-contract=off (a fused multiply-add happens only
// where fmaf is written); no fast-math.
//
// The reference evaluates the same functions through sycl::exp / sycl::log
// (tools/cmdlist/kernels.cpp:35,270,333,612-615); its harness tolerances absorb
// the last-ulp differences between its device and host. Here the result is
// defined exactly instead.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define AINFER_HD __host__ __device__ __forceinline__
#else
#define AINFER_HD inline
#endif

namespace ainfer {

AINFER_HD uint32_t f2u(float x) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(x);
#else
  uint32_t u; std::memcpy(&u, &x, 4); return u;
#endif
}
AINFER_HD float u2f(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float x; std::memcpy(&x, &u, 4); return x;
#endif
}

// BF16 RNE and exact widening (tools/cmdlist/kernels.cpp:17-27).
AINFER_HD uint16_t f32_to_bf16(float x) {
  uint32_t u = f2u(x);
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
AINFER_HD float bf16_to_f32(uint16_t b) { return u2f((uint32_t)b << 16); }

// IEEE binary16, round to nearest even, integer-only so host and device match.
AINFER_HD uint16_t f32_to_f16(float x) {
  uint32_t u = f2u(x);
  uint32_t sign = (u >> 16) & 0x8000u;
  uint32_t a = u & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) return (uint16_t)(sign | (a > 0x7F800000u ? 0x7E00u : 0x7C00u));
  if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);
  if (a < 0x38800000u) {
    if (a < 0x33000000u) return (uint16_t)sign;
    int e = (int)(a >> 23);
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    int shift = 126 - e;
    uint32_t h = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1u))) h++;
    return (uint16_t)(sign | h);
  }
  uint32_t h = (a - 0x38000000u) >> 13;
  uint32_t rem = a & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
  return (uint16_t)(sign | h);
}
AINFER_HD float f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
  if (e == 0) {
    if (m == 0) return u2f(sign);
    float v = (float)m * 5.9604644775390625e-8f;
    return sign ? -v : v;
  }
  if (e == 31) return u2f(sign | 0x7F800000u | (m << 13));
  return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

AINFER_HD float det_expf(float x) {
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

AINFER_HD float det_logf(float x) {
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

AINFER_HD float sigmoid_det(float x) { return 1.0f / (1.0f + det_expf(-x)); }
AINFER_HD float silu_det(float x) { return x / (1.0f + det_expf(-x)); }

// Counter-based draws for synthetic models: (seed, stream, index) -> u32,
// stream = FNV-1a of the tensor name.
AINFER_HD uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
inline uint64_t fnv1a64(const char *s) {
  uint64_t h = 0xCBF29CE484222325ull;
  for (; *s; ++s) { h ^= (uint8_t)*s; h *= 0x100000001B3ull; }
  return h;
}
AINFER_HD uint64_t stream_key(uint64_t seed, uint64_t stream) { return mix64(seed ^ mix64(stream)); }
AINFER_HD uint32_t draw_u32_key(uint64_t key, uint64_t idx) { return (uint32_t)(mix64(key + idx) >> 32); }

// Standard normal by the inverse CDF (Acklam's rational approximation in fp32).
AINFER_HD float normal_from_u32(uint32_t r) {
  uint32_t k = r >> 9;
  bool upper = k >= (1u << 22);
  uint32_t kk = upper ? ((1u << 23) - 1u - k) : k;
  float p = ((float)kk + 0.5f) * 1.1920928955078125e-7f;
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

}  // namespace ainfer
