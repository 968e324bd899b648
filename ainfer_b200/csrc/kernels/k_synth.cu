// Device-side synthetic model generation: value(i) = std * N(0,1) drawn from
// (seed, FNV-1a(tensor name), i), then the container's weight quantiser
// (INT4 symmetric, group 128, BF16 scales; tools/binfer.py:76-91 of the
// reference) or a BF16 store. Bit-identical to the host writer in
// runtime/synth.cpp, so an 80B-parameter-shaped model can be filled in HBM
// directly instead of being written to and read from a 40 GB file.
#include "common.cuh"

namespace ainfer {

struct SynthInt4Args {
  uint8_t *P;        // packed nibbles, 64 bytes per group
  uint16_t *S;       // bf16 scale per group
  uint64_t key;      // stream_key(seed, fnv1a(name))
  uint64_t groups;   // numel / 128
  float std_;
};
__global__ void __launch_bounds__(256) SynthInt4(const SynthInt4Args a) {
  const int lane = threadIdx.x & 31;
  const uint64_t warps = (uint64_t)gridDim.x * 8, warp = (uint64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  for (uint64_t g = warp; g < a.groups; g += warps) {
    float v[4];
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] = a.std_ * normal_from_u32(draw_u32_key(a.key, g * 128 + lane * 4 + j));
      amax = fmaxf(amax, fabsf(v[j]));
    }
    amax = warp_max(amax);
    float sc = amax == 0.0f ? 1.0f : amax / 7.0f;
    if (lane == 0) a.S[g] = f32_to_bf16(sc);
    uint32_t out = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int q = (int)rintf(v[j] / sc);
      q = q < -8 ? -8 : (q > 7 ? 7 : q);
      out |= (uint32_t)(q & 0xF) << (4 * j);
    }
    reinterpret_cast<uint16_t *>(a.P)[g * 32 + lane] = (uint16_t)out;
  }
}
#define F(f) AINFER_ARG(SynthInt4Args, f)
AINFER_REGISTER(SynthInt4, SynthInt4Args, 256, 0, 0, nullptr, F(P), F(S), F(key), F(groups), F(std_));
#undef F

struct SynthBf16Args {
  uint16_t *Out;
  uint64_t key;
  uint64_t numel;
  float std_;
  float constant;    // used when std_ == 0
};
__global__ void __launch_bounds__(256) SynthBf16(const SynthBf16Args a) {
  for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < a.numel;
       i += (uint64_t)gridDim.x * 256) {
    float v = a.std_ == 0.0f ? a.constant : a.std_ * normal_from_u32(draw_u32_key(a.key, i));
    a.Out[i] = f32_to_bf16(v);
  }
}
#define F(f) AINFER_ARG(SynthBf16Args, f)
AINFER_REGISTER(SynthBf16, SynthBf16Args, 256, 0, 0, nullptr, F(Out), F(key), F(numel), F(std_),
                F(constant));
#undef F

// Widens a BF16 tensor to fp32 (the reference's load_small does this on the
// host, tools/decode/decode_l0.cpp:301-316).
struct WidenBf16Args {
  float *Out;
  const uint16_t *In;
  uint64_t numel;
};
__global__ void __launch_bounds__(256) WidenBf16(const WidenBf16Args a) {
  for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < a.numel;
       i += (uint64_t)gridDim.x * 256)
    a.Out[i] = bf16_to_f32(a.In[i]);
}
#define F(f) AINFER_ARG(WidenBf16Args, f)
AINFER_REGISTER(WidenBf16, WidenBf16Args, 256, 0, 0, nullptr, F(Out), F(In), F(numel));
#undef F

struct SynthF32Args {
  float *Out;
  uint64_t key;
  uint64_t numel;
  float std_;
};
__global__ void __launch_bounds__(256) SynthF32(const SynthF32Args a) {
  for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < a.numel;
       i += (uint64_t)gridDim.x * 256)
    a.Out[i] = a.std_ * normal_from_u32(draw_u32_key(a.key, i));
}
#define F(f) AINFER_ARG(SynthF32Args, f)
AINFER_REGISTER(SynthF32, SynthF32Args, 256, 0, 0, nullptr, F(Out), F(key), F(numel), F(std_));
#undef F

}  // namespace ainfer
