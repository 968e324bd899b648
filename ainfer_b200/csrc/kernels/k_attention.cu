// Kernel entries of the gated GQA decode attention; bodies in attention_core.cuh
// (shared with the persistent decode kernel).
#include "attention_core.cuh"

namespace ainfer {

__global__ void __launch_bounds__(256) AttnPrep(const AttnPrepArgs a) { pdl_launch_dependents(); pdl_wait(); attn_prep_body(a, blockIdx.x, gridDim.x); }
__global__ void __launch_bounds__(256) AttnSplit(const AttnSplitArgs a) {
  pdl_launch_dependents();
  // While the predecessor (which only appends the newest token) runs: start this block's first
  // chunk of the KV cache towards L2, one 128-byte line per thread. The context length is in
  // the control block since the end of the previous step; a stale value would only change what
  // is prefetched (rows stay below max_ctx).
  {
    int T = __ldcg(a.Ctrl + CTRL_LEN);
    if (T > a.max_ctx) T = a.max_ctx;
    const int nch = (T + kAttnChunk - 1) / kAttnChunk, item = blockIdx.x;
    if (item < nch * a.nKV) {
      const int c = item / a.nKV, kv = item % a.nKV, tid = threadIdx.x;
      const int row = (tid & 127) >> 1, t = c * kAttnChunk + row;
      if (t < T) {
        const int8_t *base = (tid < 128 ? a.Kc : a.Vc) + ((size_t)t * a.nKV + kv) * kHeadDim + (tid & 1) * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base));
      }
      if (tid < 2) {
        const uint16_t *sc = (tid == 0 ? a.Ks : a.Vs) + (size_t)c * kAttnChunk * a.nKV;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(sc));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(sc + 64));
      }
    }
  }
  pdl_wait();
  attn_split_dispatch<true>(a, blockIdx.x, gridDim.x);
}
__global__ void __launch_bounds__(256) AttnCombine(const AttnCombineArgs a) { pdl_launch_dependents(); pdl_wait(); attn_combine_body(a, blockIdx.x, gridDim.x); }

#define F(f) AINFER_ARG(AttnPrepArgs, f)
AINFER_REGISTER(AttnPrep, AttnPrepArgs, 256, 8, 0, nullptr, F(Q16), F(K16), F(V16), F(QNW), F(KNW),
                F(Cos), F(Sin), F(Ctrl), F(Qn), F(Kc), F(Vc), F(Ks), F(Vs), F(nQ), F(nKV), F(rot),
                F(max_ctx), F(eps));
#undef F

#define F(f) AINFER_ARG(AttnSplitArgs, f)
AINFER_REGISTER(AttnSplit, AttnSplitArgs, 256, 1, 0, nullptr, F(Qn), F(Kc), F(Vc), F(Ks), F(Vs),
                F(Ctrl), F(Pm), F(Pse), F(Pacc), F(nQ), F(nKV), F(max_ctx), F(max_chunks));
#undef F

#define F(f) AINFER_ARG(AttnCombineArgs, f)
AINFER_REGISTER(AttnCombine, AttnCombineArgs, 256, 1, 0, nullptr, F(Pm), F(Pse), F(Pacc), F(Q16),
                F(Ctrl), F(Q8), F(SQ), F(Att), F(nQ), F(max_ctx), F(max_chunks));
#undef F

AINFER_EARLY_LAUNCH(AttnPrep);
AINFER_EARLY_LAUNCH(AttnSplit);
AINFER_EARLY_LAUNCH(AttnCombine);

}  // namespace ainfer
