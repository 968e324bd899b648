// Kernel entries of the gated GQA decode attention; bodies in attention_core.cuh
// (shared with the persistent decode kernel).
#include "attention_core.cuh"

namespace ainfer {

__global__ void __launch_bounds__(256) AttnPrep(const AttnPrepArgs a) { pdl_launch_dependents(); pdl_wait(); attn_prep_body(a, blockIdx.x, gridDim.x); }
__global__ void __launch_bounds__(256) AttnSplit(const AttnSplitArgs a) { pdl_launch_dependents(); pdl_wait(); attn_split_dispatch(a, blockIdx.x, gridDim.x); }
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
