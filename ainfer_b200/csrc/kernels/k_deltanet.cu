// DeltaNetStep kernel entry; the body lives in deltanet_core.cuh so that the
// persistent decode kernel can run the same code as one of its stages.
#include "deltanet_core.cuh"

namespace ainfer {

__global__ void __launch_bounds__(256) DeltaNetStep(const DeltaNetStepArgs a) {
  pdl_launch_dependents();
  // the recurrent state is this kernel's own (last written one token ago): fetch while waiting
  float s0[kDnSeg];
  const bool have = (int)blockIdx.x < a.nV * kDnSlices;
  if (have) deltanet_load_state(a, blockIdx.x, s0);
  pdl_wait();
  deltanet_step_body(a, blockIdx.x, gridDim.x, have ? &s0 : nullptr);
}
#define F(f) AINFER_ARG(DeltaNetStepArgs, f)
AINFER_REGISTER(DeltaNetStep, DeltaNetStepArgs, 256, 1, 0, nullptr, F(Out), F(Mx), F(S), F(Bt),
                F(Gt), F(nK), F(nV));
#undef F

AINFER_EARLY_LAUNCH(DeltaNetStep);

}  // namespace ainfer
