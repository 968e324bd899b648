// Greedy-token tail of the decode loop: two-stage first-max-wins argmax over
// the logits (ArgmaxS1/ArgmaxS2, tools/cmdlist/kernels.cpp:480-546), then the
// control-block update that the reference does on the host between tokens
// (tools/decode/decode_l0.cpp:753-756,816-818), moved on device so that
// consecutive greedy tokens need no host round trip.
#include "tail_core.cuh"

namespace ainfer {

struct ArgmaxStage1Args {
  const float *Logits;
  float *PV;
  int32_t *PI;
  int32_t V;
};
__global__ void __launch_bounds__(256) ArgmaxStage1(const ArgmaxStage1Args a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[8];
  __shared__ int si[8];
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  for (int i = blockIdx.x * 256 + threadIdx.x; i < a.V; i += gridDim.x * 256)
    argmax_merge(bv, bi, a.Logits[i], i);
  block_argmax(bv, bi, sv, si);
  if (threadIdx.x == 0) { a.PV[blockIdx.x] = bv; a.PI[blockIdx.x] = bi; }
}
#define F(f) AINFER_ARG(ArgmaxStage1Args, f)
AINFER_REGISTER(ArgmaxStage1, ArgmaxStage1Args, 256, 0, 0, nullptr, F(Logits), F(PV), F(PI), F(V));
#undef F

struct ArgmaxStage2Args {
  const float *PV;
  const int32_t *PI;
  int32_t *OutT;      // [1] selected token
  int32_t *Ctrl;      // control block (may be null)
  int32_t *History;   // optional ring of selected tokens [history_cap]
  int32_t parts;      // number of stage-1 partials
  int32_t advance;    // 1: Ctrl = {selected, position+1, active_length+1, selected}
  int32_t history_cap;
};
__global__ void __launch_bounds__(256) ArgmaxStage2(const ArgmaxStage2Args a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[8];
  __shared__ int si[8];
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  for (int i = threadIdx.x; i < a.parts; i += 256) argmax_merge(bv, bi, a.PV[i], a.PI[i]);
  block_argmax(bv, bi, sv, si);
  if (threadIdx.x == 0) {
    a.OutT[0] = bi;
    if (a.Ctrl) {
      int pos = a.Ctrl[CTRL_POS];
      if (a.History && a.history_cap > 0) a.History[pos % a.history_cap] = bi;
      a.Ctrl[CTRL_SELECTED] = bi;
      if (a.advance) {
        a.Ctrl[CTRL_TOKEN] = bi;
        a.Ctrl[CTRL_POS] = pos + 1;
        a.Ctrl[CTRL_LEN] = a.Ctrl[CTRL_LEN] + 1;
      }
    }
  }
}
#define F(f) AINFER_ARG(ArgmaxStage2Args, f)
AINFER_REGISTER(ArgmaxStage2, ArgmaxStage2Args, 256, 0, 0, nullptr, F(PV), F(PI), F(OutT), F(Ctrl),
                F(History), F(parts), F(advance), F(history_cap));
#undef F

// ControlAdvance: prompt steps produce no token; the next prompt id is taken
// from a device-resident id list so that a whole prompt replays without host
// work. Ctrl = {Ids[position+1], position+1, active_length+1, -1}.
struct ControlAdvanceArgs {
  int32_t *Ctrl;
  const int32_t *Ids;
  int32_t n_ids;
};
__global__ void ControlAdvance(const ControlAdvanceArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int pos = a.Ctrl[CTRL_POS] + 1;
    a.Ctrl[CTRL_POS] = pos;
    a.Ctrl[CTRL_LEN] = a.Ctrl[CTRL_LEN] + 1;
    if (pos < a.n_ids) a.Ctrl[CTRL_TOKEN] = a.Ids[pos];
    a.Ctrl[CTRL_SELECTED] = -1;
  }
}
#define F(f) AINFER_ARG(ControlAdvanceArgs, f)
AINFER_REGISTER(ControlAdvance, ControlAdvanceArgs, 32, 0, 0, nullptr, F(Ctrl), F(Ids), F(n_ids));
#undef F

AINFER_EARLY_LAUNCH(ArgmaxStage1);
AINFER_EARLY_LAUNCH(ArgmaxStage2);
AINFER_EARLY_LAUNCH(ControlAdvance);

}  // namespace ainfer
