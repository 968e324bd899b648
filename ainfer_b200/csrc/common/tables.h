// Device-resident tables that the runtime builds at record time and kernels
// read: plain C layouts shared by host (g++) and device (nvcc) code.
#pragma once
#include <cstdint>

namespace ainfer {

enum GemvEpilogue {
  EPI_STORE = 0,     // Y[m][n] = acc
  EPI_RESADD = 1,    // Y[m][n] = e0[m][n] + acc                     (ResAddF, kernels.cpp:646-652)
  EPI_CONV_SILU = 2, // depthwise conv k=4 + SiLU + history shift     (SsmConv, kernels.cpp:322-338)
  EPI_BETA = 3,      // Y[n] = sigmoid(acc)                           (BetaG, kernels.cpp:612)
  EPI_GDECAY = 4     // Y[n] = -exp(A_log[n]) * softplus(acc + dt[n]) (BetaG, kernels.cpp:613-615)
};

// One entry of the matrix table of an Int4GemvA8 launch (64 bytes).
struct GemvMat {
  const uint8_t *P;    // packed nibbles [N][K/2]
  const uint16_t *S;   // bf16 scales [N][K/128]
  float *Y;            // output
  const float *e0;     // EPI_RESADD: residual; CONV: weights [N][4]; GDECAY: A_log
  float *e1;           // CONV: history [N][3] (updated in place)
  const float *e2;     // GDECAY: dt_bias
  int32_t row_start;   // first global row of this matrix in the launch
  int32_t N;
  int32_t epi;
  int32_t ldy;         // row stride of Y / e0 between batch entries (elements)
};

// Device pointers of one expert's three matrices (48 bytes). A layer's table
// has n_experts entries followed by the shared expert.
struct ExpertW {
  const uint8_t *gP; const uint16_t *gS;   // gate_proj [I][H]
  const uint8_t *uP; const uint16_t *uS;   // up_proj   [I][H]
  const uint8_t *dP; const uint16_t *dS;   // down_proj [H][I]
};

}  // namespace ainfer
