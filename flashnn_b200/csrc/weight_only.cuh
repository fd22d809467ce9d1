// Declarations shared by the weight-only kernels.
#pragma once
#include "common.cuh"

namespace fnn {

struct WoParams {
  const void* act;      // [M, K] T
  const uint8_t* qw;    // int8 [N, K] or packed [N/2, K]
  const void* scale;    // [N] or [G, N]
  const void* zp;       // nullptr or like scale
  const void* bias;     // nullptr or [N]
  void* out;
  int64_t lda, ldo;
  int scale_dtype, bias_dtype;
  int M, N, K;
  int group;  // 0 = per channel
  int* status;  // device status word
};

// |x| with NaN mapped to +infinity, so that a running fmaxf keeps a non-finite input visible
__device__ __forceinline__ float nan_to_inf(float v) { return v != v ? __int_as_float(0x7f800000) : v; }

// Decode kernel on the integer tensor pipe (gemv_w4_imma.cu) for one to five tokens; bits = 4 (packed) or 8.
// Returns an fnn_status, or -1 when the shape or alignment is outside what that kernel handles.
int gemv_w4_imma(const WoParams& p, int bits, int act_dtype, cudaStream_t st);

}  // namespace fnn
