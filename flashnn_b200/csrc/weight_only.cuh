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
  // A8W8 decode through the same kernel (int8 activations): per-token scale and the optional raw accumulator
  const void* row_scale;
  int row_dtype;
  int32_t* acc_out;
  int64_t ldacc;
};

// |x| with NaN mapped to +infinity, so that a running fmaxf keeps a non-finite input visible
__device__ __forceinline__ float nan_to_inf(float v) { return v != v ? __int_as_float(0x7f800000) : v; }

// Decode kernel on the integer tensor pipe (gemv_w4_imma.cu) for one to five tokens; bits = 4 (packed) or 8.
// Returns an fnn_status, or -1 when the shape or alignment is outside what that kernel handles.
int gemv_w4_imma(const WoParams& p, int bits, int act_dtype, cudaStream_t st);

// Packed-int4 decode for 6 to 16 tokens with the activations resident on the SM (gemv_w4_tok.cu).  Returns an
// fnn_status, or -1 when the shape or alignment is outside what that kernel handles.
int gemv_w4_tok(const WoParams& p, int act_dtype, cudaStream_t st);

// A8W8 GEMM for at most 16 tokens on the same kernel (int8 activations are the MMA's column operand as they are,
// exact int32 sums, the A8W8 scaling rule in the write-out).  b must be [N, K] with pitch K.  Returns an
// fnn_status, or -1 when the shape or alignment is outside what the kernel handles.
int gemv_a8w8_imma(const int8_t* a, int64_t lda, const int8_t* b, int64_t ldb, const void* alpha_row, int row_dtype,
                   const void* alpha_col, int col_dtype, void* out, int out_dtype, int64_t ldo, int M, int N, int K,
                   int32_t* acc_out, int64_t ldacc, cudaStream_t st);

// Fused MoE with packed-int4 expert weights on the prefill (tcgen05) kernels of gemm_weight_only.cu, for blocks of 256
// sorted slots or a multiple.  Returns an fnn_status, or -1 when the shape, the alignment or the workspace is outside
// what they take.  The workspace holds the expert-sorted copy of the token rows (and their row sums with zero-points).
size_t weight_only_moe_prefill_workspace(int64_t EM, int64_t K, int64_t group, bool zp);
int weight_only_moe_prefill(const void* a, int a_dtype, int64_t lda, const void* b, int E, int N, int K, const void* scale,
                            const void* zp, int scale_dtype, int group, const void* topk_w, int topk_dtype,
                            const int32_t* sorted_ids, int EM, const int32_t* expert_ids, const int32_t* npp, int num_valid,
                            int top_k, int block_m, int mul_w, void* out, int64_t ldo, void* workspace,
                            size_t workspace_bytes, cudaStream_t st);

}  // namespace fnn
