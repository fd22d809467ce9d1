/*
 * flashnn_b200 -- C ABI of the B200 (sm_100a) quantized-GEMM kernels.
 *
 * The reference project has no FFI: its kernels are reached through Python
 * launcher functions that take caller-allocated tensors
 * (`triton_dynamic_quantize`, `triton_gemm_a8w8_forward`,
 * `triton_gemm_a16w8_forward`, `triton_gemm_a16w4_forward`).  Each entry point
 * below replaces one of those launchers and is cited beside it (paths are
 * inside the reference project).  Conventions, all entry points:
 *
 *   - every pointer is a device pointer unless stated otherwise; the caller
 *     owns all memory, the library allocates nothing on these paths;
 *   - sizes are in elements, leading dimensions (`ld*`) in elements of the
 *     tensor they belong to, row-major;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL is the
 *     default stream) and the call returns without synchronising;
 *   - the return value is an `fnn_status`; nothing is thrown, nothing exits,
 *     and on any non-zero status no kernel has been launched;
 *   - the library is re-entrant; `fnn_last_error_string` is per host thread.
 */
#ifndef FLASHNN_B200_H
#define FLASHNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FNN_VERSION 100 /* major*10000 + minor*100 + patch */

typedef enum fnn_status {
  FNN_OK = 0,
  FNN_ERR_NULL_POINTER = 1,  /* a required pointer is NULL */
  FNN_ERR_DTYPE = 2,         /* dtype code not accepted for that argument */
  FNN_ERR_SHAPE = 3,         /* negative/inconsistent sizes, ld smaller than the row */
  FNN_ERR_ALIGNMENT = 4,     /* pointer or pitch breaks a documented alignment rule */
  FNN_ERR_UNSUPPORTED = 5,   /* combination not implemented */
  FNN_ERR_WORKSPACE = 6,     /* workspace missing or smaller than *_workspace_bytes says */
  FNN_ERR_CUDA = 7,          /* a CUDA runtime/driver call failed; see fnn_last_error_string */
  FNN_ERR_DEVICE_TIMEOUT = 8 /* a kernel gave up on a bounded wait (reported by fnn_device_status) */
} fnn_status;

typedef enum fnn_dtype {
  FNN_F16 = 0,
  FNN_BF16 = 1,
  FNN_F32 = 2
} fnn_dtype;

/*
 * Process-wide options (fnn_set_option / fnn_get_option).  No counterpart in the reference.
 *
 * FNN_OPT_STATIC_WEIGHTS (default 0).  A promise by the caller: the qweight, scale, zero_points and bias buffers given
 * to fnn_gemm_weight_only are not written by the kernel that directly precedes the call in the same stream (true for
 * inference, where weights are loaded once).  With it set, the one-to-five-token decode kernel is launched with programmatic
 * stream serialisation: its CTAs may become resident while the preceding kernel drains and start fetching weights; they
 * touch neither the activations nor the output until that kernel has completed and its writes are visible
 * (griddepcontrol.wait).  Results are unchanged; back-to-back decode calls lose the launch gap between them.
 *
 * FNN_OPT_TEST_STALL_US (default 0; a hook for the library's own tests, never set it in production).  With a value
 * v > 0, fnn_gemm_a8w8 calls that run the single-CTA tensor-core kernel (at most 128 rows, or few tiles) leave out the
 * loads of one K block of every CTA's first tile and bound every wait of that launch to v microseconds instead of two
 * seconds.  The wait for the missing block then runs out: the kernel records its time-out code, drains what it has in
 * flight, frees what it holds and returns without a result, and the next fnn_device_status reports
 * FNN_ERR_DEVICE_TIMEOUT.  This is how the give-up path of the kernels is exercised without faulting the GPU.
 *
 * FNN_OPT_A8W8_PAIR_TILE (default 0 = chosen from the problem shape; a tuning hook).  128, 160, 192, 224 or 256 forces
 * that output-tile width in fnn_gemm_a8w8 wherever the CTA-pair tensor-core kernel can run (more than 128 rows).  The
 * shape-to-tile table in the library was measured with it; results do not depend on the tile.
 *
 * FNN_OPT_A8W8_BALANCED (default 0).  The CTA-pair kernel of fnn_gemm_a8w8 has a K-balanced mode for shapes whose
 * 256 x 256 tiles do not fill the last round of CTA pairs (for instance 64 tiles on 74 pairs): the (tile, K block)
 * units are dealt out evenly, a pair that stops inside a tile leaves its int32 partial sums in the workspace and the
 * pair that finishes the tile adds them (int32 additions: the accumulator stays exact whatever the order).  0 = used
 * where the shape table expects at least 3 % from it and the caller passed the workspace, 1 = wherever it can run
 * (more than 128 rows, a workspace; for tests), 2 = never.
 *
 * FNN_OPT_A8W8_EPILOGUE_WARPS (default 0; a tuning hook).  The CTA-pair kernel runs with eight epilogue warps per CTA
 * (with short K a tile's MMAs take less time than four warps need to write it out); 4 runs it with four.
 */
typedef enum fnn_option {
  FNN_OPT_STATIC_WEIGHTS = 1,
  FNN_OPT_TEST_STALL_US = 2,
  FNN_OPT_A8W8_PAIR_TILE = 3,
  FNN_OPT_A8W8_BALANCED = 4,
  FNN_OPT_A8W8_EPILOGUE_WARPS = 5
} fnn_option;

/* Sets an option; FNN_ERR_UNSUPPORTED for an unknown one.  fnn_get_option returns the value, or -1 if unknown. */
int fnn_set_option(int option, int value);
int fnn_get_option(int option);

/* Library version (FNN_VERSION of the build). */
int fnn_version(void);

/* Text of the last non-zero status returned on this host thread ("" if none). */
const char* fnn_last_error_string(void);

/* Name of a status code. */
const char* fnn_status_string(int status);

/*
 * Reads and clears the current device's kernel status word.  Kernels never trap:
 * a wait on an mbarrier that runs out of time records a code there, releases what
 * the CTA holds and returns.  *device_code receives 0 when every kernel since the
 * last call completed normally.  Synchronises the device.  Returns FNN_OK,
 * FNN_ERR_DEVICE_TIMEOUT (with the code in *device_code) or FNN_ERR_CUDA.
 */
int fnn_device_status(int* device_code);

/*
 * Per-token dynamic int8 quantisation.
 * Replaces `triton_dynamic_quantize(out, input, scale)`
 * (flashnn/triton_kernels/dynamic_quant.py:73-97); arithmetic follows
 * `DynamicQuantize._torch_impl` (flashnn/quant_gemm.py:53-57): absmax, scale =
 * absmax/127 and x/scale are each rounded to the input dtype, the quotient is
 * rounded half-to-even, and the int8 cast saturates (+128 becomes +127; the
 * reference's cast wraps it to -128).  A row of zeros gives q = 0, scale = 0.
 * Non-finite input is not hidden: a row that holds a NaN gets scale = NaN, a row
 * that holds an infinity (and no NaN) gets scale = infinity, as the reference's
 * torch path gives; every quotient of such a row is NaN or 0 and q is written
 * as 0, so a GEMM fed with the row and its scale yields NaN outputs.
 *
 *   x      [M, K]  f16 or bf16 (x_dtype), leading dimension ldx
 *   q      [M, K]  int8, leading dimension ldq
 *   scale  [M]     f16
 */
int fnn_dynamic_quant(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                      int8_t* q, int64_t ldq, void* scale_f16, void* stream);

/*
 * A8W8 GEMM:  out[m,n] = (sum_k a[m,k] * b[n,k]) * s(m,n)  cast to out_dtype.
 * Replaces `triton_gemm_a8w8_forward(out, a, b, alpha_row, alpha_col)`
 * (flashnn/triton_kernels/gemm_a8w8.py:182-221); the scale follows
 * `GemmA8W8._torch_impl` (flashnn/quant_gemm.py:96-104): when both scales have
 * the same 16-bit dtype, s = row*col rounded to that dtype; otherwise
 * s = fl32(row*col); then out = fl32(float(acc) * s) rounded once to out_dtype.
 * The accumulator is exact int32.
 *
 *   a          [M, K]  int8, lda      b          [N, K]  int8, ldb
 *   alpha_row  [M]     row_dtype      alpha_col  [N]     col_dtype  (f16/bf16/f32)
 *   out        [M, N]  f16 or bf16 (out_dtype), ldo
 *   acc_out    optional [M, N] int32 (ldacc): when not NULL the raw accumulator is
 *              written there as well (parity checks)
 *   workspace  scratch of at least fnn_gemm_a8w8_workspace_bytes(M, N, K) bytes,
 *              256-byte aligned; may be NULL when that function returns 0.  Only the
 *              K-balanced mode of the CTA-pair kernel uses it (FNN_OPT_A8W8_BALANCED); when it
 *              is missing or too small that mode is not used and the result is the same.
 *              Its contents need no initialisation and mean nothing afterwards; two calls
 *              that may run at the same time (different streams) need different workspaces.
 *
 * Fast path (TMA + tcgen05): a, b 16-byte aligned and lda, ldb multiples of 16.
 * Anything else runs a slower generic kernel with the same results.
 */
int fnn_gemm_a8w8(const int8_t* a, int64_t lda, const int8_t* b, int64_t ldb,
                  const void* alpha_row, int row_dtype, const void* alpha_col, int col_dtype,
                  void* out, int out_dtype, int64_t ldo, int64_t M, int64_t N, int64_t K,
                  int32_t* acc_out, int64_t ldacc, void* workspace, size_t workspace_bytes,
                  void* stream);

/* Scratch bytes fnn_gemm_a8w8 needs for this problem size on the current device. */
size_t fnn_gemm_a8w8_workspace_bytes(int64_t M, int64_t N, int64_t K);

/*
 * Which kernel and output-tile width fnn_gemm_a8w8 picks for a problem with 16-byte-aligned operands on the current
 * device (148 SMs are assumed when there is none): *kernel = 0 single-CTA tensor-core kernel (tile 128 x *tile_n),
 * 1 CTA-pair tensor-core kernel (tile 256 x *tile_n), 2 the streaming decode kernel (16 output channels per step),
 * 3 the CTA-pair kernel in its K-balanced mode (taken only when the call passes the workspace).
 * This is the shape -> configuration table that takes the place of the reference's autotune cache
 * (flashnn/triton_kernels/triton_utils.py:84-151); its constants are measured (flashnn_b200/csrc/a8w8_plan.h).
 * Needs no GPU.
 */
int fnn_gemm_a8w8_plan(int64_t M, int64_t N, int64_t K, int* kernel, int* tile_n);

/*
 * Fused mixture-of-experts A8W8 GEMM over expert-sorted token slots.
 * Replaces `fused_moe_a8w8_forward(A, B, C, alpha_row, alpha_col, topk_weights, topk_ids, sorted_token_ids, expert_ids,
 * num_tokens_post_padded, mul_routed_weight, top_k, BM)` (flashnn/triton_kernels/fused_moe_a8w8.py:176-290; arithmetic
 * of the kernel at :96-170).  For every slot s < *num_tokens_post_padded whose flat index f = sorted_token_ids[s] is
 * below num_valid_tokens, with e = expert_ids[s / block_m]:
 *     out[f, n] = cast( ((float(sum_k a[f / top_k, k] * b[e, n, k]) * alpha_row[f / top_k]) * alpha_col[e, n])
 *                        * (mul_routed_weight ? topk_weights[f] : 1) )
 * Rows of `out` that no slot names are left untouched.  The accumulator is exact int32.
 *
 *   a                 [M, K] int8, lda (a multiple of 16); K a multiple of 16
 *   b                 [E, N, K] int8, contiguous
 *   alpha_row         [M] row_dtype;  alpha_col [E, N] contiguous, col_dtype;  topk_weights [M * top_k] topk_dtype
 *   sorted_token_ids  [EM] int32: flat (token * top_k + choice) indices grouped by expert, every expert's group padded
 *                     to a multiple of block_m with values >= num_valid_tokens
 *   expert_ids        [EM / block_m] int32;  num_tokens_post_padded [1] int32 (device memory)
 *   out               [M * top_k, N] f16 or bf16, ldo
 *   block_m           at most 128, or a multiple of 128; a multiple of 256 with enough blocks to give every CTA pair a
 *                     tile runs on the CTA-pair kernel (prefill-sized batches: 11-15 % faster than blocks of 128)
 *   workspace         fnn_fused_moe_a8w8_workspace_bytes(EM, K) bytes, 256-byte aligned (the expert-sorted copy of
 *                     the token rows)
 */
int fnn_fused_moe_a8w8(const int8_t* a, int64_t lda, const int8_t* b, int64_t E, int64_t N, int64_t K,
                       const void* alpha_row, int row_dtype, const void* alpha_col, int col_dtype,
                       const void* topk_weights, int topk_dtype, const int32_t* sorted_token_ids, int64_t EM,
                       const int32_t* expert_ids, const int32_t* num_tokens_post_padded, int64_t num_valid_tokens,
                       int top_k, int block_m, int mul_routed_weight, void* out, int out_dtype, int64_t ldo,
                       void* workspace, size_t workspace_bytes, void* stream);
size_t fnn_fused_moe_a8w8_workspace_bytes(int64_t EM, int64_t K);

/*
 * Fused mixture-of-experts weight-only GEMM over expert-sorted token slots, packed-int4 expert weights.
 * Replaces `fused_moe_a16w4_forward(A, B, C, scale_b, zero_points, topk_weights, topk_ids, sorted_token_ids, expert_ids,
 * num_tokens_post_padded, mul_routed_weight, top_k, BM)` (flashnn/triton_kernels/fused_moe_a16w4.py:326-466; kernels at
 * :50-183 per channel and :186-323 per K group).  For every slot s < *num_tokens_post_padded whose flat index
 * f = sorted_token_ids[s] is below num_valid_tokens, with e = expert_ids[s / block_m]:
 *     out[f, n] = cast( (sum_k a[f / top_k, k] * (W[e, n, k] - zp) * scale) * (mul_routed_weight ? topk_weights[f] : 1) )
 * with scale, zp taken per (e, n) (group_size == 0) or per (e, n, k / group_size).  Products and sums are fp32 and the
 * dequantised weight is never rounded to 16 bits (the reference's per-group kernel rounds (W - zp) * scale to 16 bits
 * per weight; as for fnn_gemm_weight_only the bar here is the fp32 dequant-matmul).  Rows of `out` that no slot names
 * are left untouched.  No workspace: the token rows are gathered inside the kernel.
 *
 *   a                 [M, K] f16 or bf16 (a_dtype), lda a multiple of 8; K a multiple of 16; 16-byte aligned
 *   b                 [E, N/2, K] bytes, contiguous: byte (e, j, k) holds channel 2j in its low nibble and channel
 *                     2j+1 in its high nibble, two's complement (packing along N, fused_moe_a16w4.py:137,151)
 *   scale             [E, N] (group_size == 0) or [E, N, K/group_size], contiguous, scale_dtype; zero_points NULL or alike
 *   group_size        0, or a multiple of 64 that divides K
 *   topk_weights      [M * top_k] topk_dtype;  sorted_token_ids [EM] int32;  expert_ids [EM / block_m] int32;
 *                     num_tokens_post_padded [1] int32 (device memory) -- as for fnn_fused_moe_a8w8
 *   out               [M * top_k, N] in a_dtype, ldo
 *   block_m           at most 64, or a multiple of 64
 */
int fnn_fused_moe_a16w4(const void* a, int a_dtype, int64_t lda, const void* b, int64_t E, int64_t N, int64_t K,
                        const void* scale, const void* zero_points, int scale_dtype, int64_t group_size,
                        const void* topk_weights, int topk_dtype, const int32_t* sorted_token_ids, int64_t EM,
                        const int32_t* expert_ids, const int32_t* num_tokens_post_padded, int64_t num_valid_tokens,
                        int top_k, int block_m, int mul_routed_weight, void* out, int out_dtype, int64_t ldo, void* stream);

/*
 * The same operator with caller scratch.  With blocks of 256 sorted slots (block_m a multiple of 256), enough blocks to
 * give every CTA pair a tile and a workspace of fnn_fused_moe_a16w4_workspace_bytes(...) bytes (256-byte aligned), the
 * call runs on the tcgen05 prefill kernels of the weight-only GEMM in a fused-MoE mode: the token rows are first copied
 * into expert-sorted order in the workspace (with zero-points also their row sums per scale group).  Any other call,
 * and a call without the workspace, does exactly what fnn_fused_moe_a16w4 does.  The workspace function returns 0 for
 * block sizes that never use one.  Same results contract (fp32 dequant-matmul bound).
 */
int fnn_fused_moe_a16w4_ws(const void* a, int a_dtype, int64_t lda, const void* b, int64_t E, int64_t N, int64_t K,
                           const void* scale, const void* zero_points, int scale_dtype, int64_t group_size,
                           const void* topk_weights, int topk_dtype, const int32_t* sorted_token_ids, int64_t EM,
                           const int32_t* expert_ids, const int32_t* num_tokens_post_padded, int64_t num_valid_tokens,
                           int top_k, int block_m, int mul_routed_weight, void* out, int out_dtype, int64_t ldo,
                           void* workspace, size_t workspace_bytes, void* stream);
size_t fnn_fused_moe_a16w4_workspace_bytes(int64_t EM, int64_t K, int64_t group_size, int has_zero_points, int block_m);

/*
 * Weight-only GEMM / GEMV:  out = act . dequant(W)^T (+ bias), W int8 or packed int4.
 * Replaces `triton_gemm_a16w8_forward` (flashnn/triton_kernels/gemm_a16w8.py:275-338)
 * and `triton_gemm_a16w4_forward` (flashnn/triton_kernels/gemm_a16w4.py:336-406).
 * dequant(W)[n,k] = (W[n,k] - zp) * scale with zp, scale per channel n
 * (group_size == 0) or per (k / group_size, n).  Products and sums are fp32, the
 * dequantised weight is never rounded to 16 bits, the bias is added in fp32 and
 * the result is rounded once to out_dtype.
 *
 *   act          [M, K]   f16 or bf16 (act_dtype), lda
 *   qweight      weight_bits == 8: int8 [N, K]
 *                weight_bits == 4: bytes [N/2, K]; byte (j,k) holds channel 2j in its
 *                low nibble and channel 2j+1 in its high nibble, two's complement
 *                (flashnn/quant_gemm.py:175-190).  Row pitch is K bytes in both cases.
 *   scale        [N] (group_size == 0) or [K/group_size, N]; dtype scale_dtype
 *   zero_points  NULL or same shape and dtype as scale
 *   bias         NULL or [N] of dtype bias_dtype
 *   out          [M, N]  out_dtype (f16 or bf16), ldo
 *   workspace    scratch of at least fnn_gemm_weight_only_workspace_bytes(...) bytes,
 *                256-byte aligned; may be NULL when that function returns 0
 */
int fnn_gemm_weight_only(const void* act, int act_dtype, int64_t lda, const void* qweight,
                         int weight_bits, const void* scale, const void* zero_points,
                         int scale_dtype, int64_t group_size, const void* bias, int bias_dtype,
                         void* out, int out_dtype, int64_t ldo, int64_t M, int64_t N, int64_t K,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Scratch bytes fnn_gemm_weight_only needs for this problem on the current device. */
size_t fnn_gemm_weight_only_workspace_bytes(int64_t M, int64_t N, int64_t K, int weight_bits,
                                            int64_t group_size);

/*
 * RMSNorm / LayerNorm fused with per-token dynamic int8 quantisation (the producer of fnn_gemm_a8w8's A operand).
 * Replace `triton_rmsnorm_dquant_forward(x, weight, eps)` (flashnn/triton_kernels/rms_norm_dquant.py:80-96) and
 * `triton_layer_norm_dquant_forward(x, weight, bias, eps)` (flashnn/triton_kernels/layer_norm_dquant.py:91-105);
 * arithmetic follows `RMSNormDquant._torch_impl` (flashnn/norm.py:39-63: fp32 throughout, clamp to [-128, 127]) and
 * `LayernormDquant._torch_impl` (flashnn/norm.py:94-124: the normalised row is rounded to the input dtype, the scale
 * and the quotient are formed in that dtype, clamp to [-128, 127]).
 *
 *   x       [M, K]  f16 or bf16, ldx; K a multiple of 8 and at most 32768, rows 16-byte aligned
 *   weight  [K]     (and bias [K] for the layer norm) of dtype w_dtype: the dtype of x, or f32; 16-byte aligned
 *   q       [M, K]  int8, ldq (a multiple of 8)
 *   scale   [M]     in the dtype of x
 *
 * A row that holds a NaN or an infinity gets scale = NaN and q = 0 (every normalised value, hence every quotient,
 * is NaN there), as the reference's torch path gives.
 */
int fnn_rms_norm_dquant(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* weight,
                        int w_dtype, float eps, int8_t* q, int64_t ldq, void* scale, void* stream);
int fnn_layer_norm_dquant(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* weight,
                          const void* bias, int w_dtype, float eps, int8_t* q, int64_t ldq, void* scale,
                          void* stream);

/*
 * Weight-only GEMM with per-channel scales that needs no workspace from the caller and allocates nothing.
 * No counterpart in the reference; it exists for callers that cannot obtain device memory at call time:
 * a plugin inside a host process that owns every allocation, a server whose memory pool was carved up at
 * start-up, a latency-critical loop where a cudaMalloc (and the device-wide synchronisation it implies) is
 * not acceptable.  Same tensor-core kernel and same results as fnn_gemm_weight_only for per-channel scales;
 * the one piece of scratch that kernel uses (fp32 row sums of the activations, read when zero-points are
 * given) lives in a 256 KB array inside the library image instead of a caller buffer.
 *
 *   - group_size is implicitly 0 (scale, zero_points are [N]); all other arguments as fnn_gemm_weight_only;
 *   - M may not exceed 65536 rows: larger calls are refused with FNN_ERR_WORKSPACE (use fnn_gemm_weight_only);
 *   - act and qweight 16-byte aligned, lda a multiple of 8, K a multiple of 16 (else FNN_ERR_ALIGNMENT);
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
 *     first call outside any stream capture;
 *   - every call on a device shares the one array: calls that can overlap on the GPU (different streams) race
 *     on it and must be serialised by the caller.  Nothing in it has to be cleared between calls: each call
 *     rewrites the rows it reads;
 *   - every GPU that loads the library holds the 256 KB until the process exits.
 */
int fnn_gemm_weight_only_prefill_static(const void* act, int act_dtype, int64_t lda, const void* qweight,
                                        int weight_bits, const void* scale, const void* zero_points,
                                        int scale_dtype, const void* bias, int bias_dtype, void* out,
                                        int out_dtype, int64_t ldo, int64_t M, int64_t N, int64_t K, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHNN_B200_H */
