// Per-token dynamic int8 quantisation (the prologue of the A8W8 GEMM).
//
// One CTA owns one row.  The row is read from HBM once: every thread keeps its
// 16-byte chunks in registers between the absmax reduction and the quantise
// pass, so the traffic is 2 bytes in + 1 byte out per element.
//
// Arithmetic reproduces DynamicQuantize._torch_impl of the reference
// (flashnn/quant_gemm.py:53-57), which works in the input dtype T:
//     s = T(absmax / 127)            q = rint(T(x / s))          scale_out = half(s)
// with IEEE division in fp32 followed by one rounding to T, exactly what the CPU
// computes for 16-bit tensors.  The int8 cast saturates.
//
// The per-element division is replaced by two multiplications with a bracketed
// reciprocal (quantise.cuh): where both products round to the same T value the exact
// quotient does too; only the rare elements next to a rounding midpoint of T take the
// exact division.  rint and the int8 cast are one magic-number addition (no conversion
// instructions).
#include "common.cuh"
#include "quantise.cuh"

namespace fnn {
namespace {

constexpr int kDqThreads = 256;     // block size of the generic kernel
constexpr int kDqMaxThreads = 1024;  // largest block of the vector kernel

// Vector path: K % 8 == 0, 16-byte aligned rows in, 8-byte aligned rows out.
// NCHUNK = 16-byte chunks per thread (row held in registers).
template <typename T, int NCHUNK>
__global__ void __launch_bounds__(kDqMaxThreads)
dq_row_vec_kernel(const T* __restrict__ x, int64_t ldx, int8_t* __restrict__ q, int64_t ldq,
                  __half* __restrict__ scale, int K) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  const int nvec = K >> 3;
  uint4 v[NCHUNK];
  uint32_t m2 = 0;  // packed pair of running maxima (+0, +0)
#pragma unroll
  for (int c = 0; c < NCHUNK; ++c) {
    const int i = c * blockDim.x + threadIdx.x;
    v[c] = (i < nvec) ? __ldcs(xr + i) : make_uint4(0, 0, 0, 0);
    m2 = absmax2(absmax2(absmax2(absmax2(m2, v[c].x, T()), v[c].y, T()), v[c].z, T()), v[c].w, T());
  }
  const float amax = block_absmax_keep_nan(max_keep_nan(lo_of<T>(m2), hi_of<T>(m2)), red);
  const float s = round_to<T>(__fdiv_rn(amax, 127.0f));
  if (threadIdx.x == 0) scale[row] = __float2half_rn(s);
  uint2* qr = reinterpret_cast<uint2*>(q + row * ldq);
  const InvBracket inv2 = inv_bracket(s);
  if (!usable_scale(s) || inv_overflowed(inv2)) {
    // all-zero row, a scale that underflowed to zero in T, one too small to invert, or a row with a NaN or an
    // infinity in it (scale NaN / infinite): the plain form, in which a NaN quotient is written as 0
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int i = c * blockDim.x + threadIdx.x;
      if (i < nvec) {
        const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
        uint32_t o[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int q0 = quantise_one<T>(lo_of<T>(w[2 * h]), s);
          const int q1 = quantise_one<T>(hi_of<T>(w[2 * h]), s);
          const int q2 = quantise_one<T>(lo_of<T>(w[2 * h + 1]), s);
          const int q3 = quantise_one<T>(hi_of<T>(w[2 * h + 1]), s);
          o[h] = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) | ((q3 & 0xff) << 24);
        }
        __stcs(qr + i, make_uint2(o[0], o[1]));
      }
    }
    return;
  }
  const float inv_s = __frcp_rn(s);
#pragma unroll
  for (int c = 0; c < NCHUNK; ++c) {
    const int i = c * blockDim.x + threadIdx.x;
    if (i < nvec) {
      const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
      uint32_t o[2];
      uint32_t amb = 0;
#pragma unroll
      for (int h = 0; h < 2; ++h)  // [q0,q1,..] and [q2,q3,..] -> [q0,q1,q2,q3]
        o[h] = __byte_perm(quantise_pair<T>(w[2 * h], inv2, amb), quantise_pair<T>(w[2 * h + 1], inv2, amb), 0x5410);
      if (amb != 0) {
        // some element of this chunk sits next to a rounding midpoint: redo the chunk element by element
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t q0 = quantise_fast<T>(lo_of<T>(w[2 * h]), s, inv_s);
          const uint32_t q1 = quantise_fast<T>(hi_of<T>(w[2 * h]), s, inv_s);
          const uint32_t q2 = quantise_fast<T>(lo_of<T>(w[2 * h + 1]), s, inv_s);
          const uint32_t q3 = quantise_fast<T>(hi_of<T>(w[2 * h + 1]), s, inv_s);
          o[h] = __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
        }
      }
      __stcs(qr + i, make_uint2(o[0], o[1]));
    }
  }
}

// Any K, any alignment, any row length: two passes over the row (the second
// one is served by L2).
template <typename T>
__global__ void __launch_bounds__(kDqThreads)
dq_row_generic_kernel(const T* __restrict__ x, int64_t ldx, int8_t* __restrict__ q, int64_t ldq,
                      __half* __restrict__ scale, int K) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * ldx;
  float amax = 0.f;
  for (int i = threadIdx.x; i < K; i += blockDim.x) amax = max_keep_nan(amax, to_f32(xr[i]));
  amax = block_absmax_keep_nan(amax, red);
  const float s = round_to<T>(__fdiv_rn(amax, 127.0f));
  if (threadIdx.x == 0) scale[row] = __float2half_rn(s);
  int8_t* qr = q + row * ldq;
  for (int i = threadIdx.x; i < K; i += blockDim.x)
    qr[i] = static_cast<int8_t>(quantise_one<T>(to_f32(xr[i]), s));
}

template <typename T>
int launch_dq(const T* x, int64_t M, int64_t K, int64_t ldx, int8_t* q, int64_t ldq, __half* scale,
              cudaStream_t st) {
  const bool vec = (K % 8 == 0) && (ldx % 8 == 0) && (ldq % 8 == 0) &&
                   (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(q) % 8 == 0) && (K <= int64_t(kDqMaxThreads) * 8 * 8);
  const dim3 grid(static_cast<unsigned>(M));
  if (!vec) {
    dq_row_generic_kernel<T><<<grid, kDqThreads, 0, st>>>(x, ldx, q, ldq, scale, int(K));
    return check_cuda(cudaGetLastError(), "dynamic_quant (generic) launch");
  }
  // block size: eight chunks per thread where the row is long enough (few threads with much work in flight each,
  // and several CTAs per SM in different phases, measured faster than wide blocks of four-chunk threads)
  const int nvec = int(K / 8);
  int threads = (((nvec + 7) / 8 + 31) / 32) * 32;
  if (threads < 64) threads = ((nvec + 31) / 32) * 32 < 64 ? ((nvec + 31) / 32) * 32 : 64;
  if (threads > kDqMaxThreads) threads = kDqMaxThreads;
  const int nchunk = (nvec + threads - 1) / threads;
#define FNN_DQ_CASE(N)                                                                     \
  dq_row_vec_kernel<T, N><<<grid, threads, 0, st>>>(x, ldx, q, ldq, scale, int(K))
  if (nchunk <= 1) FNN_DQ_CASE(1);
  else if (nchunk <= 2) FNN_DQ_CASE(2);
  else if (nchunk <= 4) FNN_DQ_CASE(4);
  else FNN_DQ_CASE(8);
#undef FNN_DQ_CASE
  return check_cuda(cudaGetLastError(), "dynamic_quant launch");
}

}  // namespace
}  // namespace fnn

extern "C" int fnn_dynamic_quant(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                                 int8_t* q, int64_t ldq, void* scale_f16, void* stream) {
  using namespace fnn;
  if (M < 0 || K < 0 || ldx < K || ldq < K) return fail(FNN_ERR_SHAPE, "dynamic_quant: M=%lld K=%lld ldx=%lld ldq=%lld", (long long)M, (long long)K, (long long)ldx, (long long)ldq);
  if (x_dtype != FNN_F16 && x_dtype != FNN_BF16) return fail(FNN_ERR_DTYPE, "dynamic_quant: input must be f16 or bf16 (got dtype code %d)", x_dtype);
  if (M == 0) return FNN_OK;
  if (!x || !q || !scale_f16) return fail(FNN_ERR_NULL_POINTER, "dynamic_quant: null tensor pointer");
  if (K == 0 || K > INT32_MAX || M > INT32_MAX) return fail(FNN_ERR_SHAPE, "dynamic_quant: K must be in [1, 2^31), M below 2^31");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (x_dtype == FNN_F16)
    return launch_dq<__half>(static_cast<const __half*>(x), M, K, ldx, q, ldq, static_cast<__half*>(scale_f16), st);
  return launch_dq<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(x), M, K, ldx, q, ldq, static_cast<__half*>(scale_f16), st);
}
