// RMSNorm / LayerNorm fused with per-token dynamic int8 quantisation: the producer of the A8W8 GEMM's
// activation operand in a transformer block.  One CTA owns one row and reads it from HBM once (the row stays
// in registers across the statistics, absmax and quantise passes); the norm weights are re-read from L1/L2.
//
// Arithmetic follows the reference's torch implementations (flashnn/norm.py:39-63 and :94-124):
//   RMSNormDquant   everything in fp32: n = (x * rsqrt(mean(x^2) + eps)) * w, s = max|n| / 127,
//                   q = clamp(rint(n / s), -128, 127); the scale is returned in the input dtype.
//   LayernormDquant y = layer_norm(x) is rounded to the input dtype T first; then, in T arithmetic as the
//                   reference does it, s = T(max|y| / 127), q = clamp(rint(T(y / s)), -128, 127).
// The fp32 row sums are formed in a different order than torch's, so the statistics can differ in the last
// bit and a quantised value that sits on a rounding boundary can come out one step away.
#include "common.cuh"
#include "quantise.cuh"

namespace fnn {
namespace {

constexpr int kNdMaxThreads = 1024;
constexpr float kRintMagic = 12582912.f;  // 1.5 * 2^23: adding it rounds |t| < 2^22 to an integer, half to even

template <bool MAX> __device__ __forceinline__ float block_reduce(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = MAX ? fmaxf(v, u) : v + u;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = (blockDim.x + 31) >> 5;
  __syncthreads();  // `red` may still be read from the previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  v = (lane < nwarp) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = MAX ? fmaxf(v, u) : v + u;
  }
  return v;
}

// eight consecutive norm parameters, chunk i of the vector, as fp32
template <typename W> __device__ __forceinline__ void load_param8(const void* p, int i, float (&w)[8]) {
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(p) + i);
  const uint32_t a[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    w[2 * j] = lo_of<W>(a[j]);
    w[2 * j + 1] = hi_of<W>(a[j]);
  }
}
template <> __device__ __forceinline__ void load_param8<float>(const void* p, int i, float (&w)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p) + 2 * i);
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 2 * i + 1);
  w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
  w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
}

struct NdParams {
  const void* x;
  const void* weight;
  const void* bias;  // layer norm only
  int8_t* q;
  void* scale;       // [M] in the input dtype
  int64_t ldx, ldq;
  int K;
  float eps;
};

// fp32 quotients n / s of two elements, rounded half-to-even and saturated, in the low bytes of the two results.
// Both ends of the bracketed reciprocal are multiplied in and rounded to an integer by the magic addition (packed fp32
// instructions: two elements per issue slot); rounding is monotonic, so where the two agree the exact quotient rounds
// to the same integer.  Where they differ (the quotient is within a few ulp of a half-integer, or is not finite) a
// bit is ORed into `amb` and the caller redoes the chunk with quantise_f32_exact.
__device__ __forceinline__ void quantise_f32_pair(float n0, float n1, const InvBracket& inv, uint32_t& amb, uint32_t& q0, uint32_t& q1) {
  const uint64_t n2 = f32x2(n0, n1);
  float a0, a1, b0, b1;
  split_f32x2(mul_f32x2(n2, f32x2(inv.lo, inv.lo)), a0, a1);
  split_f32x2(add_f32x2(mul_f32x2(n2, f32x2(inv.hi, inv.hi)), f32x2(kRintMagic, kRintMagic)), b0, b1);
  float m0, m1;
  split_f32x2(add_f32x2(f32x2(fminf(a0, 127.f), fminf(a1, 127.f)), f32x2(kRintMagic, kRintMagic)), m0, m1);
  q0 = __float_as_uint(m0);
  q1 = __float_as_uint(m1);
  amb |= (q0 ^ __float_as_uint(b0)) | (q1 ^ __float_as_uint(b1));
}
__device__ __forceinline__ uint32_t quantise_f32_exact(float n, float s) {
  return __float_as_uint(__fadd_rn(fminf(__fdiv_rn(n, s), 127.f), kRintMagic));
}

// LN = false: RMSNorm, LN = true: LayerNorm.  T: dtype of x, W: dtype of the norm parameters (T or float).
// K % 8 == 0, rows of x 16-byte aligned, NCHUNK = 16-byte chunks of the row held by each thread.
template <typename T, typename W, int NCHUNK, bool LN>
__global__ void __launch_bounds__(kNdMaxThreads)
norm_dquant_kernel(const NdParams p) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.x) + row * p.ldx);
  uint2* qr = reinterpret_cast<uint2*>(p.q + row * p.ldq);
  const int nvec = p.K >> 3;
  const float inv_k = 1.f / float(p.K);
  float v[NCHUNK][8];
  float s1 = 0.f;
#pragma unroll
  for (int c = 0; c < NCHUNK; ++c) {
    const int i = c * blockDim.x + threadIdx.x;
    const uint4 u = (i < nvec) ? __ldcs(xr + i) : make_uint4(0, 0, 0, 0);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[c][2 * j] = lo_of<T>(w[j]);
      v[c][2 * j + 1] = hi_of<T>(w[j]);
      if (LN) s1 += v[c][2 * j] + v[c][2 * j + 1];
      else s1 = fmaf(v[c][2 * j], v[c][2 * j], fmaf(v[c][2 * j + 1], v[c][2 * j + 1], s1));
    }
  }
  s1 = block_reduce<false>(s1, red);
  float mean = 0.f, rstd;
  if (LN) {
    mean = s1 * inv_k;
    float s2 = 0.f;
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      if (c * blockDim.x + threadIdx.x < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) s2 = fmaf(v[c][j] - mean, v[c][j] - mean, s2);
      }
    }
    s2 = block_reduce<false>(s2, red);
    rstd = __fdiv_rn(1.f, __fsqrt_rn(s2 * inv_k + p.eps));
  } else {
    rstd = __fdiv_rn(1.f, __fsqrt_rn(s1 * inv_k + p.eps));
  }

  if (LN) {
    // y = layer_norm(x) rounded to T and re-packed; from here on this is the per-token quantiser on y
    uint4 y[NCHUNK];
    uint32_t m2 = 0;
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int i = c * blockDim.x + threadIdx.x;
      y[c] = make_uint4(0, 0, 0, 0);
      if (i < nvec) {
        float w[8], b[8];
        load_param8<W>(p.weight, i, w);
        load_param8<W>(p.bias, i, b);
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float n0 = __fmul_rn(__fmul_rn(v[c][2 * j] - mean, rstd), w[2 * j]) + b[2 * j];
          const float n1 = __fmul_rn(__fmul_rn(v[c][2 * j + 1] - mean, rstd), w[2 * j + 1]) + b[2 * j + 1];
          o[j] = pack2<T>(n0, n1);
          m2 = absmax2(m2, o[j], T());
        }
        y[c] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
    const float amax = block_absmax_keep_nan(max_keep_nan(lo_of<T>(m2), hi_of<T>(m2)), red);
    const float s = round_to<T>(__fdiv_rn(amax, 127.0f));
    if (threadIdx.x == 0) reinterpret_cast<T*>(p.scale)[row] = from_f32<T>(s);
    const InvBracket inv2 = inv_bracket(s);
    // constant row and zero bias (0 / 0, which the cast turns into 0), a scale too small to invert, or a row with a
    // NaN or an infinity in it (every normalised value and the scale are NaN; NaN quotients are written as 0)
    const bool plain = !usable_scale(s) || inv_overflowed(inv2);
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int i = c * blockDim.x + threadIdx.x;
      if (i < nvec) {
        const uint32_t w[4] = {y[c].x, y[c].y, y[c].z, y[c].w};
        uint32_t o[2];
        uint32_t amb = plain ? 1u : 0u;
        if (!plain) {
#pragma unroll
          for (int h = 0; h < 2; ++h)
            o[h] = __byte_perm(quantise_pair<T>(w[2 * h], inv2, amb), quantise_pair<T>(w[2 * h + 1], inv2, amb), 0x5410);
        }
        if (amb != 0) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int q0 = quantise_one<T>(lo_of<T>(w[2 * h]), s), q1 = quantise_one<T>(hi_of<T>(w[2 * h]), s);
            const int q2 = quantise_one<T>(lo_of<T>(w[2 * h + 1]), s), q3 = quantise_one<T>(hi_of<T>(w[2 * h + 1]), s);
            o[h] = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) | (uint32_t(q3 & 0xff) << 24);
          }
        }
        __stcs(qr + i, make_uint2(o[0], o[1]));
      }
    }
  } else {
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int i = c * blockDim.x + threadIdx.x;
      if (i < nvec) {
        float w[8];
        load_param8<W>(p.weight, i, w);
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          // (x * rstd) * w, two elements per instruction
          split_f32x2(mul_f32x2(mul_f32x2(f32x2(v[c][j], v[c][j + 1]), f32x2(rstd, rstd)), f32x2(w[j], w[j + 1])), v[c][j], v[c][j + 1]);
          amax = max_keep_nan(max_keep_nan(amax, v[c][j]), v[c][j + 1]);
        }
      }
    }
    amax = block_absmax_keep_nan(amax, red);
    const float s = __fdiv_rn(amax, 127.f);
    if (threadIdx.x == 0) reinterpret_cast<T*>(p.scale)[row] = from_f32<T>(s);
    // every normalised value is 0 (0 / 0, which the cast turns into 0), or the row holds a NaN or an infinity: then
    // the scale is NaN (infinite if only the product overflowed), every quotient is NaN or 0, and q is written as 0
    const bool zero = !usable_scale(s);
    const InvBracket inv2 = inv_bracket(s);
    const uint32_t amb0 = inv_overflowed(inv2) ? 1u : 0u;
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int i = c * blockDim.x + threadIdx.x;
      if (i < nvec) {
        uint32_t o[2] = {0u, 0u};
        if (!zero) {
          uint32_t amb = amb0;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t q0, q1, q2, q3;
            quantise_f32_pair(v[c][4 * h], v[c][4 * h + 1], inv2, amb, q0, q1);
            quantise_f32_pair(v[c][4 * h + 2], v[c][4 * h + 3], inv2, amb, q2, q3);
            o[h] = __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
          }
          if (amb != 0) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t q0 = quantise_f32_exact(v[c][4 * h], s), q1 = quantise_f32_exact(v[c][4 * h + 1], s);
              const uint32_t q2 = quantise_f32_exact(v[c][4 * h + 2], s), q3 = quantise_f32_exact(v[c][4 * h + 3], s);
              o[h] = __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
            }
          }
        }
        __stcs(qr + i, make_uint2(o[0], o[1]));
      }
    }
  }
}

template <typename T, typename W, bool LN>
int launch_nd(const NdParams& p, int64_t M, cudaStream_t st) {
  // block size: the smallest of 256 / 512 / 1024 that keeps a thread at <= 4 chunks
  const int nvec = p.K / 8;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 256) threads = (nvec <= 256 * 4) ? 256 : (nvec <= 512 * 4) ? 512 : kNdMaxThreads;
  const int nchunk = (nvec + threads - 1) / threads;
  const dim3 grid(static_cast<unsigned>(M));
  if (nchunk <= 1) norm_dquant_kernel<T, W, 1, LN><<<grid, threads, 0, st>>>(p);
  else if (nchunk <= 2) norm_dquant_kernel<T, W, 2, LN><<<grid, threads, 0, st>>>(p);
  else norm_dquant_kernel<T, W, 4, LN><<<grid, threads, 0, st>>>(p);
  return check_cuda(cudaGetLastError(), LN ? "layer_norm_dquant launch" : "rms_norm_dquant launch");
}

template <typename T, bool LN>
int launch_nd_w(const NdParams& p, int w_dtype, int64_t M, cudaStream_t st) {
  return w_dtype == FNN_F32 ? launch_nd<T, float, LN>(p, M, st) : launch_nd<T, T, LN>(p, M, st);
}

int norm_dquant(bool ln, const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* weight,
                const void* bias, int w_dtype, float eps, int8_t* q, int64_t ldq, void* scale, void* stream) {
  const char* name = ln ? "layer_norm_dquant" : "rms_norm_dquant";
  if (M < 0 || K <= 0 || ldx < K || ldq < K) return fail(FNN_ERR_SHAPE, "%s: M=%lld K=%lld ldx=%lld ldq=%lld", name, (long long)M, (long long)K, (long long)ldx, (long long)ldq);
  if (x_dtype != FNN_F16 && x_dtype != FNN_BF16) return fail(FNN_ERR_DTYPE, "%s: input must be f16 or bf16 (got dtype code %d)", name, x_dtype);
  if (w_dtype != x_dtype && w_dtype != FNN_F32)
    return fail(FNN_ERR_DTYPE, "%s: the norm parameters must have the dtype of x or be f32 (got dtype code %d)", name, w_dtype);
  if (M == 0) return FNN_OK;
  if (!x || !weight || !q || !scale || (ln && !bias)) return fail(FNN_ERR_NULL_POINTER, "%s: null tensor pointer", name);
  if (K % 8 != 0 || K > int64_t(kNdMaxThreads) * 8 * 4)
    return fail(FNN_ERR_UNSUPPORTED, "%s: the row length must be a multiple of 8 and at most %d (got %lld)", name, kNdMaxThreads * 32, (long long)K);
  if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || ldx % 8 != 0 || reinterpret_cast<uintptr_t>(q) % 8 != 0 || ldq % 8 != 0)
    return fail(FNN_ERR_ALIGNMENT, "%s: rows of x must be 16-byte aligned and rows of q 8-byte aligned", name);
  if (reinterpret_cast<uintptr_t>(weight) % 16 != 0 || (ln && reinterpret_cast<uintptr_t>(bias) % 16 != 0))
    return fail(FNN_ERR_ALIGNMENT, "%s: the norm parameters must be 16-byte aligned", name);
  if (M > INT32_MAX) return fail(FNN_ERR_SHAPE, "%s: M must be below 2^31", name);
  NdParams p{x, weight, bias, q, scale, ldx, ldq, int(K), eps};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (x_dtype == FNN_F16) return ln ? launch_nd_w<__half, true>(p, w_dtype, M, st) : launch_nd_w<__half, false>(p, w_dtype, M, st);
  return ln ? launch_nd_w<__nv_bfloat16, true>(p, w_dtype, M, st) : launch_nd_w<__nv_bfloat16, false>(p, w_dtype, M, st);
}

}  // namespace
}  // namespace fnn

extern "C" int fnn_rms_norm_dquant(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* weight,
                                   int w_dtype, float eps, int8_t* q, int64_t ldq, void* scale, void* stream) {
  return fnn::norm_dquant(false, x, x_dtype, M, K, ldx, weight, nullptr, w_dtype, eps, q, ldq, scale, stream);
}

extern "C" int fnn_layer_norm_dquant(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const void* weight,
                                     const void* bias, int w_dtype, float eps, int8_t* q, int64_t ldq, void* scale,
                                     void* stream) {
  return fnn::norm_dquant(true, x, x_dtype, M, K, ldx, weight, bias, w_dtype, eps, q, ldq, scale, stream);
}
