// Device helpers shared by the kernels that quantise a row to int8 in the arithmetic of a 16-bit dtype T
// (per-token dynamic quantisation and the layer-norm producer): q = rint(T(x / s)) with the int8 cast saturating.
//
// The per-element division is replaced by two multiplications with a reciprocal bracketed from below and above:
// where both products round to the same T value the exact quotient does too; only the rare elements next to a
// rounding midpoint of T take the exact division.  rint and the int8 cast are one magic-number addition (no
// conversion instructions).
#pragma once
#include "common.cuh"

namespace fnn {

template <typename T> __device__ __forceinline__ float round_to(float v) {
  return to_f32(from_f32<T>(v));
}

template <typename T> __device__ __forceinline__ int quantise_one(float x, float s) {
  const float r = rintf(round_to<T>(__fdiv_rn(x, s)));
  if (r != r) return 0;  // 0/0 on an all-zero row, anything over a NaN scale, infinity over an infinite scale
  return static_cast<int>(fminf(fmaxf(r, -128.f), 127.f));
}

// The two halves of a packed pair as fp32.  bf16 is the top half of an fp32, so one shift or one mask each.
template <typename T> __device__ __forceinline__ float lo_of(uint32_t w);
template <typename T> __device__ __forceinline__ float hi_of(uint32_t w);
template <> __device__ __forceinline__ float lo_of<__nv_bfloat16>(uint32_t w) { return __uint_as_float(w << 16); }
template <> __device__ __forceinline__ float hi_of<__nv_bfloat16>(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
template <> __device__ __forceinline__ float lo_of<__half>(uint32_t w) {
  return __low2float(*reinterpret_cast<const __half2*>(&w));
}
template <> __device__ __forceinline__ float hi_of<__half>(uint32_t w) {
  return __high2float(*reinterpret_cast<const __half2*>(&w));
}

// Bits of fp32 that a conversion to T drops, and the midpoint pattern among them.
template <typename T> struct DropBits;
template <> struct DropBits<__nv_bfloat16> { static constexpr uint32_t mask = 0xFFFFu, mid = 0x8000u; };
template <> struct DropBits<__half> { static constexpr uint32_t mask = 0x1FFFu, mid = 0x1000u; };

// 1/s bracketed from below and above: x * lo and x * hi enclose the true quotient x / s (the reciprocal and the
// product are each within half an ulp, the factors move it by 8 ulp).
struct InvBracket {
  float lo, hi;
};
__device__ __forceinline__ InvBracket inv_bracket(float s) {
  const float inv = __frcp_rn(s);
  return {__fmul_rn(inv, 0.99999952316284f), __fmul_rn(inv, 1.00000047683716f)};  // 1 -+ 2^-21
}

// A subnormal scale has no finite reciprocal: such rows take the exact division throughout.
__device__ __forceinline__ bool inv_overflowed(const InvBracket& inv) { return !(inv.hi <= 3.4028234e38f); }

// min(t, 127) on a packed pair
__device__ __forceinline__ uint32_t min2_127(uint32_t t2, __half) {
  const __half2 r = __hmin2(*reinterpret_cast<const __half2*>(&t2), __float2half2_rn(127.f));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t min2_127(uint32_t t2, __nv_bfloat16) {
  const __nv_bfloat162 r = __hmin2(*reinterpret_cast<const __nv_bfloat162*>(&t2), __float2bfloat162_rn(127.f));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// Packed fp32 arithmetic (two independent IEEE operations per instruction, half the issue slots).
__device__ __forceinline__ uint64_t f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ void split_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// Two elements at once: returns the two quantised bytes in bits 0-7 and 8-15.  Both ends of the bracket are
// rounded to T (one packed conversion each); rounding is monotonic, so where the two agree the exact quotient rounds
// to the same T value.  Where they differ a bit is ORed into `amb` and the caller redoes the chunk with the exact
// division (about one element in 5000).  The two multiplications per end and the two magic additions are packed
// fp32 instructions.
template <typename T> __device__ __forceinline__ uint32_t quantise_pair(uint32_t w, const InvBracket& inv, uint32_t& amb) {
  const uint64_t x = f32x2(lo_of<T>(w), hi_of<T>(w));
  float a0, a1, b0, b1;
  split_f32x2(mul_f32x2(x, f32x2(inv.lo, inv.lo)), a0, a1);
  split_f32x2(mul_f32x2(x, f32x2(inv.hi, inv.hi)), b0, b1);
  const uint32_t t2 = pack2<T>(a0, a1);
  amb |= t2 ^ pack2<T>(b0, b1);
  const uint32_t tc = min2_127(t2, T());  // |t| <= 128; only +128 needs the clamp (one packed instruction)
  float q0, q1;
  split_f32x2(add_f32x2(f32x2(lo_of<T>(tc), hi_of<T>(tc)), f32x2(12582912.f, 12582912.f)), q0, q1);
  return __byte_perm(__float_as_uint(q0), __float_as_uint(q1), 0x0040);  // low bytes of q0, q1 in bytes 0 and 1
}

// Same result as quantise_one for s > 0, returned in the low byte (two's complement).
template <typename T> __device__ __forceinline__ uint32_t quantise_fast(float x, float s, float inv_s) {
  float r = __fmul_rn(x, inv_s);
  // ambiguous when the dropped bits are within 3 ulp of the rounding midpoint
  const uint32_t d = (__float_as_uint(r) & DropBits<T>::mask) - (DropBits<T>::mid - 3u);
  if (d <= 6u) r = __fdiv_rn(x, s);
  const float t = fminf(round_to<T>(r), 127.f);  // |t| <= 128; only +128 needs the clamp
  // 1.5 * 2^23 + t rounds t half-to-even and leaves the integer in the low mantissa bits
  return __float_as_uint(__fadd_rn(t, 12582912.f));
}

// running max of |x| over packed pairs, kept as a packed pair (no conversion in the first pass); a NaN element
// makes its half NaN from then on
__device__ __forceinline__ uint32_t absmax2(uint32_t m, uint32_t w, __half) {
  const __half2 r = __hmax2_nan(*reinterpret_cast<__half2*>(&m), __habs2(*reinterpret_cast<__half2*>(&w)));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t absmax2(uint32_t m, uint32_t w, __nv_bfloat16) {
  const __nv_bfloat162 r = __hmax2_nan(*reinterpret_cast<__nv_bfloat162*>(&m), __habs2(*reinterpret_cast<__nv_bfloat162*>(&w)));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// Maximum that keeps a NaN (fmaxf would drop it): one instruction, max.NaN.f32.  `max_keep_nan(a, b)` takes |b|,
// so a running maximum that starts at 0 stays non-negative.
__device__ __forceinline__ float max_keep_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(fabsf(b)));
  return r;
}
// max_keep_nan over the whole block; `red` holds 32 floats.  Every thread gets the result.
__device__ __forceinline__ float block_absmax_keep_nan(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max_keep_nan(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = (blockDim.x + 31) >> 5;
  __syncthreads();  // `red` may still be read from an earlier reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  v = (lane < nwarp) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max_keep_nan(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// a scale the fast path can use: positive and finite (NaN and infinity fail both comparisons or the second)
__device__ __forceinline__ bool usable_scale(float s) { return s > 0.f && s <= 3.4028234e38f; }

}  // namespace fnn
