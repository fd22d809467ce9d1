// Device helpers shared by the kernels that quantise a row to int8 in the arithmetic of a 16-bit dtype T
// (per-token dynamic quantisation and the layer-norm producer): q = rint(T(x / s)) with the int8 cast saturating.
//
// The per-element division is replaced by a multiplication with 1/s plus a check: x * (1/s) is within 2 ulp of
// the true quotient, so rounding it to T gives the same value unless it lies within a few ulp of a midpoint
// between two T values; only those rare elements take the exact division.  rint and the int8 cast are one
// magic-number addition (no conversion instructions).
#pragma once
#include "common.cuh"

namespace fnn {

template <typename T> __device__ __forceinline__ float round_to(float v) {
  return to_f32(from_f32<T>(v));
}

template <typename T> __device__ __forceinline__ int quantise_one(float x, float s) {
  const float r = rintf(round_to<T>(__fdiv_rn(x, s)));
  if (r != r) return 0;  // 0/0 on an all-zero row
  return static_cast<int>(fminf(fmaxf(r, -128.f), 127.f));
}

template <typename T> __device__ __forceinline__ float lo_of(uint32_t w) {
  const uint16_t l = static_cast<uint16_t>(w & 0xffffu);
  return to_f32(*reinterpret_cast<const T*>(&l));
}
template <typename T> __device__ __forceinline__ float hi_of(uint32_t w) {
  const uint16_t h = static_cast<uint16_t>(w >> 16);
  return to_f32(*reinterpret_cast<const T*>(&h));
}

// Bits of fp32 that a conversion to T drops, and the midpoint pattern among them.
template <typename T> struct DropBits;
template <> struct DropBits<__nv_bfloat16> { static constexpr uint32_t mask = 0xFFFFu, mid = 0x8000u; };
template <> struct DropBits<__half> { static constexpr uint32_t mask = 0x1FFFu, mid = 0x1000u; };

// Two elements at once: returns the two quantised bytes in bits 0-7 and 8-15, and ORs into `amb` a word whose
// sign bit is set when either x * (1/s) lies within 3 ulp of a rounding midpoint of T (the caller then redoes
// the whole chunk with the exact division; that is rare).
template <typename T> __device__ __forceinline__ uint32_t quantise_pair(uint32_t w, float inv_s, uint32_t& amb) {
  const float r0 = __fmul_rn(lo_of<T>(w), inv_s), r1 = __fmul_rn(hi_of<T>(w), inv_s);
  // (dropped bits) - (mid - 3) - 7 wraps below zero exactly when the dropped bits are in [mid-3, mid+3]
  amb |= ((__float_as_uint(r0) & DropBits<T>::mask) - (DropBits<T>::mid + 4u)) & ~((__float_as_uint(r0) & DropBits<T>::mask) - (DropBits<T>::mid - 3u));
  amb |= ((__float_as_uint(r1) & DropBits<T>::mask) - (DropBits<T>::mid + 4u)) & ~((__float_as_uint(r1) & DropBits<T>::mask) - (DropBits<T>::mid - 3u));
  const uint32_t t2 = pack2<T>(r0, r1);  // both rounded to T in one instruction
  const float t0 = fminf(lo_of<T>(t2), 127.f), t1 = fminf(hi_of<T>(t2), 127.f);
  const uint32_t q0 = __float_as_uint(__fadd_rn(t0, 12582912.f)), q1 = __float_as_uint(__fadd_rn(t1, 12582912.f));
  return __byte_perm(q0, q1, 0x0040);  // low bytes of q0, q1 in bytes 0 and 1
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

// running max of |x| over packed pairs, kept as a packed pair (no conversion in the first pass)
__device__ __forceinline__ uint32_t absmax2(uint32_t m, uint32_t w, __half) {
  const __half2 r = __hmax2(*reinterpret_cast<__half2*>(&m), __habs2(*reinterpret_cast<__half2*>(&w)));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t absmax2(uint32_t m, uint32_t w, __nv_bfloat16) {
  const __nv_bfloat162 r = __hmax2(*reinterpret_cast<__nv_bfloat162*>(&m), __habs2(*reinterpret_cast<__nv_bfloat162*>(&w)));
  return *reinterpret_cast<const uint32_t*>(&r);
}

}  // namespace fnn
