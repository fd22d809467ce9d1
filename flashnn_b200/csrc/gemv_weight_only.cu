// Weight-only GEMV / skinny GEMM for decode shapes (M <= 16): fp16/bf16
// activations x int8 or packed-int4 weights, per-channel or group-wise scales.
//
// The op is HBM-bound (every weight byte is read exactly once), so the kernel is
// built around 16-byte-per-lane asynchronous weight copies and register-level expansion:
//   - a CTA owns 16 output channels (8 packed rows for int4, 16 rows for int8)
//     and its 8 warps split K;
//   - each lane expands its weight bytes to 16-bit floats with
//     PRMT/LOP3 bit tricks (no int->float conversions) and uses them as the
//     16 x 16 operand of mma.sync.m16n8k16; the activations are the narrow
//     16 x 8 operand, so one weight fragment serves up to 8 tokens (two MMAs
//     for 9..16 tokens);
//   - the MMA accumulates x*w in fp32 over one scale group; the group scale
//     (and zero-point) is applied to that partial sum in fp32, so w*s is never
//     rounded to 16 bits;
//   - partial sums of the 8 warps meet in shared memory; bias is added in fp32
//     and the result is rounded once.
// The int4 fragments carry a constant offset (and zero-points add another): both are
// removed per group as  -(offset + zp) * s * sum_k x, with sum_k x produced in the
// accumulator layout by a second MMA against an all-ones operand.
#include <type_traits>

#include "async_copy.cuh"
#include "common.cuh"
#include "weight_only.cuh"

namespace fnn {
constexpr int kStepK = 64;   // K covered by one warp-wide 128-bit load per row (4 lanes x 16 B)
namespace {

constexpr int kGemvWarps = 8;
constexpr int kGemvThreads = kGemvWarps * 32;

template <typename T> struct Mma;
template <> struct Mma<__half> {
  // d = a * b (no accumulator input)
  static __device__ __forceinline__ void run0(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
  }
  static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct Mma<__nv_bfloat16> {
  static __device__ __forceinline__ void run0(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
  }
  static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

// (a & b) ^ c in one LOP3 (truth table 0x6A); b and c are register operands so the compiler cannot split it
// into two immediate-operand instructions
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b, __half) {
  __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

// Four packed bytes (4 consecutive k of one packed row) -> the MMA A fragment:
//   a[0] = low nibbles  (channel 2j)   at k0, k0+1      a[1] = high nibbles (channel 2j+1) at k0, k0+1
//   a[2] = low nibbles  (channel 2j)   at k0+2, k0+3    a[3] = high nibbles (channel 2j+1) at k0+2, k0+3
// The fragment holds kAlpha * (n + kOffset) for the signed nibble n, exactly, built with logic ops and
// byte permutes only: no conversion and no subtraction per element.  The constant part is taken out
// once per scale group:  sum_k n_k x_k = (sum_k a_k x_k) / kAlpha - kOffset * sum_k x_k.
template <typename T> struct Ones;  // two packed 1.0 values
template <> struct Ones<__nv_bfloat16> { static constexpr uint32_t v = 0x3F803F80u; };
template <> struct Ones<__half> { static constexpr uint32_t v = 0x3C003C00u; };

template <typename T> struct Int4Frag;
template <> struct Int4Frag<__nv_bfloat16> {
  // byte (n ^ 8) under a 0x43 high byte is the bf16 value 128 + (n ^ 8) = n + 136
  static constexpr float kInvAlpha = 1.f, kOffset = 136.f;
  static __device__ __forceinline__ void make(uint32_t w, uint32_t (&a)[4]) {
    const uint32_t lo = and_xor(w, 0x0F0F0F0Fu, 0x08080808u);
    const uint32_t hi = and_xor(w >> 4, 0x0F0F0F0Fu, 0x08080808u);
    const uint32_t m = 0x43434343u;
    a[0] = prmt(lo, m, 0x4140); a[1] = prmt(hi, m, 0x4140);
    a[2] = prmt(lo, m, 0x4342); a[3] = prmt(hi, m, 0x4342);
  }
};
template <> struct Int4Frag<__half> {
  // byte ((n ^ 8) << 4) under a 0x64 high byte is the fp16 value 1024 + 16 (n ^ 8) = 16 (n + 72)
  static constexpr float kInvAlpha = 0.0625f, kOffset = 72.f;
  static __device__ __forceinline__ void make(uint32_t w, uint32_t (&a)[4]) {
    const uint32_t lo = and_xor(w << 4, 0xF0F0F0F0u, 0x80808080u);
    const uint32_t hi = and_xor(w, 0xF0F0F0F0u, 0x80808080u);
    const uint32_t m = 0x64646464u;
    a[0] = prmt(lo, m, 0x4140); a[1] = prmt(hi, m, 0x4140);
    a[2] = prmt(lo, m, 0x4342); a[3] = prmt(hi, m, 0x4342);
  }
};

// Four int8 (4 consecutive k of one weight row) -> two fragment registers (k0,k0+1), (k0+2,k0+3).
template <typename T> __device__ __forceinline__ void dequant_int8(uint32_t w, uint32_t& r01, uint32_t& r23);
template <> __device__ __forceinline__ void dequant_int8<__half>(uint32_t w, uint32_t& r01, uint32_t& r23) {
  // byte ^ 0x80 under a 0x64 high byte is the fp16 value 1024 + (b + 128)
  const uint32_t u = w ^ 0x80808080u;
  const uint32_t m = 0x64646464u, off = 0x64806480u;  // 1152.0 twice
  r01 = sub2(prmt(u, m, 0x4140), off, __half());
  r23 = sub2(prmt(u, m, 0x4342), off, __half());
}
template <> __device__ __forceinline__ void dequant_int8<__nv_bfloat16>(uint32_t w, uint32_t& r01, uint32_t& r23) {
  // bf16 has no spare mantissa for an 8-bit magic number: go through fp32 (2^23 + u) - (2^23 + 128)
  const uint32_t u = w ^ 0x80808080u;
  const float f0 = __uint_as_float(prmt(u, 0x4B000000u, 0x7650)) - 8388736.f;
  const float f1 = __uint_as_float(prmt(u, 0x4B000000u, 0x7651)) - 8388736.f;
  const float f2 = __uint_as_float(prmt(u, 0x4B000000u, 0x7652)) - 8388736.f;
  const float f3 = __uint_as_float(prmt(u, 0x4B000000u, 0x7653)) - 8388736.f;
  r01 = pack2<__nv_bfloat16>(f0, f1);
  r23 = pack2<__nv_bfloat16>(f2, f3);
}

template <typename T> __device__ __forceinline__ float lo16_f32(uint32_t v);
template <typename T> __device__ __forceinline__ float hi16_f32(uint32_t v);
template <> __device__ __forceinline__ float lo16_f32<__nv_bfloat16>(uint32_t v) { return __uint_as_float(v << 16); }
template <> __device__ __forceinline__ float hi16_f32<__nv_bfloat16>(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
template <> __device__ __forceinline__ float lo16_f32<__half>(uint32_t v) { return __low2float(*reinterpret_cast<__half2*>(&v)); }
template <> __device__ __forceinline__ float hi16_f32<__half>(uint32_t v) { return __high2float(*reinterpret_cast<__half2*>(&v)); }

constexpr int kRing = 8;  // steps (of 64 k) a lane keeps in flight in its shared-memory FIFO

template <int BITS> struct GemvSmem {
  static constexpr int kLaneBytes = (BITS == 4) ? 16 : 32;    // bytes per lane per step
  static constexpr int kSlotBytes = 32 * kLaneBytes;          // one step of one warp
  static constexpr int kWarpBytes = kRing * kSlotBytes;       // [slot][lane]
  static constexpr int kBytes = kGemvWarps * kWarpBytes;
};


// One CTA per row group (16 output channels); its 8 warps split K into equal slices.  Every lane
// streams exactly the weight bytes its own MMA fragments need: 16 bytes per step (64 k) of one
// packed row, copied asynchronously from HBM into the lane's private slot of a shared-memory FIFO
// (cp.async, kRing steps deep, no registers held, no cross-lane traffic, waits stall in hardware
// rather than spin), then read back with one 128-bit shared load.
//   SPU    steps (of 64 k) per partial-sum flush: the scale group for group-wise scales (64, 128 or
//          256), a pseudo-group of 64 or 128 for per-channel scales.  At every flush the fp32 MMA
//          accumulator is corrected for the fragment offset / zero-point, scaled, and added to the
//          running total; partial sums therefore stay small.  The correction needs sum_k x over the
//          group: a second MMA per fragment with an all-ones operand produces it in the accumulator
//          layout, on the otherwise idle tensor pipe.
//   PERCH  per-channel scales: the flush uses scale 1 and the channel scale is applied at the end.
// Host guarantees: K % 512 == 0, the warp slice K/8 is a whole number of flush groups, scale dtype == T
// for group-wise scales.  Tokens beyond M are computed from a clamped (duplicate) row and never stored.
template <typename T, int BITS, int NT, int SPU, bool PERCH>
__global__ void __launch_bounds__(kGemvThreads, (BITS == 4 && NT == 1) ? 4 : 2)
gemv_mma_kernel(const WoParams p) {
  using S = GemvSmem<BITS>;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float red[kGemvWarps][NT][4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int rg = blockIdx.x;
  // channels behind accumulator registers {0,1} (ch_a) and {2,3} (ch_b)
  const int ch_a = (BITS == 4) ? rg * 16 + 2 * g : rg * 16 + g;
  const int ch_b = (BITS == 4) ? ch_a + 1 : ch_a + 8;
  const int64_t last_row = (BITS == 4 ? p.N / 2 : p.N) - 1;
  const int steps_w = p.K / (kStepK * kGemvWarps);
  const int k_begin = warp * steps_w * kStepK;
  const uint8_t* wp = p.qw + min(int64_t(BITS == 4 ? rg * 8 + g : ch_a), last_row) * p.K + k_begin + tig * 16;
  const uint8_t* wp2 = p.qw + min(int64_t(ch_b), last_row) * p.K + k_begin + tig * 16;  // int8 only
  const uint32_t fifo = smem_u32(smem) + warp * S::kWarpBytes + lane * S::kLaneBytes;

  // copy of step (base + J) into FIFO slot J; pointers are advanced by the caller, offsets are immediates
  auto issue = [&](int slot, const uint8_t* w, const uint8_t* w2) {
    cp_async16(fifo + slot * S::kSlotBytes, w);
    if (BITS == 8) cp_async16(fifo + slot * S::kSlotBytes + 16, w2);
  };
  // prologue: the first kRing steps (every step commits a group, real or empty, so counts stay constant)
#pragma unroll
  for (int j = 0; j < kRing; ++j) {
    if (j < steps_w) issue(j, wp + j * kStepK, wp2 + j * kStepK);
    cp_async_commit();
  }

  const uint8_t* xp[NT];  // activations of token g (and g+8), 16 consecutive k per step starting at tig*16
#pragma unroll
  for (int t = 0; t < NT; ++t)
    xp[t] = reinterpret_cast<const uint8_t*>(reinterpret_cast<const T*>(p.act) + int64_t(min(g + 8 * t, p.M - 1)) * p.lda + k_begin + tig * 16);
  // scale pairs: for int4 the two channels are adjacent (one aligned 32-bit load)
  const int sa_i = (BITS == 4) ? min(ch_a, p.N - 2) : min(ch_a, p.N - 1);
  const int sb_i = (BITS == 4) ? sa_i + 1 : min(ch_b, p.N - 1);
  const int64_t group_pitch = int64_t(p.N) * int64_t(sizeof(T));
  const uint8_t* sp = reinterpret_cast<const uint8_t*>(reinterpret_cast<const T*>(p.scale) + int64_t(warp) * (steps_w / SPU) * p.N);
  const uint8_t* zpp = p.zp ? reinterpret_cast<const uint8_t*>(p.zp) + (sp - reinterpret_cast<const uint8_t*>(p.scale)) : nullptr;

  // constant part of the int4 fragment encoding (none for int8, which is expanded exactly)
  constexpr float kInvAlpha = (BITS == 4) ? Int4Frag<T>::kInvAlpha : 1.f;
  constexpr float kOffset = (BITS == 4) ? Int4Frag<T>::kOffset : 0.f;
  constexpr bool kOnes = (BITS == 4);        // always track sum_k x
  const bool ones = kOnes || p.zp != nullptr;  // int8: only when zero-points are given
  const uint32_t one2[4] = {Ones<T>::v, Ones<T>::v, Ones<T>::v, Ones<T>::v};

  float tot[NT][4], acc[NT][4], xsum[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) tot[t][i] = acc[t][i] = xsum[t][i] = 0.f;

  auto load_pair = [&](const uint8_t* base) -> uint32_t {
    const T* s = reinterpret_cast<const T*>(base);
    if (BITS == 4) return __ldg(reinterpret_cast<const uint32_t*>(s + sa_i));
    return uint32_t(__ldg(reinterpret_cast<const uint16_t*>(s + sa_i))) |
           (uint32_t(__ldg(reinterpret_cast<const uint16_t*>(s + sb_i))) << 16);
  };
  // per-channel zero-points are constant along K; group-wise ones are read at each flush
  float za = kOffset / kInvAlpha, zb = kOffset / kInvAlpha;
  if (PERCH && p.zp) {
    za += load_as_f32(p.zp, p.scale_dtype, sa_i) / kInvAlpha;
    zb += load_as_f32(p.zp, p.scale_dtype, sb_i) / kInvAlpha;
  }

  // one step: fragments of 64 k; `first` starts a new flush group (accumulators are overwritten)
  auto compute_step = [&](const uint4& wv, const uint4& w2v, const uint8_t* xstep, bool first) {
    uint32_t xw[NT][8];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const uint4* x4 = reinterpret_cast<const uint4*>(xstep + (xp[t] - xp[0]));
      const uint4 x0 = __ldg(x4), x1 = __ldg(x4 + 1);
      xw[t][0] = x0.x; xw[t][1] = x0.y; xw[t][2] = x0.z; xw[t][3] = x0.w;
      xw[t][4] = x1.x; xw[t][5] = x1.y; xw[t][6] = x1.z; xw[t][7] = x1.w;
    }
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    const uint32_t ww2[4] = {w2v.x, w2v.y, w2v.z, w2v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t a[4];
      if (BITS == 4) {
        Int4Frag<T>::make(ww[q], a);
      } else {
        dequant_int8<T>(ww[q], a[0], a[2]);
        dequant_int8<T>(ww2[q], a[1], a[3]);
      }
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        if (first && q == 0) {
          Mma<T>::run0(acc[t], a, xw[t][0], xw[t][1]);
          if (ones) Mma<T>::run0(xsum[t], one2, xw[t][0], xw[t][1]);
        } else {
          Mma<T>::run(acc[t], a, xw[t][2 * q], xw[t][2 * q + 1]);
          if (ones) Mma<T>::run(xsum[t], one2, xw[t][2 * q], xw[t][2 * q + 1]);
        }
      }
    }
  };
  auto flush = [&](uint32_t sc, const uint8_t* zp_group) {
    float sa = kInvAlpha, sb = kInvAlpha;
    if (!PERCH) { sa *= lo16_f32<T>(sc); sb *= hi16_f32<T>(sc); }
    if (ones) {
      float fa = za, fb = zb;
      if (!PERCH && p.zp) {
        fa += load_as_f32(zp_group, p.scale_dtype, sa_i) / kInvAlpha;
        fb += load_as_f32(zp_group, p.scale_dtype, sb_i) / kInvAlpha;
      }
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        acc[t][0] = fmaf(-fa, xsum[t][0], acc[t][0]); acc[t][1] = fmaf(-fa, xsum[t][1], acc[t][1]);
        acc[t][2] = fmaf(-fb, xsum[t][0], acc[t][2]); acc[t][3] = fmaf(-fb, xsum[t][1], acc[t][3]);
      }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      tot[t][0] = fmaf(sa, acc[t][0], tot[t][0]);
      tot[t][1] = fmaf(sa, acc[t][1], tot[t][1]);
      tot[t][2] = fmaf(sb, acc[t][2], tot[t][2]);
      tot[t][3] = fmaf(sb, acc[t][3], tot[t][3]);
    }
  };

  // main loop: kRing steps per iteration, every shared / global offset an immediate
  const int full = steps_w / kRing * kRing;
  const uint8_t* xq = xp[0];
  for (int s0 = 0; s0 < full; s0 += kRing) {
    uint32_t sc[kRing / SPU];
    if (!PERCH) {
#pragma unroll
      for (int i = 0; i < kRing / SPU; ++i) sc[i] = load_pair(sp + i * group_pitch);
    }
    const bool refill = s0 + 2 * kRing <= steps_w;  // the next-but-one block of steps is complete
#pragma unroll
    for (int j = 0; j < kRing; ++j) {
      cp_async_wait<kRing - 1>();  // step s0+j has landed (at most kRing-1 newer groups pending)
      const uint4 wv = lds128(fifo + j * S::kSlotBytes);
      uint4 w2v = wv;
      if (BITS == 8) w2v = lds128(fifo + j * S::kSlotBytes + 16);
      compute_step(wv, w2v, xq + j * (kStepK * int(sizeof(T))), j % SPU == 0);
      if (refill) issue(j, wp + (kRing + j) * kStepK, wp2 + (kRing + j) * kStepK);
      else if (s0 + kRing + j < steps_w) issue(j, wp + (kRing + j) * kStepK, wp2 + (kRing + j) * kStepK);
      cp_async_commit();
      if ((j + 1) % SPU == 0) flush(PERCH ? 0u : sc[j / SPU], zpp ? zpp + (j / SPU) * group_pitch : nullptr);
    }
    wp += kRing * kStepK;
    wp2 += kRing * kStepK;
    xq += kRing * kStepK * int(sizeof(T));
    sp += (kRing / SPU) * group_pitch;
    if (zpp) zpp += (kRing / SPU) * group_pitch;
  }
  // remainder: fewer than kRing steps, already requested by the block before (or by the prologue)
  for (int s = full; s < steps_w; ++s) {
    const int j = s - full;
    cp_async_wait<0>();
    const uint4 wv = lds128(fifo + j * S::kSlotBytes);
    uint4 w2v = wv;
    if (BITS == 8) w2v = lds128(fifo + j * S::kSlotBytes + 16);
    compute_step(wv, w2v, xq + j * (kStepK * int(sizeof(T))), j % SPU == 0);
    if ((j + 1) % SPU == 0) {
      const int gi = j / SPU;
      flush(PERCH ? 0u : load_pair(sp + gi * group_pitch), zpp ? zpp + gi * group_pitch : nullptr);
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[warp][t][i][lane] = tot[t][i];
  __syncthreads();
  if (warp == 0) {
    T* out = reinterpret_cast<T*>(p.out);
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kGemvWarps; ++w) v += red[w][t][i][lane];
        const int ch = (i < 2) ? ch_a : ch_b;
        const int m = t * 8 + 2 * tig + (i & 1);
        if (ch < p.N && m < p.M) {
          if (PERCH) v *= load_as_f32(p.scale, p.scale_dtype, ch);
          if (p.bias) v += load_as_f32(p.bias, p.bias_dtype, ch);
          out[int64_t(m) * p.ldo + ch] = from_f32<T>(v);
        }
      }
  }
}

// Persistent form of gemv_mma_kernel for the common case (N % 16 == 0, K % 4096 == 0): CTA b handles row
// groups b, b + gridDim.x, ... with the same eight warps and the same K slices throughout, so the per-warp
// set-up is paid once, and each lane's cp.async FIFO (16 steps deep here) runs on across row-group boundaries.
// Activation fragments are fetched one step ahead of their use.  Per row group the only CTA-wide event is
// one barrier for the cross-warp sum; the partial-sum buffer is double-buffered so no second barrier is needed.
template <typename T, int BITS, int NT, int SPU, bool PERCH>
__global__ void __launch_bounds__(kGemvThreads, 2)
gemv_mma_persistent_kernel(const WoParams p, const int num_rg) {
  using S = GemvSmem<BITS>;
  constexpr int kDepth = 2 * kRing;  // FIFO slots per lane: two blocks of kRing steps
  constexpr int kWarpFifo = kDepth * S::kSlotBytes;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float red[2][kGemvWarps][NT][4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  constexpr int R = (BITS == 4) ? 8 : 16;  // weight rows per row group
  const int steps_w = p.K / (kStepK * kGemvWarps);
  const int k_begin = warp * steps_w * kStepK;
  int rg = blockIdx.x;
  const uint8_t* wp = p.qw + (int64_t(rg) * R + g) * p.K + k_begin + tig * 16;  // row of accumulators {0,1}
  const int64_t row_b = int64_t(8) * p.K;                                        // int8: row of accumulators {2,3}
  const int64_t rg_stride = int64_t(gridDim.x) * R * p.K;
  const uint32_t fifo = smem_u32(smem) + warp * kWarpFifo + lane * S::kLaneBytes;
  const int groups_w = steps_w / SPU;
  float* xs = reinterpret_cast<float*>(smem + kGemvWarps * kWarpFifo) + warp * groups_w * (8 * NT);  // [group][token]
  auto issue = [&](uint32_t slot_addr, const uint8_t* w) {
    cp_async16(slot_addr, w);
    if (BITS == 8) cp_async16(slot_addr + 16, w + row_b);
  };
  // weights of step `v` counted from the first step of row group `rg_from` onwards (v may run into later row
  // groups of this CTA); nullptr past the last row group
  auto step_ptr = [&](const uint8_t* wbase, int rg_from, int v) -> const uint8_t* {
    while (v >= steps_w) { v -= steps_w; wbase += rg_stride; rg_from += gridDim.x; }
    return rg_from < num_rg ? wbase + v * kStepK : nullptr;
  };
  // prologue: the first kDepth steps of this CTA's work (every step commits a group, real or empty)
  for (int b = 0; b < 2; ++b) {
    const uint8_t* w = step_ptr(wp, rg, b * kRing);
#pragma unroll
    for (int j = 0; j < kRing; ++j) {
      if (w) issue(fifo + (b * kRing + j) * S::kSlotBytes, w + j * kStepK);
      cp_async_commit();
    }
  }

  const uint8_t* xp[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t)
    xp[t] = reinterpret_cast<const uint8_t*>(reinterpret_cast<const T*>(p.act) + int64_t(min(g + 8 * t, p.M - 1)) * p.lda + k_begin + tig * 16);
  // channel offsets inside a row group, and this warp's first scale group
  const int ca = (BITS == 4) ? 2 * g : g;
  const int cb = (BITS == 4) ? 2 * g + 1 : g + 8;
  const int64_t group_pitch = int64_t(p.N) * int64_t(sizeof(T));
  const uint8_t* sp0 = reinterpret_cast<const uint8_t*>(reinterpret_cast<const T*>(p.scale) + int64_t(warp) * (steps_w / SPU) * p.N);
  const uint8_t* zp0 = p.zp ? reinterpret_cast<const uint8_t*>(p.zp) + (sp0 - reinterpret_cast<const uint8_t*>(p.scale)) : nullptr;

  constexpr float kInvAlpha = (BITS == 4) ? Int4Frag<T>::kInvAlpha : 1.f;
  constexpr float kOffset = (BITS == 4) ? Int4Frag<T>::kOffset : 0.f;
  const bool ones = (BITS == 4) || p.zp != nullptr;
  const uint32_t one2[4] = {Ones<T>::v, Ones<T>::v, Ones<T>::v, Ones<T>::v};

  float tot[NT][4], acc[NT][4], xsum[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) tot[t][i] = acc[t][i] = xsum[t][i] = 0.f;

  auto compute_step = [&](const uint4& wv, const uint4& w2v, const uint4 (&xv)[NT][2], bool first) {
    uint32_t xw[NT][8];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      xw[t][0] = xv[t][0].x; xw[t][1] = xv[t][0].y; xw[t][2] = xv[t][0].z; xw[t][3] = xv[t][0].w;
      xw[t][4] = xv[t][1].x; xw[t][5] = xv[t][1].y; xw[t][6] = xv[t][1].z; xw[t][7] = xv[t][1].w;
    }
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    const uint32_t ww2[4] = {w2v.x, w2v.y, w2v.z, w2v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t a[4];
      if (BITS == 4) {
        Int4Frag<T>::make(ww[q], a);
      } else {
        dequant_int8<T>(ww[q], a[0], a[2]);
        dequant_int8<T>(ww2[q], a[1], a[3]);
      }
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        if (first && q == 0) Mma<T>::run0(acc[t], a, xw[t][0], xw[t][1]);
        else Mma<T>::run(acc[t], a, xw[t][2 * q], xw[t][2 * q + 1]);
      }
    }
  };

  // sum_k x over every flush group of this warp's K slice, once per CTA: an all-ones operand against the
  // activation fragments leaves the sums in the accumulator layout (columns = tokens); lanes 0..3 store them
  if (ones) {
    const uint8_t* xq = xp[0];
    for (int gi = 0; gi < groups_w; ++gi) {
#pragma unroll
      for (int j = 0; j < SPU; ++j) {
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const uint4* x4 = reinterpret_cast<const uint4*>(xq + (xp[t] - xp[0]));
          const uint4 x0 = __ldg(x4), x1 = __ldg(x4 + 1);
          if (j == 0) Mma<T>::run0(xsum[t], one2, x0.x, x0.y); else Mma<T>::run(xsum[t], one2, x0.x, x0.y);
          Mma<T>::run(xsum[t], one2, x0.z, x0.w);
          Mma<T>::run(xsum[t], one2, x1.x, x1.y);
          Mma<T>::run(xsum[t], one2, x1.z, x1.w);
        }
        xq += kStepK * int(sizeof(T));
      }
      if (g == 0) {
#pragma unroll
        for (int t = 0; t < NT; ++t)
          *reinterpret_cast<float2*>(xs + gi * (8 * NT) + t * 8 + 2 * tig) = make_float2(xsum[t][0], xsum[t][1]);
      }
    }
    __syncwarp();
  }

  int parity = 0;
  uint32_t half = 0;  // which half of the FIFO the block being consumed sits in
  for (; rg < num_rg; rg += gridDim.x) {
    const int ch_a = rg * 16 + ca, ch_b = rg * 16 + cb;
    const uint8_t* sp = sp0;
    const uint8_t* zpp = zp0;
    float za = kOffset / kInvAlpha, zb = kOffset / kInvAlpha;
    if (PERCH && p.zp) {
      za += load_as_f32(p.zp, p.scale_dtype, ch_a) / kInvAlpha;
      zb += load_as_f32(p.zp, p.scale_dtype, ch_b) / kInvAlpha;
    }
    auto load_pair = [&](const uint8_t* base) -> uint32_t {
      const T* sc = reinterpret_cast<const T*>(base);
      if (BITS == 4) return __ldg(reinterpret_cast<const uint32_t*>(sc + ch_a));
      return uint32_t(__ldg(reinterpret_cast<const uint16_t*>(sc + ch_a))) |
             (uint32_t(__ldg(reinterpret_cast<const uint16_t*>(sc + ch_b))) << 16);
    };
    auto flush = [&](int gi, uint32_t sc, const uint8_t* zp_group) {
      float sa = kInvAlpha, sb = kInvAlpha;
      if (!PERCH) { sa *= lo16_f32<T>(sc); sb *= hi16_f32<T>(sc); }
      if (ones) {
        float fa = za, fb = zb;
        if (!PERCH && p.zp) {
          fa += load_as_f32(zp_group, p.scale_dtype, ch_a) / kInvAlpha;
          fb += load_as_f32(zp_group, p.scale_dtype, ch_b) / kInvAlpha;
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const float2 x = *reinterpret_cast<const float2*>(xs + gi * (8 * NT) + t * 8 + 2 * tig);
          acc[t][0] = fmaf(-fa, x.x, acc[t][0]); acc[t][1] = fmaf(-fa, x.y, acc[t][1]);
          acc[t][2] = fmaf(-fb, x.x, acc[t][2]); acc[t][3] = fmaf(-fb, x.y, acc[t][3]);
        }
      }
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        tot[t][0] = fmaf(sa, acc[t][0], tot[t][0]);
        tot[t][1] = fmaf(sa, acc[t][1], tot[t][1]);
        tot[t][2] = fmaf(sb, acc[t][2], tot[t][2]);
        tot[t][3] = fmaf(sb, acc[t][3], tot[t][3]);
      }
    };

    const uint8_t* xq = xp[0];
    for (int s0 = 0; s0 < steps_w; s0 += kRing) {
      uint32_t sc[kRing / SPU];
      if (!PERCH) {
#pragma unroll
        for (int i = 0; i < kRing / SPU; ++i) sc[i] = load_pair(sp + i * group_pitch);
      }
      // the slots of this block are refilled with the block two ahead (same row group or a later one)
      const uint8_t* wfill = step_ptr(wp, rg, s0 + kDepth);
      const uint32_t slots = fifo + half * (kRing * S::kSlotBytes);
      // activations are fetched one step ahead of their use
      uint4 xn[NT][2];
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const uint4* x4 = reinterpret_cast<const uint4*>(xq + (xp[t] - xp[0]));
        xn[t][0] = __ldg(x4);
        xn[t][1] = __ldg(x4 + 1);
      }
#pragma unroll
      for (int j = 0; j < kRing; ++j) {
        uint4 xc[NT][2];
#pragma unroll
        for (int t = 0; t < NT; ++t) { xc[t][0] = xn[t][0]; xc[t][1] = xn[t][1]; }
        if (j + 1 < kRing) {
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const uint4* x4 = reinterpret_cast<const uint4*>(xq + (j + 1) * (kStepK * int(sizeof(T))) + (xp[t] - xp[0]));
            xn[t][0] = __ldg(x4);
            xn[t][1] = __ldg(x4 + 1);
          }
        }
        cp_async_wait<kDepth - 1>();  // step s0+j has landed (at most kDepth-1 newer groups pending)
        const uint4 wv = lds128(slots + j * S::kSlotBytes);
        uint4 w2v = wv;
        if (BITS == 8) w2v = lds128(slots + j * S::kSlotBytes + 16);
        compute_step(wv, w2v, xc, j % SPU == 0);
        if (wfill) issue(slots + j * S::kSlotBytes, wfill + j * kStepK);
        cp_async_commit();
        if ((j + 1) % SPU == 0) flush((s0 + j) / SPU, PERCH ? 0u : sc[j / SPU], zpp ? zpp + (j / SPU) * group_pitch : nullptr);
      }
      half ^= 1;
      xq += kRing * kStepK * int(sizeof(T));
      sp += (kRing / SPU) * group_pitch;
      if (zpp) zpp += (kRing / SPU) * group_pitch;
    }

    // cross-warp sum of this row group; the other half of `red` is still being read from the previous one
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) { red[parity][warp][t][i][lane] = tot[t][i]; tot[t][i] = 0.f; }
    __syncthreads();
    if (warp == 0) {
      T* out = reinterpret_cast<T*>(p.out);
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < kGemvWarps; ++w) v += red[parity][w][t][i][lane];
          const int ch = (i < 2) ? ch_a : ch_b;
          const int m = t * 8 + 2 * tig + (i & 1);
          if (m < p.M) {
            if (PERCH) v *= load_as_f32(p.scale, p.scale_dtype, ch);
            if (p.bias) v += load_as_f32(p.bias, p.bias_dtype, ch);
            out[int64_t(m) * p.ldo + ch] = from_f32<T>(v);
          }
        }
    }
    parity ^= 1;
    wp += rg_stride;
  }
  cp_async_wait<0>();
}

// Correctness path for everything the fast kernels do not cover (any M, K, group size):
// one thread per output element, fp32 throughout, same order of operations per group.
template <typename T, int BITS>
__global__ void wo_generic_kernel(const WoParams p) {
  const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= int64_t(p.M) * p.N) return;
  const int m = int(idx / p.N), n = int(idx % p.N);
  const T* x = reinterpret_cast<const T*>(p.act) + int64_t(m) * p.lda;
  const uint8_t* wr = p.qw + int64_t(BITS == 4 ? n / 2 : n) * p.K;
  const int glen = p.group > 0 ? p.group : p.K;
  float total = 0.f;
  for (int k0 = 0, gi = 0; k0 < p.K; k0 += glen, ++gi) {
    const int64_t so = p.group > 0 ? int64_t(gi) * p.N + n : n;
    const float s = load_as_f32(p.scale, p.scale_dtype, so);
    const float z = p.zp ? load_as_f32(p.zp, p.scale_dtype, so) : 0.f;
    float acc = 0.f, xs = 0.f;
    const int k1 = min(k0 + glen, p.K);
    for (int k = k0; k < k1; ++k) {
      int w;
      if (BITS == 4) {
        const int b = wr[k];
        const int nib = (n & 1) ? (b >> 4) : (b & 0xF);
        w = (nib ^ 8) - 8;
      } else {
        w = int(static_cast<int8_t>(wr[k]));
      }
      const float xf = to_f32(x[k]);
      acc = fmaf(xf, float(w), acc);
      xs += xf;
    }
    total += s * (acc - z * xs);
  }
  if (p.bias) total += load_as_f32(p.bias, p.bias_dtype, n);
  reinterpret_cast<T*>(p.out)[int64_t(m) * p.ldo + n] = from_f32<T>(total);
}

// Decode shapes the tensor-core kernels decline (K not a multiple of 512, unusual group sizes): one warp per weight
// row (two channels of packed int4, one of int8), lanes stride over K with coalesced 16-byte loads, fp32 throughout,
// one scale group at a time so that w*s is never rounded.  K % 16 == 0, group % 16 == 0 (or per-channel), M <= 16.
template <typename T, int BITS, int MT>
__global__ void __launch_bounds__(256) wo_row_warp_kernel(const WoParams p) {
  constexpr int CH = (BITS == 4) ? 2 : 1;  // channels per weight row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  const int rows = (BITS == 4) ? p.N / 2 : p.N;
  if (row >= rows) return;
  const uint8_t* wr = p.qw + int64_t(row) * p.K;
  const T* x = reinterpret_cast<const T*>(p.act);
  const int glen = p.group > 0 ? p.group : p.K;
  float tot[MT][CH];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int c = 0; c < CH; ++c) tot[m][c] = 0.f;
  for (int k0 = lane * 16; k0 < p.K; k0 += 32 * 16) {
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wr + k0));
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    float wf[CH][16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int b = int((ww[j >> 2] >> (8 * (j & 3))) & 0xffu);
      if (BITS == 4) {
        wf[0][j] = float(((b & 0xF) ^ 8) - 8);
        wf[CH - 1][j] = float(((b >> 4) ^ 8) - 8);
      } else {
        wf[0][j] = float(int(int8_t(b)));
      }
    }
    // the 16 k of this chunk lie in one scale group
    const int64_t g_off = p.group > 0 ? int64_t(k0 / glen) * p.N : 0;
    float s[CH], z[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int ch = row * CH + c;
      s[c] = load_as_f32(p.scale, p.scale_dtype, g_off + ch);
      z[c] = p.zp ? load_as_f32(p.zp, p.scale_dtype, g_off + ch) : 0.f;
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < p.M) {
        const uint4* xp = reinterpret_cast<const uint4*>(x + int64_t(m) * p.lda + k0);
        const uint4 xa = __ldg(xp), xb = __ldg(xp + 1);
        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        float acc[CH], xs = 0.f;
#pragma unroll
        for (int c = 0; c < CH; ++c) acc[c] = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const uint16_t h = uint16_t(xw[j >> 1] >> (16 * (j & 1)));
          const float xf = to_f32(*reinterpret_cast<const T*>(&h));
          xs += xf;
#pragma unroll
          for (int c = 0; c < CH; ++c) acc[c] = fmaf(xf, wf[c][j], acc[c]);
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) tot[m][c] = fmaf(s[c], acc[c] - z[c] * xs, tot[m][c]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      float v = tot[m][c];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      tot[m][c] = v;
    }
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < p.M) {
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const int ch = row * CH + c;
          float v = tot[m][c];
          if (p.bias) v += load_as_f32(p.bias, p.bias_dtype, ch);
          reinterpret_cast<T*>(p.out)[int64_t(m) * p.ldo + ch] = from_f32<T>(v);
        }
      }
    }
  }
}

// Steps (of 64 k) per partial-sum flush of the fast kernel, or -1 when the fast kernel does not apply.
int gemv_spu(const WoParams& p, int bits, int act_dtype) {
  if (p.M > 16) return -1;
  if (p.K % (kStepK * kGemvWarps) != 0) return -1;
  if (reinterpret_cast<uintptr_t>(p.qw) % 16 != 0) return -1;
  if (reinterpret_cast<uintptr_t>(p.act) % 16 != 0 || p.lda % 8 != 0) return -1;
  if (bits == 4 && (p.N % 2 != 0 || p.N < 2)) return -1;
  const int slice = p.K / kGemvWarps;
  if (p.group == 0) return (slice % (2 * kStepK) == 0) ? 2 : 1;  // pseudo-groups of 128 or 64
  if (p.scale_dtype != act_dtype) return -1;  // group scales are read as packed pairs of T
  if (reinterpret_cast<uintptr_t>(p.scale) % 4 != 0) return -1;
  if (slice % p.group != 0) return -1;  // a warp's K slice must be whole groups
  const int spu = p.group / kStepK;
  if (p.group % kStepK != 0 || (spu != 1 && spu != 2 && spu != 4)) return -1;
  return spu;
}

template <typename T, int BITS>
int launch_wo(WoParams p, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (p.M <= 16) {
    // one to five tokens: integer tensor-pipe kernel (declines shapes it does not cover)
    const int r = gemv_w4_imma(p, BITS, std::is_same<T, __half>::value ? FNN_F16 : FNN_BF16, st);
    if (r >= 0) return r;
    // six to sixteen tokens of packed int4: the kernel that keeps the activations on the SM
    if (BITS == 4 && p.M >= 6) {
      const int r2 = gemv_w4_tok(p, std::is_same<T, __half>::value ? FNN_F16 : FNN_BF16, st);
      if (r2 >= 0) return r2;
    }
  }
  const int spu = gemv_spu(p, BITS, std::is_same<T, __half>::value ? FNN_F16 : FNN_BF16);
  if (spu < 0) {
    // decode shapes outside the tensor-core kernels: coalesced warp-per-row kernel when the rows can be read in
    // 16-byte pieces, else one thread per output
    const bool rows16 = p.M <= 16 && p.K % 16 == 0 && (p.group == 0 || p.group % 16 == 0) &&
                        reinterpret_cast<uintptr_t>(p.qw) % 16 == 0 && reinterpret_cast<uintptr_t>(p.act) % 16 == 0 &&
                        p.lda % 8 == 0 && (BITS == 8 || p.N % 2 == 0);
    if (rows16) {
      const int rows = (BITS == 4) ? p.N / 2 : p.N;
      const unsigned grid = unsigned((rows + 7) / 8);
      if (p.M <= 4) wo_row_warp_kernel<T, BITS, 4><<<grid, 256, 0, st>>>(p);
      else wo_row_warp_kernel<T, BITS, 16><<<grid, 256, 0, st>>>(p);
      return check_cuda(cudaGetLastError(), "weight-only row-per-warp launch");
    }
    const int64_t total = int64_t(p.M) * p.N;
    wo_generic_kernel<T, BITS><<<unsigned((total + 255) / 256), 256, 0, st>>>(p);
    return check_cuda(cudaGetLastError(), "weight-only generic launch");
  }
  const bool perch = p.group == 0;
  (void)workspace;
  (void)workspace_bytes;
  p.status = device_status_word();
  const int nt = p.M <= 8 ? 1 : 2;
  const unsigned grid = unsigned((p.N + 15) / 16);
  const size_t smem_bytes = GemvSmem<BITS>::kBytes;
  // the persistent kernel's FIFO is twice as deep, followed by the per-warp table of activation sums
  const size_t psmem_bytes = 2 * GemvSmem<BITS>::kBytes + size_t(p.K / (spu * kStepK)) * 8 * nt * sizeof(float);
  cudaError_t err;
  // persistent form (int4): whole row groups only, K slices that are whole FIFO blocks; two resident CTAs per SM
  const size_t psmem_cap = 2 * GemvSmem<BITS>::kBytes + 16384;
  const bool persistent = (BITS == 4) && (p.N % 16 == 0) && (p.K % (kStepK * kGemvWarps * kRing) == 0) && psmem_bytes <= psmem_cap;
  const int num_rg = p.N / 16;
  const int resident = 2;
  const unsigned pgrid = unsigned(num_rg < resident * sm_count() ? num_rg : resident * sm_count());
#define FNN_GEMV_CASE(NT, SPU, PC)                                                                          \
  do {                                                                                                      \
    static bool configured[64] = {};                                                                        \
    int dev = 0;                                                                                            \
    cudaGetDevice(&dev);                                                                                    \
    err = cudaSuccess;                                                                                      \
    if (!configured[dev & 63]) {                                                                            \
      err = cudaFuncSetAttribute(gemv_mma_kernel<T, BITS, NT, SPU, PC>,                                     \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes));             \
      if (err == cudaSuccess)                                                                               \
        err = cudaFuncSetAttribute(gemv_mma_persistent_kernel<T, BITS, NT, SPU, PC>,                        \
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, int(psmem_cap));            \
      configured[dev & 63] = (err == cudaSuccess);                                                          \
    }                                                                                                       \
    if (err == cudaSuccess) {                                                                               \
      if (persistent)                                                                                       \
        gemv_mma_persistent_kernel<T, BITS, NT, SPU, PC><<<pgrid, kGemvThreads, psmem_bytes, st>>>(p, num_rg); \
      else                                                                                                  \
        gemv_mma_kernel<T, BITS, NT, SPU, PC><<<grid, kGemvThreads, smem_bytes, st>>>(p);                   \
      err = cudaGetLastError();                                                                             \
    }                                                                                                       \
  } while (0)
#define FNN_GEMV_NT(NT)                                        \
  if (perch) { if (spu == 1) FNN_GEMV_CASE(NT, 1, true); else FNN_GEMV_CASE(NT, 2, true); } \
  else if (spu == 1) FNN_GEMV_CASE(NT, 1, false);              \
  else if (spu == 2) FNN_GEMV_CASE(NT, 2, false);              \
  else FNN_GEMV_CASE(NT, 4, false)
  if (nt == 1) { FNN_GEMV_NT(1); } else { FNN_GEMV_NT(2); }
#undef FNN_GEMV_NT
#undef FNN_GEMV_CASE
  return check_cuda(err, "weight-only gemv launch");
}

}  // namespace
}  // namespace fnn

extern "C" size_t fnn_gemm_weight_only_workspace_bytes(int64_t M, int64_t N, int64_t K, int weight_bits, int64_t group_size) {
  (void)N; (void)weight_bits;
  // prefill kernels (M > 16): row sums of the activations, one per row or one per row and scale group, read when
  // zero-points are given
  if (M > 16 && group_size == 0) return (size_t(M) * sizeof(float) + 255) / 256 * 256;
  if (M > 16 && group_size > 0 && K > 0) return (size_t(M) * size_t((K + group_size - 1) / group_size) * sizeof(float) + 255) / 256 * 256;
  return 0;  // neither the decode kernel nor the generic kernel uses scratch
}

extern "C" int fnn_gemm_weight_only(const void* act, int act_dtype, int64_t lda, const void* qweight, int weight_bits,
                                    const void* scale, const void* zero_points, int scale_dtype, int64_t group_size,
                                    const void* bias, int bias_dtype, void* out, int out_dtype, int64_t ldo, int64_t M,
                                    int64_t N, int64_t K, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace fnn;
  if (M < 0 || N < 0 || K < 0 || lda < K || ldo < N || group_size < 0)
    return fail(FNN_ERR_SHAPE, "gemm_weight_only: M=%lld N=%lld K=%lld lda=%lld ldo=%lld group=%lld", (long long)M, (long long)N,
                (long long)K, (long long)lda, (long long)ldo, (long long)group_size);
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(FNN_ERR_SHAPE, "gemm_weight_only: sizes must be below 2^31");
  if (weight_bits != 4 && weight_bits != 8) return fail(FNN_ERR_UNSUPPORTED, "gemm_weight_only: weight_bits must be 4 or 8 (got %d)", weight_bits);
  if (weight_bits == 4 && (N % 2) != 0) return fail(FNN_ERR_SHAPE, "gemm_weight_only: packed int4 needs an even N (got %lld)", (long long)N);
  if (group_size > 0 && K % group_size != 0) return fail(FNN_ERR_SHAPE, "gemm_weight_only: K=%lld is not a multiple of group_size=%lld", (long long)K, (long long)group_size);
  if (act_dtype != FNN_F16 && act_dtype != FNN_BF16) return fail(FNN_ERR_DTYPE, "gemm_weight_only: activations must be f16 or bf16 (got dtype code %d)", act_dtype);
  if (out_dtype != act_dtype) return fail(FNN_ERR_DTYPE, "gemm_weight_only: output dtype must equal the activation dtype");
  if (scale_dtype < FNN_F16 || scale_dtype > FNN_F32) return fail(FNN_ERR_DTYPE, "gemm_weight_only: bad scale dtype code %d", scale_dtype);
  if (bias && (bias_dtype < FNN_F16 || bias_dtype > FNN_F32)) return fail(FNN_ERR_DTYPE, "gemm_weight_only: bad bias dtype code %d", bias_dtype);
  if (M == 0 || N == 0) return FNN_OK;
  if (!act || !qweight || !scale || !out) return fail(FNN_ERR_NULL_POINTER, "gemm_weight_only: null tensor pointer");
  if (K == 0) return fail(FNN_ERR_SHAPE, "gemm_weight_only: K must be positive");
  WoParams p{};
  p.act = act; p.qw = static_cast<const uint8_t*>(qweight); p.scale = scale; p.zp = zero_points; p.bias = bias;
  p.out = out; p.lda = lda; p.ldo = ldo; p.scale_dtype = scale_dtype; p.bias_dtype = bias_dtype;
  p.M = int(M); p.N = int(N); p.K = int(K); p.group = int(group_size);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M > 16) {
    // prefill shapes: tensor-core kernel (falls through when TMA cannot address the operands or the group size is odd)
    const int r = weight_only_prefill(act, act_dtype, lda, qweight, weight_bits, scale, zero_points, scale_dtype,
                                      int(group_size), bias, bias_dtype, out, ldo, int(M), int(N), int(K), workspace,
                                      workspace_bytes, st);
    if (r >= 0) return r;
  }
  if (act_dtype == FNN_F16)
    return weight_bits == 4 ? launch_wo<__half, 4>(p, workspace, workspace_bytes, st) : launch_wo<__half, 8>(p, workspace, workspace_bytes, st);
  return weight_bits == 4 ? launch_wo<__nv_bfloat16, 4>(p, workspace, workspace_bytes, st) : launch_wo<__nv_bfloat16, 8>(p, workspace, workspace_bytes, st);
}
