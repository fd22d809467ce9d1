// Packed-int4 decode GEMV for 6 to 16 tokens with the activations resident on the SM.
//
// For more than a handful of tokens the activations are the larger operand per weight byte: 16 tokens x K = 8192 in
// 16 bits are 256 KB, and a kernel that re-reads its K slice of them for every group of output channels pulls four
// bytes of activations out of L2 for every byte of weights.  Here they are read once per CTA and stay on the SM for
// the whole (persistent) kernel, split between the two places that together can hold them: the first 256 k of every
// warp's K slice as MMA fragments in registers (64 registers per thread), the rest as fragments in shared memory
// (128 KB for K = 8192).  To hold them as fragments the roles of the MMA operands are swapped against the other
// decode kernels: the 16 token rows are the 16 x 16 row operand of mma.sync.m16n8k16, the weights the 16 x 8 column
// operand.  One CTA of 16 warps per SM; the warps split K 16 ways; CTA b walks the groups of 16 output channels
// b, b + grid, ...
//
// Weights: byte (j, k) of the packed matrix carries channel 2j in its low nibble and 2j + 1 in its high nibble
// (flashnn/quant_gemm.py:175-190).  Lane (g, t) of a warp (g = lane / 4, t = lane % 4) streams 16 consecutive bytes
// of packed row 8 rg + g per 64-k chunk through a private cp.async FIFO; each 4-byte word gives the column-operand
// registers of two MMAs, one over the low nibbles (channels 0, 2, .., 14 of the group) and one over the high nibbles
// (channels 1, 3, .., 15), by one LOP3 (two for the high nibbles) and two byte permutes each: the fragment holds
// alpha (n + offset) exactly (bf16: n + 136; fp16: 16 (n + 72)) and the constant part leaves per scale group as
// -(offset + zp) s sum_k x, with sum_k x per token and group formed once at the start.  The k order inside a 16-k
// step is permuted the same way on both operands (a lane's four consecutive bytes are k columns 2t, 2t+1, 2t+8,
// 2t+9 of the MMA), which turns every operand fetch into a 16-byte access.  fp32 accumulators per scale group, scale
// applied in fp32, so w * s is never rounded to 16 bits.  Per channel group the 16 warps' partial sums meet in shared
// memory behind one barrier (double-buffered), 256 threads add them in a fixed order, add the bias and round once.
#include <mutex>
#include <type_traits>

#include "async_copy.cuh"
#include "common.cuh"
#include "weight_only.cuh"

namespace fnn {
namespace {

constexpr int kTkWarps = 16;
constexpr int kTkThreads = kTkWarps * 32;
constexpr int kTkSlots = 7;       // FIFO depth per lane, in 64-k chunks
constexpr int kTkRegChunks = 4;   // chunks of a warp's slice whose activation fragments live in registers

__device__ __forceinline__ void cp_async8(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
template <typename T> __device__ __forceinline__ float lo_half(uint32_t w);
template <typename T> __device__ __forceinline__ float hi_half(uint32_t w);
template <> __device__ __forceinline__ float lo_half<__nv_bfloat16>(uint32_t w) { return __uint_as_float(w << 16); }
template <> __device__ __forceinline__ float hi_half<__nv_bfloat16>(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
template <> __device__ __forceinline__ float lo_half<__half>(uint32_t w) { return __low2float(*reinterpret_cast<const __half2*>(&w)); }
template <> __device__ __forceinline__ float hi_half<__half>(uint32_t w) { return __high2float(*reinterpret_cast<const __half2*>(&w)); }

__device__ __forceinline__ uint32_t tk_and_xor(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t tk_prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
template <typename T> struct TkFrag;
template <> struct TkFrag<__nv_bfloat16> {
  static constexpr float kInvAlpha = 1.f, kOffset = 136.f;  // byte (n ^ 8) under 0x43: 128 + (n ^ 8) = n + 136
  static __device__ __forceinline__ void make(uint32_t w, uint32_t (&lo)[2], uint32_t (&hi)[2]) {
    const uint32_t l = tk_and_xor(w, 0x0F0F0F0Fu, 0x08080808u);
    const uint32_t h = tk_and_xor(w >> 4, 0x0F0F0F0Fu, 0x08080808u);
    lo[0] = tk_prmt(l, 0x43434343u, 0x4140); lo[1] = tk_prmt(l, 0x43434343u, 0x4342);
    hi[0] = tk_prmt(h, 0x43434343u, 0x4140); hi[1] = tk_prmt(h, 0x43434343u, 0x4342);
  }
  static __device__ __forceinline__ void mma(float (&d)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
  }
  // d = a * b: the first MMA of a fold starts a fresh accumulator without clearing registers
  static __device__ __forceinline__ void mma0(float (&d)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1), "f"(0.f));
  }
};
template <> struct TkFrag<__half> {
  static constexpr float kInvAlpha = 0.0625f, kOffset = 72.f;  // byte ((n ^ 8) << 4) under 0x64: 1024 + 16 (n ^ 8)
  static __device__ __forceinline__ void make(uint32_t w, uint32_t (&lo)[2], uint32_t (&hi)[2]) {
    const uint32_t l = tk_and_xor(w << 4, 0xF0F0F0F0u, 0x80808080u);
    const uint32_t h = tk_and_xor(w, 0xF0F0F0F0u, 0x80808080u);
    lo[0] = tk_prmt(l, 0x64646464u, 0x4140); lo[1] = tk_prmt(l, 0x64646464u, 0x4342);
    hi[0] = tk_prmt(h, 0x64646464u, 0x4140); hi[1] = tk_prmt(h, 0x64646464u, 0x4342);
  }
  static __device__ __forceinline__ void mma(float (&d)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ void mma0(float (&d)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1), "f"(0.f));
  }
};

// CHUNKS: 64-k chunks per warp slice (4: K = 4096, 8: K = 8192).  CPF: chunks per fold, the span over which an fp32
// accumulator collects alpha (n + offset) x before the constant part is taken out (1 or 2: at most 128 k, which keeps the
// cancellation against the offset small).  FPG: folds per scale group (1, 2, or all folds of the slice for per-channel
// scales, which run with a unit scale here; the channel's scale is applied by the reducing threads).
template <typename T, int CHUNKS, int CPF, int FPG, bool PERCH>
__global__ void __launch_bounds__(kTkThreads, 1) gemv_w4_tok_kernel(const WoParams p, const int num_rg) {
  constexpr int SMEM_CHUNKS = CHUNKS > kTkRegChunks ? CHUNKS - kTkRegChunks : 0;
  constexpr int REG_CHUNKS = CHUNKS - SMEM_CHUNKS;
  constexpr int FOLDS = CHUNKS / CPF;
  constexpr int NSG = FOLDS / FPG;  // scale groups per warp slice (1 for per-channel scales)
  static_assert(NSG >= 1 && NSG <= 4, "the scale ring holds at most four groups per slice");
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* a_smem = smem;                                                        // [warp][SMEM_CHUNKS][4 steps][32 lanes] uint4
  uint8_t* fifo_base = a_smem + kTkWarps * SMEM_CHUNKS * 4 * 512;                // [warp][kTkSlots][32 lanes] uint4
  uint8_t* ring_base = fifo_base + kTkWarps * kTkSlots * 512;                    // [warp][2][scale, zp][4 groups][4 t] 8 bytes
  float* red = reinterpret_cast<float*>(ring_base + kTkWarps * 2 * 256);         // [2][warp][16 tokens][16 channels]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  constexpr int slice = CHUNKS * 64;
  const int k_warp = warp * slice;
  const bool has_zp = p.zp != nullptr;

  // ---- weight FIFO: lane (g, t) streams bytes [k_warp + 64 c + 16 t, + 16) of packed row 8 rg + g ----
  const uint32_t fifo = smem_u32(fifo_base) + (warp * kTkSlots) * 512 + lane * 16;
  const uint8_t* wlane = p.qw + int64_t(g) * p.K + k_warp + t * 16;
  const int64_t rg_bytes = int64_t(8) * p.K;
  // chunk `v` counted from the first chunk of row group `rg_from` on (runs into this CTA's later row groups)
  auto chunk_ptr = [&](int rg_from, int v) -> const uint8_t* {
    const int rgv = rg_from + (v / CHUNKS) * int(gridDim.x);
    return rgv < num_rg ? wlane + int64_t(rgv) * rg_bytes + (v % CHUNKS) * 64 : nullptr;
  };
  // ---- scale ring: the 4 x 16-bit scales (and zero-points) of channels 4 tt .. 4 tt + 3 for every scale group of
  // this warp's slice, one row group ahead; lane i < 4 NSG copies group i / 4, tt = i % 4 (lanes 16 .. copy the zero-points)
  const uint32_t ring = smem_u32(ring_base) + warp * 512;
  auto issue_scales = [&](int rgv, int slot) {
    if (rgv >= num_rg) return;
    const int i = lane & 15;
    if (i < 4 * NSG) {
      const int64_t at = (PERCH ? int64_t(0) : int64_t(warp * NSG + (i >> 2)) * p.N) + rgv * 16 + 4 * (i & 3);
      if (lane < 16) {
        if (!PERCH) cp_async8(ring + slot * 256 + i * 8, reinterpret_cast<const T*>(p.scale) + at);
      } else if (has_zp) {
        cp_async8(ring + slot * 256 + 128 + i * 8, reinterpret_cast<const T*>(p.zp) + at);
      }
    }
  };
  int rg = blockIdx.x;
  issue_scales(rg, 0);
#pragma unroll
  for (int v = 0; v < kTkSlots; ++v) {
    const uint8_t* w = chunk_ptr(rg, v);
    if (w) cp_async16(fifo + v * 512, w);
    cp_async_commit();
  }
  // the chunk that goes into the slot consumed next: kTkSlots chunks ahead, as a running (row group, chunk, pointer)
  int fill_rg = rg + (kTkSlots / CHUNKS) * int(gridDim.x), fill_c = kTkSlots % CHUNKS;
  const uint8_t* fill_ptr = wlane + int64_t(fill_rg) * rg_bytes + fill_c * 64;
  const int64_t rg_jump = int64_t(gridDim.x) * rg_bytes - (CHUNKS - 1) * 64;  // from the last chunk of a row group to the next one's first

  // ---- activations: this warp's slice of the 16 token rows, as A fragments (rows g and g + 8 of this lane) ----
  const T* act = reinterpret_cast<const T*>(p.act);
  uint4 areg[REG_CHUNKS * 4];
  float xsum[FOLDS][2];
#pragma unroll
  for (int f = 0; f < FOLDS; ++f) xsum[f][0] = xsum[f][1] = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    // the lane's 16 k of chunk c: k_warp + 64 c + 16 t .. + 15, four steps of four
    uint4 lo[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)}, hi[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    if (g < p.M) {
      const uint4* src = reinterpret_cast<const uint4*>(act + int64_t(g) * p.lda + k_warp + c * 64 + t * 16);
      lo[0] = __ldg(src);
      lo[1] = __ldg(src + 1);
    }
    if (g + 8 < p.M) {
      const uint4* src = reinterpret_cast<const uint4*>(act + int64_t(g + 8) * p.lda + k_warp + c * 64 + t * 16);
      hi[0] = __ldg(src);
      hi[1] = __ldg(src + 1);
    }
    const uint32_t lw[8] = {lo[0].x, lo[0].y, lo[0].z, lo[0].w, lo[1].x, lo[1].y, lo[1].z, lo[1].w};
    const uint32_t hw[8] = {hi[0].x, hi[0].y, hi[0].z, hi[0].w, hi[1].x, hi[1].y, hi[1].z, hi[1].w};
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      // step s: k columns (2t, 2t+1) = words 2s, (2t+8, 2t+9) = words 2s+1, of row g (a0, a2) and row g + 8 (a1, a3)
      const uint4 frag = make_uint4(lw[2 * s], hw[2 * s], lw[2 * s + 1], hw[2 * s + 1]);
      if (c < REG_CHUNKS) areg[c * 4 + s] = frag;
      else *reinterpret_cast<uint4*>(a_smem + ((warp * SMEM_CHUNKS + (c - REG_CHUNKS)) * 4 + s) * 512 + lane * 16) = frag;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const T* pl = reinterpret_cast<const T*>(&lw[i]);
      const T* ph = reinterpret_cast<const T*>(&hw[i]);
      s0 += to_f32(pl[0]) + to_f32(pl[1]);
      s1 += to_f32(ph[0]) + to_f32(ph[1]);
    }
    xsum[c / CPF][0] += s0;
    xsum[c / CPF][1] += s1;
  }
  // sum over the four lanes of a row: every lane then holds sum_k x of tokens g and g + 8 for each of its folds
#pragma unroll
  for (int f = 0; f < FOLDS; ++f) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      xsum[f][h] += __shfl_xor_sync(0xffffffffu, xsum[f][h], 1);
      xsum[f][h] += __shfl_xor_sync(0xffffffffu, xsum[f][h], 2);
    }
  }
  __syncwarp();

  constexpr float kInvAlpha = TkFrag<T>::kInvAlpha, kOffset = TkFrag<T>::kOffset;
  const uint32_t a_lane = smem_u32(a_smem) + warp * SMEM_CHUNKS * 4 * 512 + lane * 16;
  int parity = 0;
  int slot = 0;   // FIFO slot of the next chunk to consume
  int sslot = 0;  // scale-ring slot of the current row group
  for (; rg < num_rg; rg += gridDim.x) {
    issue_scales(rg + int(gridDim.x), sslot ^ 1);  // rides the commit of this row group's first chunk
    float tot[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) tot[i] = 0.f;
    float accl[4], acch[4];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      // chunk c has landed.  The scales of this row group were committed one row group (CHUNKS commits) ago; where
      // that is fewer than the FIFO is deep, the first wait of the row group has to reach back to them explicitly
      if (CHUNKS < kTkSlots && c == 0) cp_async_wait<CHUNKS - 1>();
      else cp_async_wait<kTkSlots - 1>();
      const uint4 wv = lds128(fifo + slot * 512);
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        uint32_t bl[2], bh[2];
        TkFrag<T>::make(ww[s], bl, bh);
        uint4 a;
        if (c < REG_CHUNKS) a = areg[c * 4 + s];
        else a = lds128(a_lane + ((c - REG_CHUNKS) * 4 + s) * 512);
        if (c % CPF == 0 && s == 0) {
          TkFrag<T>::mma0(accl, a, bl[0], bl[1]);
          TkFrag<T>::mma0(acch, a, bh[0], bh[1]);
        } else {
          TkFrag<T>::mma(accl, a, bl[0], bl[1]);
          TkFrag<T>::mma(acch, a, bh[0], bh[1]);
        }
      }
      {  // refill this slot with the chunk kTkSlots ahead
        if (fill_rg < num_rg) cp_async16(fifo + slot * 512, fill_ptr);
        cp_async_commit();
        slot = slot + 1 == kTkSlots ? 0 : slot + 1;
        if (++fill_c == CHUNKS) { fill_c = 0; fill_rg += int(gridDim.x); fill_ptr += rg_jump; }
        else fill_ptr += 64;
      }
      if ((c + 1) % CPF == 0) {
        // end of a fold: total += s * (acc / alpha - (offset + zp) * sum_k x), channels 4t .. 4t + 3
        constexpr float kZ0 = kOffset / kInvAlpha;
        const int fold = c / CPF;
        float sc[4] = {kInvAlpha, kInvAlpha, kInvAlpha, kInvAlpha};
        float zo[4] = {kZ0, kZ0, kZ0, kZ0};
        const uint32_t at = ring + sslot * 256 + ((fold / FPG) * 4 + t) * 8;
        if (!PERCH) {
          uint32_t s01, s23;
          asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(s01), "=r"(s23) : "r"(at));
          sc[0] *= lo_half<T>(s01); sc[1] *= hi_half<T>(s01); sc[2] *= lo_half<T>(s23); sc[3] *= hi_half<T>(s23);
        }
        if (has_zp) {
          uint32_t z01, z23;
          asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(z01), "=r"(z23) : "r"(at + 128));
          zo[0] += lo_half<T>(z01) / kInvAlpha; zo[1] += hi_half<T>(z01) / kInvAlpha;
          zo[2] += lo_half<T>(z23) / kInvAlpha; zo[3] += hi_half<T>(z23) / kInvAlpha;
        }
        const float x0 = xsum[fold][0], x1 = xsum[fold][1];
        // accl: (row g: cols 2t, 2t+1 -> channels 4t, 4t+2), (row g+8: same); acch: channels 4t+1, 4t+3
        tot[0] = fmaf(sc[0], fmaf(-zo[0], x0, accl[0]), tot[0]);
        tot[1] = fmaf(sc[1], fmaf(-zo[1], x0, acch[0]), tot[1]);
        tot[2] = fmaf(sc[2], fmaf(-zo[2], x0, accl[1]), tot[2]);
        tot[3] = fmaf(sc[3], fmaf(-zo[3], x0, acch[1]), tot[3]);
        tot[4] = fmaf(sc[0], fmaf(-zo[0], x1, accl[2]), tot[4]);
        tot[5] = fmaf(sc[1], fmaf(-zo[1], x1, acch[2]), tot[5]);
        tot[6] = fmaf(sc[2], fmaf(-zo[2], x1, accl[3]), tot[6]);
        tot[7] = fmaf(sc[3], fmaf(-zo[3], x1, acch[3]), tot[7]);
      }
    }
    sslot ^= 1;
    // partial sums of this warp: token g -> channels 4t .. 4t+3, token g + 8 likewise
    float* mine = red + (parity * kTkWarps + warp) * 256;
    *reinterpret_cast<float4*>(mine + g * 16 + 4 * t) = make_float4(tot[0], tot[1], tot[2], tot[3]);
    *reinterpret_cast<float4*>(mine + (g + 8) * 16 + 4 * t) = make_float4(tot[4], tot[5], tot[6], tot[7]);
    // what the reducing threads need from global memory is requested before the barrier
    const int token = threadIdx.x >> 4, ch = rg * 16 + (threadIdx.x & 15);
    float ch_scale = 1.f, ch_bias = 0.f;
    if (threadIdx.x < 256) {
      if (PERCH) ch_scale = load_as_f32(p.scale, p.scale_dtype, ch);
      if (p.bias) ch_bias = load_as_f32(p.bias, p.bias_dtype, ch);
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kTkWarps; ++w) v += red[(parity * kTkWarps + w) * 256 + threadIdx.x];
      if (token < p.M) reinterpret_cast<T*>(p.out)[int64_t(token) * p.ldo + ch] = from_f32<T>(fmaf(v, ch_scale, ch_bias));
    }
    parity ^= 1;
  }
  cp_async_wait<0>();
}

template <typename T, int CHUNKS, int CPF, int FPG, bool PERCH>
int launch_tok(const WoParams& p, cudaStream_t st) {
  constexpr int SMEM_CHUNKS = CHUNKS > kTkRegChunks ? CHUNKS - kTkRegChunks : 0;
  constexpr int kBytes = kTkWarps * SMEM_CHUNKS * 4 * 512 + kTkWarps * kTkSlots * 512 + kTkWarps * 2 * 256 + 2 * kTkWarps * 256 * 4;
  static_assert(kBytes <= 227 * 1024, "shared memory budget");
  auto kern = gemv_w4_tok_kernel<T, CHUNKS, CPF, FPG, PERCH>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::call_once(once[dev], [&] { attr_err[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes); });
  if (attr_err[dev] != cudaSuccess) return check_cuda(attr_err[dev], "cudaFuncSetAttribute(int4 decode, resident activations)");
  const int num_rg = p.N / 16;
  const int grid = num_rg < sm_count() ? num_rg : sm_count();
  kern<<<grid, kTkThreads, kBytes, st>>>(p, num_rg);
  return check_cuda(cudaGetLastError(), "int4 decode (resident activations) launch");
}

template <typename T, int CHUNKS>
int dispatch_tok(const WoParams& p, cudaStream_t st) {
  constexpr int slice = CHUNKS * 64;
  if (p.group == 0) return launch_tok<T, CHUNKS, 2, CHUNKS / 2, true>(p, st);  // folds of 128 k, one (unit) scale
  if (slice % p.group != 0 || slice / p.group > 4) return -1;
  switch (p.group) {
    case 64:
      if constexpr (CHUNKS <= 4) return launch_tok<T, CHUNKS, 1, 1, false>(p, st);
      else return -1;
    case 128: return launch_tok<T, CHUNKS, 2, 1, false>(p, st);
    case 256: return launch_tok<T, CHUNKS, 2, 2, false>(p, st);
    default: return -1;
  }
}

}  // namespace

// Packed-int4 decode for 6 to 16 tokens with the activations resident on the SM (this file).  Returns an
// fnn_status, or -1 when the shape or alignment is outside what the kernel handles: K must be 4096 or 8192,
// N a multiple of 16, the group size 64 (K = 4096 only), 128 or 256 (or per-channel scales), operands 16-byte aligned,
// group scales and zero-points in the activation dtype.
int gemv_w4_tok(const WoParams& p, int act_dtype, cudaStream_t st) {
  if (p.M < 1 || p.M > 16 || p.N % 16 != 0 || p.N < 16) return -1;
  if (p.K != 4096 && p.K != 8192) return -1;
  if (p.group != 0 && p.group != 64 && p.group != 128 && p.group != 256) return -1;
  if (reinterpret_cast<uintptr_t>(p.qw) % 16 != 0 || reinterpret_cast<uintptr_t>(p.act) % 16 != 0 || p.lda % 8 != 0) return -1;
  // group scales and zero-points are copied 8 bytes (four 16-bit values) at a time
  if ((p.group != 0 || p.zp) && (p.scale_dtype != act_dtype || reinterpret_cast<uintptr_t>(p.scale) % 8 != 0 ||
                                 (p.zp && reinterpret_cast<uintptr_t>(p.zp) % 8 != 0)))
    return -1;
  if (act_dtype == FNN_F16) return p.K == 8192 ? dispatch_tok<__half, 8>(p, st) : dispatch_tok<__half, 4>(p, st);
  return p.K == 8192 ? dispatch_tok<__nv_bfloat16, 8>(p, st) : dispatch_tok<__nv_bfloat16, 4>(p, st);
}

}  // namespace fnn
