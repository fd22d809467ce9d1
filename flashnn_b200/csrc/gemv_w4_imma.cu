// Weight-only GEMV for one to five tokens on the integer tensor pipe: packed int4 weights, and int8 weights, which
// need no expansion at all.
//
// The op is HBM-bound: every weight byte is read once, so what decides the speed is how few instructions a
// warp spends per weight byte.  Expanding a nibble to a 16-bit float costs about one integer-pipe instruction
// per nibble; expanding it to an int8 costs 3 instructions per 8 nibbles:
//     (w << 4) & 0xF0F0F0F0   four low nibbles  -> four int8 holding 16 * n (the sign comes out right)
//      w       & 0xF0F0F0F0   four high nibbles -> four int8 holding 16 * n
// and a 32-bit word of the packed weights (4 consecutive k of channels 2j and 2j+1) becomes two registers of
// the 16 x 32 operand of mma.sync.m16n8k32.s8 as it is.  The activations are 16-bit floats, so they are turned
// into exact fixed point once per CTA: with 2^e the power of two above the row's absmax,
//     X_k = rint(x_k * 2^(22 - e))  (|X| <= 2^22),    X = d2 * 65536 + d1 * 256 + d0,  d in [-128, 127]
// and the three digit planes of a token are three of the eight columns of the MMA's 32 x 8 operand.  A bf16 /
// fp16 value keeps every mantissa bit down to 2^-15 / 2^-12 of the row's absmax and is rounded at 2^-23 of it
// below that, so the products are exact and the int32 accumulator holds exact sums: the only roundings are the
// fp32 scale-and-add per scale group and the final cast, fewer than an fp32 dot product makes.
//     out[m, n] = 2^(e - 22) / 16 * sum_g s[g, n] * (A2 * 65536 + A1 * 256 + A0 - 16 zp[g, n] * (digit sums))
//
// Structure: one persistent CTA per SM; its 16 worker warps own row groups of 16 output channels (8 packed rows)
// and split K.  Every lane streams exactly the 16 bytes per 64-k step that its own fragments need through a
// private cp.async FIFO in shared memory (16 steps deep, refilled four steps at a time with the next work of this
// CTA, so a warp asks for 256 contiguous bytes of each of its 8 rows at once; the group scales ride along), takes
// the matching 16 bytes of a digit plane from registers (K = 8192) or shared memory, and issues two MMAs.  Per
// scale group the int32 accumulators are converted, scaled and added to fp32 totals.  A 17th warp adds up the
// workers' totals of a row group in a fixed order and writes the outputs; the workers hand their totals over
// through a double-buffered array and two pairs of named barriers and never wait for each other.
// A non-finite activation makes the whole output row NaN.
// int8 weights take the same route with 32 bytes per lane and step (16 bytes of each of its two weight rows, which go
// into the MMA operand as they are) and an 8-step FIFO of the same size in bytes.
#include "async_copy.cuh"
#include "common.cuh"
#include "weight_only.cuh"

namespace fnn {
namespace {

constexpr int kImmaWarps = 16;
constexpr int kImmaThreads = kImmaWarps * 32;   // worker threads: they stream the weights and issue the MMAs
constexpr int kImmaCtaThreads = kImmaThreads + 32;  // plus one warp that sums the workers' totals and writes the outputs
constexpr int kImmaStepK = 64;        // k per warp step: 4 lanes x 16 bytes of one packed row
constexpr int kImmaBlk = 4;           // steps per unrolled block of the main loop; the FIFO holds depth / 4 blocks
__host__ __device__ constexpr int imma_slot_bytes(int bits) { return bits == 4 ? 512 : 1024; }  // one step of one warp
__host__ __device__ constexpr int imma_deep(int bits) { return bits == 4 ? 16 : 8; }  // FIFO steps per lane when shared memory allows (else half)
constexpr int kImmaPlanePad = 64;     // plane pitch = K + 64 bytes: the eight planes a warp reads hit distinct banks
constexpr int kImmaMaxTokens = 5;     // 3 planes per token, 16 MMA columns
constexpr int kImmaSmemCap = 226 * 1024;  // dynamic shared memory a CTA may ask for

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
// 128-bit shared load executed only by lanes with `on` set; the others keep what `v` held
__device__ __forceinline__ void lds128_if(uint4& v, uint32_t addr, uint32_t on) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %5, 0;\n\t@p ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n\t}"
               : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w) : "r"(addr), "r"(on));
}
// named CTA barriers over all 544 threads (ids 1..4; __syncthreads owns id 0)
__device__ __forceinline__ void named_barrier_sync(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(544) : "memory"); }
__device__ __forceinline__ void named_barrier_arrive(int id) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "n"(544) : "memory"); }
// d += a (16 x 32 int8, row major) * b (32 x 8 int8, column major)
__device__ __forceinline__ void imma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ float lo16(uint32_t v);
template <typename T> __device__ __forceinline__ float hi16(uint32_t v);
template <> __device__ __forceinline__ float lo16<__nv_bfloat16>(uint32_t v) { return __uint_as_float(v << 16); }
template <> __device__ __forceinline__ float hi16<__nv_bfloat16>(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
template <> __device__ __forceinline__ float lo16<__half>(uint32_t v) { return __low2float(*reinterpret_cast<__half2*>(&v)); }
template <> __device__ __forceinline__ float hi16<__half>(uint32_t v) { return __high2float(*reinterpret_cast<__half2*>(&v)); }

// Shared memory, in this order (byte offsets are multiples of 16):
//   fifo    [16 warps][depth slots][32 lanes][16 B]                     128 KB (depth 16) or 64 KB (depth 8)
//   planes  [3 * M][K + 64] int8
//   red     [2][16 warps][NF][32 lanes][4] fp32   the workers' totals, double buffered
//   fin     [2][16 rows][16 cols] fp32         reduced totals of the row group being written (first half used)
//   sx      [8] fp32                           per token: 2^(e - 22) / 16 (NaN for a non-finite row)
//   xsum    [8] fp32                           per token: sum_k x (per-channel zero-points)
//   sring   [16 warps][8][8] u32 (x2)          group scales (and zero-points) of the blocks in the FIFO: a packed pair
//                                              of channels per lane group, fetched together with the block's weights
//   csum    [K / group][8 * NF] fp32           per scale group and MMA column: sum of the digits (group zero-points)
struct ImmaLayout {
  int planes, red, fin, sx, xsum, sring, csum, total;
};
// bytes per warp of one scale ring: (scale groups held by the FIFO) x 8 words
__host__ __device__ constexpr int imma_sring_warp(int depth, int spu, bool perch) { return perch ? 0 : (depth / spu) * 32; }
// depth: FIFO steps per lane; sring_warp: imma_sring_warp(); zp_groups: K / group when group-wise zero-points are
// given, else 0
__host__ __device__ inline ImmaLayout imma_layout(int bits, int M, int K, int nf, int depth, int sring_warp, int zp_groups,
                                                  int planes_per_token = 3) {
  const int groups = zp_groups;
  ImmaLayout l;
  l.planes = kImmaWarps * depth * imma_slot_bytes(bits);
  l.red = l.planes + planes_per_token * M * (K + kImmaPlanePad);
  l.fin = l.red + 2 * kImmaWarps * nf * 4 * 32 * 4;
  l.sx = l.fin + 2 * 16 * 16 * 4;
  l.xsum = l.sx + 32;
  l.sring = l.xsum + 32;
  l.csum = l.sring + (zp_groups > 0 ? 2 : 1) * kImmaWarps * sring_warp;
  l.total = l.csum + groups * 8 * nf * 4;
  return l;
}

// d = a * b with a zero accumulator input (first MMA of a scale group)
__device__ __forceinline__ void imma0(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}


// NF: MMA column blocks (1: up to 2 tokens, 2: up to 5).  SPU: steps per scale group (1, 2 or 4); with per-channel
// scales (PERCH) the int32 accumulator runs over the warp's whole K slice and is flushed once, with scale 1.
// Host guarantees: K a multiple of 64 * 16 * 4, N a multiple of 16 (so a warp's K slice is whole scale groups).
// GZP: group-wise zero-points are given (per-channel ones are applied when the row group is written).
// DEPTH: steps a lane keeps in flight (16, or 8 when the digit planes leave no room for more).
// One CTA per SM: the 128 registers this allows keep a block of four steps free of reloads.
// XREG: K == 8192, one column block: a lane's digit-plane fragments (8 steps x 16 bytes, the same for every row
// group) stay in registers instead of being re-read from shared memory at every step.
// A8: the activations are int8 already (A8W8 decode): they are copied into the planes as they are, one column per
// token, the int32 sums stay exact all the way to the reducer, which applies the A8W8 scaling rule.
template <typename T, int BITS, int NF, int SPU, bool PERCH, bool GZP, int DEPTH, bool XREG, bool A8 = false>
__global__ void __launch_bounds__(kImmaCtaThreads, 1)
gemv_w4_imma_kernel(const WoParams p, const int num_rg) {
  constexpr int kImmaSlotBytes = imma_slot_bytes(BITS);
  constexpr bool W8 = BITS == 8;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const bool worker = warp < kImmaWarps;  // warp 16 only sums the workers' totals and writes the outputs
  const int K = p.K, M = p.M;
  constexpr bool group_zp = GZP;
  const int groups = PERCH ? 0 : K / (SPU * kImmaStepK);
  constexpr int kImmaSringWarp = imma_sring_warp(DEPTH, SPU, PERCH);
  constexpr int kImmaSringBytes = kImmaWarps * kImmaSringWarp;
  const ImmaLayout L = imma_layout(BITS, M, K, NF, DEPTH, kImmaSringWarp, group_zp ? groups : 0, A8 ? 1 : 3);
  const int pitch = K + kImmaPlanePad;
  constexpr int kRingBlocks = DEPTH / kImmaBlk;
  const int nblk = K / (kImmaStepK * kImmaWarps * kImmaBlk);  // blocks per row group in a warp's K slice
  const int k_begin = warp * nblk * (kImmaBlk * kImmaStepK);

  // Under programmatic stream serialisation this grid may start while the preceding kernel drains: let the next
  // launch do the same, fetch weights (which that kernel does not write), and only then wait for it.  Without
  // that launch attribute both instructions do nothing.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ---- weights: start the FIFO before anything else -------------------------------------------------------------
  // a slot is [32 lanes][16 B]; int8 weights use two such halves (the lane's first and second weight row)
  const uint32_t fifo = smem_u32(smem) + warp * (DEPTH * kImmaSlotBytes) + lane * 16;
  // weight rows of a row group: 8 packed rows (int4) or 16 rows (int8); this lane reads packed row g, or rows 2g and
  // 2g + 1, which are MMA rows g and g + 8 in both cases (channels 2g and 2g + 1 of the group)
  const int64_t rg_stride = int64_t(gridDim.x) * (W8 ? 16 : 8) * K;
  // fill cursor: the next block of this CTA's work to request; it runs kRingBlocks blocks ahead of the consumer
  const uint8_t* wfill = p.qw + (int64_t(blockIdx.x) * (W8 ? 16 : 8) + (W8 ? 2 * g : g)) * K + k_begin + tig * 16;
  auto copy_step = [&](uint32_t slot_addr, const uint8_t* w) {
    cp_async16(slot_addr, w);
    if (W8) cp_async16(slot_addr + 512, w + K);
  };
  int fill_rg = worker ? int(blockIdx.x) : num_rg, fill_blk = 0;  // (the reducer warp never requests anything)
  const int64_t fill_wrap = rg_stride - int64_t(nblk - 1) * (kImmaBlk * kImmaStepK);  // last block -> first of the next row group
  // the block's group scales (zero-points) travel with it: lanes with tig == 0 copy the packed pair of their two channels
  constexpr int kGroupsPerBlk = PERCH ? 1 : kImmaBlk / SPU;
  const int groups_w = PERCH ? 0 : nblk * kGroupsPerBlk;  // scale groups in a warp's K slice
  const int64_t group_pitch = int64_t(p.N) * int64_t(sizeof(T));
  const int64_t sfill_wrap = int64_t(gridDim.x) * 16 * int64_t(sizeof(T)) - int64_t(nblk - 1) * kGroupsPerBlk * group_pitch;
  int64_t sfill = ((int64_t(warp) * groups_w) * p.N + int64_t(blockIdx.x) * 16 + 2 * g) * int64_t(sizeof(T));  // byte offset into scale / zp
  const uint32_t sring = smem_u32(smem) + L.sring + warp * kImmaSringWarp + g * 4;
  auto fill_scales = [&](int ring_blk) {
    if (!PERCH && tig == 0 && fill_rg < num_rg) {
#pragma unroll
      for (int i = 0; i < kGroupsPerBlk; ++i) {
        cp_async4(sring + (ring_blk * kGroupsPerBlk + i) * 32, reinterpret_cast<const uint8_t*>(p.scale) + sfill + i * group_pitch);
        if (GZP) cp_async4(sring + kImmaSringBytes + (ring_blk * kGroupsPerBlk + i) * 32, reinterpret_cast<const uint8_t*>(p.zp) + sfill + i * group_pitch);
      }
    }
  };
  auto advance_fill = [&]() {
    const bool wrap = (++fill_blk == nblk);
    wfill += wrap ? fill_wrap : int64_t(kImmaBlk * kImmaStepK);
    if (!PERCH) sfill += wrap ? sfill_wrap : kGroupsPerBlk * group_pitch;
    fill_rg += wrap ? int(gridDim.x) : 0;
    fill_blk = wrap ? 0 : fill_blk;
  };
#pragma unroll
  for (int b = 0; b < kRingBlocks; ++b) {
    fill_scales(b);
#pragma unroll
    for (int j = 0; j < kImmaBlk; ++j)
      if (fill_rg < num_rg) copy_step(fifo + (b * kImmaBlk + j) * kImmaSlotBytes, wfill + j * kImmaStepK);
    cp_async_commit();  // one group per block, real or empty, keeps the wait count fixed
    advance_fill();
  }

  asm volatile("griddepcontrol.wait;" ::: "memory");  // activations and outputs belong to the stream order

  // ---- activations -> digit planes (once per CTA) ----------------------------------------------------------------
  float* sx = reinterpret_cast<float*>(smem + L.sx);
  float* xsum = reinterpret_cast<float*>(smem + L.xsum);
  float* fin2 = reinterpret_cast<float*>(smem + L.fin);
  if (A8) {
    // int8 activations: row m becomes plane m as it is
    for (int m = 0; m < M; ++m) {
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const int8_t*>(p.act) + int64_t(m) * p.lda);
      uint4* dst = reinterpret_cast<uint4*>(smem + L.planes + m * pitch);
      for (int i = worker ? int(threadIdx.x) : K / 16; i < K / 16; i += kImmaThreads) dst[i] = __ldg(src + i);
    }
    __syncthreads();
  } else {
    float* scratch = fin2;  // [2][16 warps] floats, free until the first row group is written
    constexpr int kHold = 4;  // 16-byte chunks of a row a thread keeps in registers between the two passes
    for (int m = 0; m < M; ++m) {
      const uint4* xr = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.act) + int64_t(m) * p.lda);
      const int nvec = worker ? K / 8 : 0;
      uint4 hold[kHold];
      float amax = 0.f, sum = 0.f;
      auto scan = [&](const uint4& u) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = lo16<T>(w[j]), b = hi16<T>(w[j]);
          // a NaN counts as an infinity, which the maximum keeps: both must reach the check below
          amax = fmaxf(amax, fmaxf(nan_to_inf(fabsf(a)), nan_to_inf(fabsf(b))));
          sum += a + b;
        }
      };
#pragma unroll
      for (int c = 0; c < kHold; ++c) {
        const int i = c * kImmaThreads + threadIdx.x;
        hold[c] = (i < nvec) ? __ldg(xr + i) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int c = 0; c < kHold; ++c) scan(hold[c]);
      for (int i = kHold * kImmaThreads + threadIdx.x; i < nvec; i += kImmaThreads) scan(__ldg(xr + i));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
      }
      if (lane == 0 && worker) { scratch[warp] = amax; scratch[kImmaWarps + warp] = sum; }
      __syncthreads();
      amax = 0.f; sum = 0.f;
      bool bad = false;
#pragma unroll
      for (int w = 0; w < kImmaWarps; ++w) {
        const float a = scratch[w];
        bad |= !(a < __int_as_float(0x7f800000));  // NaN or infinity
        amax = fmaxf(amax, a);
        sum += scratch[kImmaWarps + w];
      }
      __syncthreads();
      // 2^e > amax >= 2^(e-1); shift = 22 - e, kept inside the range of normal fp32 powers of two
      int e = 0;
      if (amax > 0.f) e = int((__float_as_uint(amax) >> 23) & 0xff) - 126;  // subnormal fp32 cannot occur: inputs are 16-bit
      int shift = 22 - e;
      shift = shift > 120 ? 120 : shift;
      const float up = bad ? 0.f : __uint_as_float(uint32_t(127 + shift) << 23);  // 2^shift
      const float down = __uint_as_float(uint32_t(127 - shift - (W8 ? 0 : 4)) << 23);  // 2^-shift (/ 16 for int4, whose int8 form is 16 n)
      if (threadIdx.x == 0) {
        sx[m] = bad ? __int_as_float(0x7fc00000) : down;
        xsum[m] = sum;
      }
      uint8_t* pl = smem + L.planes + (3 * m) * pitch;
      // X + 0x808080 has the plain base-256 digits d + 128; flipping each digit's top bit gives d in two's complement
      auto digits = [&](float xv) -> uint32_t {
        const float t = bad ? 0.f : xv * up;  // (a non-finite value times 0 is NaN)
        return uint32_t(__float2int_rn(t) + 0x808080) ^ 0x808080u;
      };
      auto convert = [&](const uint4& u, int i) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
        uint32_t z[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) { z[2 * j] = digits(lo16<T>(w[j])); z[2 * j + 1] = digits(hi16<T>(w[j])); }
        // byte b of z[0..3] / z[4..7] -> the two words of digit plane b
        uint32_t o[3][2];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int bsel = 0; bsel < 3; ++bsel) {
            const uint32_t pick = 0x0040u + 0x0011u * bsel;  // byte bsel of the first register, byte bsel of the second
            o[bsel][h] = prmt(prmt(z[4 * h], z[4 * h + 1], pick), prmt(z[4 * h + 2], z[4 * h + 3], pick), 0x5410);
          }
        // plane order per token: most significant digit first
        *reinterpret_cast<uint2*>(pl + 0 * pitch + i * 8) = make_uint2(o[2][0], o[2][1]);
        *reinterpret_cast<uint2*>(pl + 1 * pitch + i * 8) = make_uint2(o[1][0], o[1][1]);
        *reinterpret_cast<uint2*>(pl + 2 * pitch + i * 8) = make_uint2(o[0][0], o[0][1]);
      };
#pragma unroll
      for (int c = 0; c < kHold; ++c) {
        const int i = c * kImmaThreads + threadIdx.x;
        if (i < nvec) convert(hold[c], i);
      }
      for (int i = kHold * kImmaThreads + threadIdx.x; i < nvec; i += kImmaThreads) convert(__ldg(xr + i), i);
    }
    __syncthreads();
    // digit sums per scale group and MMA column, for group-wise zero-points
    if (group_zp) {
      float* csum = reinterpret_cast<float*>(smem + L.csum);
      for (int i = worker ? int(threadIdx.x) : groups * 8 * NF; i < groups * 8 * NF; i += kImmaThreads) {
        const int gi = i / (8 * NF), col = i % (8 * NF);
        int s = 0;
        if (col < 3 * M) {
          const int8_t* pl = reinterpret_cast<const int8_t*>(smem + L.planes + col * pitch + gi * (SPU * kImmaStepK));
          for (int k = 0; k < SPU * kImmaStepK; ++k) s += pl[k];
        }
        csum[i] = float(s);
      }
      __syncthreads();
    }
  }

  // ---- reducer warp --------------------------------------------------------------------------------------------
  // Per row group: wait until every worker has stored its totals into this half of `red` (barrier 1 + half), add
  // them up in a fixed order, scale, add the bias, write the outputs, and hand the half back (barrier 3 + half).
  float* red = reinterpret_cast<float*>(smem + L.red);
  if (!worker) {
    float* fin = fin2;
    int half = 0;
    for (int rg = blockIdx.x; rg < num_rg; rg += gridDim.x, half ^= 1) {
      named_barrier_sync(1 + half);
      if (A8) {
        // exact int32 totals; MMA column c is token c
        int* fi = reinterpret_cast<int*>(fin);
#pragma unroll
        for (int f = 0; f < NF; ++f) {
          int4 v = make_int4(0, 0, 0, 0);
#pragma unroll
          for (int w = 0; w < kImmaWarps; ++w) {
            const int4 t = *reinterpret_cast<const int4*>(red + (((half * kImmaWarps + w) * NF + f) * 32 + lane) * 4);
            v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
          }
          *reinterpret_cast<int2*>(fi + g * 16 + 8 * f + 2 * tig) = make_int2(v.x, v.y);
          *reinterpret_cast<int2*>(fi + (g + 8) * 16 + 8 * f + 2 * tig) = make_int2(v.z, v.w);
        }
        if (rg + 2 * int(gridDim.x) < num_rg) named_barrier_arrive(3 + half);
        __syncwarp();
        T* out = reinterpret_cast<T*>(p.out);
        const bool same16 = (p.row_dtype == p.scale_dtype) && (p.row_dtype != FNN_F32);
        for (int idx = lane; idx < 16 * M; idx += 32) {
          const int cl = idx & 15, tok = idx >> 4;
          const int row = (cl & 1) ? (cl >> 1) + 8 : (cl >> 1);
          const int acc = fi[row * 16 + tok];
          const int ch = rg * 16 + cl;
          if (p.acc_out) p.acc_out[int64_t(tok) * p.ldacc + ch] = acc;
          float sc = __fmul_rn(load_as_f32(p.row_scale, p.row_dtype, tok), load_as_f32(p.scale, p.scale_dtype, ch));
          if (same16) sc = round_through(sc, p.row_dtype);
          out[int64_t(tok) * p.ldo + ch] = from_f32<T>(__fmul_rn(float(acc), sc));
        }
        __syncwarp();
      } else {
#pragma unroll
      for (int f = 0; f < NF; ++f) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < kImmaWarps; ++w) {
          const float4 t = *reinterpret_cast<const float4*>(red + (((half * kImmaWarps + w) * NF + f) * 32 + lane) * 4);
          v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
        }
        *reinterpret_cast<float2*>(fin + g * 16 + 8 * f + 2 * tig) = make_float2(v.x, v.y);
        *reinterpret_cast<float2*>(fin + (g + 8) * 16 + 8 * f + 2 * tig) = make_float2(v.z, v.w);
      }
      if (rg + 2 * int(gridDim.x) < num_rg) named_barrier_arrive(3 + half);  // the workers will store into this half again
      __syncwarp();
      T* out = reinterpret_cast<T*>(p.out);
      for (int idx = lane; idx < 16 * M; idx += 32) {
        const int cl = idx & 15, tok = idx >> 4;
        const int row = (cl & 1) ? (cl >> 1) + 8 : (cl >> 1);
        const float* fr = fin + row * 16 + 3 * tok;
        float v = fmaf(fr[0], 65536.f, fmaf(fr[1], 256.f, fr[2])) * sx[tok];
        const int ch = rg * 16 + cl;
        if (PERCH) {
          if (p.zp) v = fmaf(-load_as_f32(p.zp, p.scale_dtype, ch), xsum[tok], v);
          v *= load_as_f32(p.scale, p.scale_dtype, ch);
        }
        if (p.bias) v += load_as_f32(p.bias, p.bias_dtype, ch);
        out[int64_t(tok) * p.ldo + ch] = from_f32<T>(v);
      }
      __syncwarp();
      }
    }
    return;
  }

  // ---- main loop ---------------------------------------------------------------------------------------------------
  const int ncol = A8 ? M : 3 * M;
  // lanes whose MMA column lies past the last digit plane feed zeros and never load
  uint32_t xbase[NF], xon[NF];
#pragma unroll
  for (int f = 0; f < NF; ++f) {
    xon[f] = (8 * f + g) < ncol ? 1u : 0u;
    xbase[f] = smem_u32(smem) + L.planes + min(8 * f + g, ncol - 1) * pitch + k_begin + tig * 16;
  }
  uint4 xv[NF];
#pragma unroll
  for (int f = 0; f < NF; ++f) xv[f] = make_uint4(0, 0, 0, 0);
  constexpr int kXRegBlocks = 2;  // K == 8192: two blocks of four steps per warp and row group
  uint4 xr[NF][XREG ? kXRegBlocks * kImmaBlk : 1];
  if (XREG) {
#pragma unroll
    for (int f = 0; f < NF; ++f)
#pragma unroll
      for (int s2 = 0; s2 < kXRegBlocks * kImmaBlk; ++s2) {
        xr[f][s2] = make_uint4(0, 0, 0, 0);
        lds128_if(xr[f][s2], xbase[f] + s2 * kImmaStepK, xon[f]);
      }
  }
  const float* csum = reinterpret_cast<const float*>(smem + L.csum);
  uint32_t ring = 0;  // which block of the FIFO is being consumed
  int parity = 0, it = 0;

  for (int rg = blockIdx.x; rg < num_rg; rg += gridDim.x) {
    int gi = warp * groups_w;
    float tot[NF][4];
    int acc[NF][4];
#pragma unroll
    for (int f = 0; f < NF; ++f)
#pragma unroll
      for (int i = 0; i < 4; ++i) { tot[f][i] = 0.f; acc[f][i] = 0; }
    uint32_t xa[NF];
#pragma unroll
    for (int f = 0; f < NF; ++f) xa[f] = xbase[f];

#pragma unroll(XREG ? kXRegBlocks : 1)
    for (int blk = 0; blk < (XREG ? kXRegBlocks : nblk); ++blk) {
      const uint32_t slots = fifo + ring * (kImmaBlk * kImmaSlotBytes);
      const bool fill_ok = fill_rg < num_rg;
      uint32_t sc[kGroupsPerBlk], zc[kGroupsPerBlk];
      cp_async_wait<kRingBlocks - 1>();  // the oldest pending block has landed
      if (!PERCH) {
        __syncwarp();  // the words were copied by the tig == 0 lane of each lane group
#pragma unroll
        for (int i = 0; i < kGroupsPerBlk; ++i) {
          sc[i] = lds32(sring + (ring * kGroupsPerBlk + i) * 32);
          if (GZP) zc[i] = lds32(sring + kImmaSringBytes + (ring * kGroupsPerBlk + i) * 32);
        }
      }
#pragma unroll
      for (int j = 0; j < kImmaBlk; ++j) {
#pragma unroll
        for (int f = 0; f < NF; ++f) {
          if (XREG) xv[f] = xr[f][(XREG ? blk : 0) * kImmaBlk + j];
          else lds128_if(xv[f], xa[f] + j * kImmaStepK, xon[f]);
        }
        const uint4 wv = lds128(slots + j * kImmaSlotBytes);
        uint32_t a0, a1, a2, a3, c0, c1, c2, c3;
        if (W8) {  // 16 bytes of row 2g and of row 2g + 1, used as they are
          const uint4 w2 = lds128(slots + j * kImmaSlotBytes + 512);
          a0 = wv.x; a1 = w2.x; a2 = wv.y; a3 = w2.y;
          c0 = wv.z; c1 = w2.z; c2 = wv.w; c3 = w2.w;
        } else {
          a0 = (wv.x << 4) & 0xF0F0F0F0u; a1 = wv.x & 0xF0F0F0F0u;
          a2 = (wv.y << 4) & 0xF0F0F0F0u; a3 = wv.y & 0xF0F0F0F0u;
          c0 = (wv.z << 4) & 0xF0F0F0F0u; c1 = wv.z & 0xF0F0F0F0u;
          c2 = (wv.w << 4) & 0xF0F0F0F0u; c3 = wv.w & 0xF0F0F0F0u;
        }
        const bool first = !PERCH && (j % SPU == 0);  // per-channel scales: the accumulator was zeroed above
#pragma unroll
        for (int f = 0; f < NF; ++f) {
          if (first) imma0(acc[f], a0, a1, a2, a3, xv[f].x, xv[f].y);
          else imma(acc[f], a0, a1, a2, a3, xv[f].x, xv[f].y);
          imma(acc[f], c0, c1, c2, c3, xv[f].z, xv[f].w);
        }
        const bool last = PERCH ? (j == kImmaBlk - 1 && blk == nblk - 1) : ((j + 1) % SPU == 0);
        if (last) {
          float sa = 1.f, sb = 1.f, za = 0.f, zb = 0.f;
          if (!PERCH) {
            sa = lo16<T>(sc[j / SPU]); sb = hi16<T>(sc[j / SPU]);
            if (GZP) { za = (W8 ? 1.f : 16.f) * lo16<T>(zc[j / SPU]); zb = (W8 ? 1.f : 16.f) * hi16<T>(zc[j / SPU]); }
          }
#pragma unroll
          for (int f = 0; f < NF; ++f) {
            if (A8) {  // exact sums: the bits travel to the reducer as they are
              tot[f][0] = __int_as_float(acc[f][0]); tot[f][1] = __int_as_float(acc[f][1]);
              tot[f][2] = __int_as_float(acc[f][2]); tot[f][3] = __int_as_float(acc[f][3]);
              continue;
            }
            float v0 = float(acc[f][0]), v1 = float(acc[f][1]), v2 = float(acc[f][2]), v3 = float(acc[f][3]);
            if (GZP) {
              const float2 cs = *reinterpret_cast<const float2*>(csum + (gi + j / SPU) * (8 * NF) + 8 * f + 2 * tig);
              v0 = fmaf(-za, cs.x, v0); v1 = fmaf(-za, cs.y, v1);
              v2 = fmaf(-zb, cs.x, v2); v3 = fmaf(-zb, cs.y, v3);
            }
            tot[f][0] = fmaf(sa, v0, tot[f][0]); tot[f][1] = fmaf(sa, v1, tot[f][1]);
            tot[f][2] = fmaf(sb, v2, tot[f][2]); tot[f][3] = fmaf(sb, v3, tot[f][3]);
          }
        }
      }
      // Refill the block just consumed with the block that enters the FIFO next, its scales included.  The four
      // copies of a lane are 64 bytes apart, so the warp asks for 256 contiguous bytes of each of its 8 rows at once.
      if (fill_ok) {
#pragma unroll
        for (int j = 0; j < kImmaBlk; ++j) copy_step(slots + j * kImmaSlotBytes, wfill + j * kImmaStepK);
      }
      fill_scales(ring);
      cp_async_commit();
      ring = (ring + 1 == kRingBlocks) ? 0 : ring + 1;
      if (GZP) gi += kGroupsPerBlk;
      advance_fill();
#pragma unroll
      for (int f = 0; f < NF; ++f) xa[f] += kImmaBlk * kImmaStepK;
    }

    // Hand the totals to the reducer warp.  `red` has two halves, so a worker never waits here unless the reducer is
    // two row groups behind: store, arrive on the half's "data" barrier, go on with the next row group.
    if (it >= 2) named_barrier_sync(3 + parity);
#pragma unroll
    for (int f = 0; f < NF; ++f)
      *reinterpret_cast<float4*>(red + (((parity * kImmaWarps + warp) * NF + f) * 32 + lane) * 4) =
          make_float4(tot[f][0], tot[f][1], tot[f][2], tot[f][3]);
    __threadfence_block();
    named_barrier_arrive(1 + parity);
    parity ^= 1;
    ++it;
  }
  cp_async_wait<0>();
}

template <typename T, int BITS, int NF, int SPU, bool PERCH, bool GZP, int DEPTH, bool XREG>
int launch_imma_x(const WoParams& p, size_t smem_bytes, cudaStream_t st) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    const cudaError_t err = cudaFuncSetAttribute(gemv_w4_imma_kernel<T, BITS, NF, SPU, PERCH, GZP, DEPTH, XREG>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, kImmaSmemCap);
    if (err != cudaSuccess) return check_cuda(err, "weight-only decode kernel attribute");
    configured[dev & 63] = true;
  }
  const int num_rg = p.N / 16;
  const int cap = sm_count();  // one CTA per SM
  // fewest CTAs that still reach the smallest possible number of row groups per CTA
  const int rounds = (num_rg + cap - 1) / cap;
  const int grid = (num_rg + rounds - 1) / rounds;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(grid));
  cfg.blockDim = dim3(kImmaCtaThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = opt_static_weights() ? 1 : 0;
  return check_cuda(cudaLaunchKernelEx(&cfg, gemv_w4_imma_kernel<T, BITS, NF, SPU, PERCH, GZP, DEPTH, XREG>, p, num_rg),
                    "weight-only decode (integer tensor pipe) launch");
}

template <typename T, int BITS, int NF, int SPU, bool PERCH, bool GZP, int DEPTH>
int launch_imma(const WoParams& p, size_t smem_bytes, cudaStream_t st) {
  constexpr bool kCanHold = NF == 1 && DEPTH == imma_deep(BITS);
  if (kCanHold && p.K == 8192) return launch_imma_x<T, BITS, NF, SPU, PERCH, GZP, DEPTH, kCanHold>(p, smem_bytes, st);
  return launch_imma_x<T, BITS, NF, SPU, PERCH, GZP, DEPTH, false>(p, smem_bytes, st);
}

template <typename T, int BITS, int NF, int DEPTH>
int launch_imma_spu(const WoParams& p, int spu, size_t smem_bytes, cudaStream_t st) {
  if (p.group == 0) return launch_imma<T, BITS, NF, 4, true, false, DEPTH>(p, smem_bytes, st);
  if (p.zp) {
    if (spu == 1) return launch_imma<T, BITS, NF, 1, false, true, DEPTH>(p, smem_bytes, st);
    if (spu == 2) return launch_imma<T, BITS, NF, 2, false, true, DEPTH>(p, smem_bytes, st);
    return launch_imma<T, BITS, NF, 4, false, true, DEPTH>(p, smem_bytes, st);
  }
  if (spu == 1) return launch_imma<T, BITS, NF, 1, false, false, DEPTH>(p, smem_bytes, st);
  if (spu == 2) return launch_imma<T, BITS, NF, 2, false, false, DEPTH>(p, smem_bytes, st);
  return launch_imma<T, BITS, NF, 4, false, false, DEPTH>(p, smem_bytes, st);
}

template <typename T, int BITS>
int launch_imma_shape(const WoParams& p, int spu, int nf, int depth, size_t smem_bytes, cudaStream_t st) {
  constexpr int kDeep = imma_deep(BITS), kShallow = kDeep / 2;
  if (nf == 1) return depth == kDeep ? launch_imma_spu<T, BITS, 1, kDeep>(p, spu, smem_bytes, st) : launch_imma_spu<T, BITS, 1, kShallow>(p, spu, smem_bytes, st);
  return depth == kDeep ? launch_imma_spu<T, BITS, 2, kDeep>(p, spu, smem_bytes, st) : launch_imma_spu<T, BITS, 2, kShallow>(p, spu, smem_bytes, st);
}

template <typename T, int NF, int DEPTH, bool XREG>
int launch_a8(const WoParams& p, size_t smem_bytes, cudaStream_t st) {
  auto kern = gemv_w4_imma_kernel<T, 8, NF, 4, true, false, DEPTH, XREG, true>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    const cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kImmaSmemCap);
    if (err != cudaSuccess) return check_cuda(err, "a8w8 decode kernel attribute");
    configured[dev & 63] = true;
  }
  const int num_rg = p.N / 16;
  const int cap = sm_count();
  const int rounds = (num_rg + cap - 1) / cap;
  const int grid = (num_rg + rounds - 1) / rounds;
  kern<<<grid, kImmaCtaThreads, smem_bytes, st>>>(p, num_rg);
  return check_cuda(cudaGetLastError(), "a8w8 decode (integer tensor pipe) launch");
}

template <typename T>
int launch_a8_shape(const WoParams& p, int nf, int depth, size_t smem_bytes, cudaStream_t st) {
  if (nf == 1) {
    if (depth == 8) return p.K == 8192 ? launch_a8<T, 1, 8, true>(p, smem_bytes, st) : launch_a8<T, 1, 8, false>(p, smem_bytes, st);
    return launch_a8<T, 1, 4, false>(p, smem_bytes, st);
  }
  return depth == 8 ? launch_a8<T, 2, 8, false>(p, smem_bytes, st) : launch_a8<T, 2, 4, false>(p, smem_bytes, st);
}

}  // namespace

int gemv_a8w8_imma(const int8_t* a, int64_t lda, const int8_t* b, int64_t ldb, const void* alpha_row, int row_dtype,
                   const void* alpha_col, int col_dtype, void* out, int out_dtype, int64_t ldo, int M, int N, int K,
                   int32_t* acc_out, int64_t ldacc, cudaStream_t st) {
  if (M < 1 || M > 16 || N % 16 != 0 || K % (kImmaStepK * kImmaWarps * kImmaBlk) != 0 || ldb != K) return -1;
  if (reinterpret_cast<uintptr_t>(a) % 16 != 0 || lda % 16 != 0 || reinterpret_cast<uintptr_t>(b) % 16 != 0) return -1;
  if (K / kImmaWarps > 65536) return -1;  // |acc| of a warp's K slice stays below 2^31
  WoParams p{};
  p.act = a; p.qw = reinterpret_cast<const uint8_t*>(b); p.scale = alpha_col; p.zp = nullptr; p.bias = nullptr;
  p.out = out; p.lda = lda; p.ldo = ldo; p.scale_dtype = col_dtype; p.bias_dtype = 0;
  p.M = M; p.N = N; p.K = K; p.group = 0; p.status = nullptr;
  p.row_scale = alpha_row; p.row_dtype = row_dtype; p.acc_out = acc_out; p.ldacc = ldacc;
  const int nf = M <= 8 ? 1 : 2;
  int depth = 8;
  ImmaLayout L = imma_layout(8, M, K, nf, depth, 0, 0, 1);
  if (L.total > kImmaSmemCap) {
    depth = 4;
    L = imma_layout(8, M, K, nf, depth, 0, 0, 1);
  }
  if (L.total > kImmaSmemCap) return -1;
  if (out_dtype == FNN_F16) return launch_a8_shape<__half>(p, nf, depth, L.total, st);
  return launch_a8_shape<__nv_bfloat16>(p, nf, depth, L.total, st);
}

int gemv_w4_imma(const WoParams& p, int bits, int act_dtype, cudaStream_t st) {
  if (p.M < 1 || p.M > kImmaMaxTokens) return -1;
  if (p.N % 16 != 0) return -1;
  if (reinterpret_cast<uintptr_t>(p.qw) % 16 != 0) return -1;
  if (reinterpret_cast<uintptr_t>(p.act) % 16 != 0 || p.lda % 8 != 0) return -1;
  const int slice = p.K / kImmaWarps;
  int spu = 0, groups = 0;
  if (p.group > 0) {
    if (p.scale_dtype != act_dtype) return -1;  // group scales (and zero-points) are read as packed pairs of T
    if (reinterpret_cast<uintptr_t>(p.scale) % 4 != 0 || (p.zp && reinterpret_cast<uintptr_t>(p.zp) % 4 != 0)) return -1;
    spu = p.group / kImmaStepK;
    if (p.group % kImmaStepK != 0 || (spu != 1 && spu != 2 && spu != 4)) return -1;
    groups = p.zp ? p.K / p.group : 0;
  } else if (slice > 65536) {
    return -1;  // the int32 accumulator runs over the whole slice: |acc| <= slice * 128 * 128
  }
  if (p.K % (kImmaStepK * kImmaWarps * kImmaBlk) != 0) return -1;
  const int nf = p.M <= 2 ? 1 : 2;
  const int deep = imma_deep(bits);
  int depth = deep;
  ImmaLayout L = imma_layout(bits, p.M, p.K, nf, depth, imma_sring_warp(depth, spu, p.group == 0), groups);
  if (L.total > kImmaSmemCap) {
    depth = deep / 2;
    L = imma_layout(bits, p.M, p.K, nf, depth, imma_sring_warp(depth, spu, p.group == 0), groups);
  }
  if (L.total > kImmaSmemCap) return -1;
  if (bits == 4) {
    if (act_dtype == FNN_F16) return launch_imma_shape<__half, 4>(p, spu, nf, depth, L.total, st);
    return launch_imma_shape<__nv_bfloat16, 4>(p, spu, nf, depth, L.total, st);
  }
  if (act_dtype == FNN_F16) return launch_imma_shape<__half, 8>(p, spu, nf, depth, L.total, st);
  return launch_imma_shape<__nv_bfloat16, 8>(p, spu, nf, depth, L.total, st);
}

}  // namespace fnn
