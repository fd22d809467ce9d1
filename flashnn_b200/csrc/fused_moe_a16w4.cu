// Fused mixture-of-experts weight-only GEMM: fp16/bf16 tokens x the packed-int4 weights of the expert each block of
// expert-sorted slots belongs to (replaces fused_moe_a16w4_forward, flashnn/triton_kernels/fused_moe_a16w4.py:326-466;
// per-channel kernel :50-183, sub-channel kernel :186-323).
//
// One CTA (8 warps) computes a tile of TOK sorted slots (one expert) x 128 output channels.  The token rows named by
// the slots are gathered straight into shared memory (cp.async, 16 bytes per copy; slots that name no token are
// zero-filled), next to the raw packed weight bytes of the tile's 64 packed rows, through a four-stage ring of
// 128-k blocks.  Warp w owns packed rows 8w .. 8w+7, i.e. 16 channels: byte (j, k) carries channel 2j in its low
// nibble and 2j+1 in its high nibble (fused_moe_a16w4.py:137,151), which is exactly the row pair (r, r + 8) one lane of
// an m16n8k16 A fragment holds, so a lane expands 4 consecutive bytes of one packed row into its four A registers
// (exact integers in T, LOP3/PRMT only) and the k order inside a 16-k step is permuted the same way on the token
// side.  Tokens are the MMA's 8-column operand (TOK / 8 column blocks per weight fragment), accumulators fp32.
//
// Scales are applied in fp32 and w * s is never rounded to 16 bits: per channel after the K loop, per K group by
// folding the group's accumulator into a running total, total += s[e, n, g] * (acc_g - zp[e, n, g] * xsum_g), where
// xsum_g (the sum of the group's activations per token) comes from one more MMA against an all-ones A fragment, which
// leaves it in the accumulator layout.  The reference's sub-channel kernel rounds (w - zp) * s to 16 bits per weight
// (:289-303); as for GemmWeightOnly, this kernel is held to the fp32 dequant-matmul instead.  The epilogue multiplies
// by the routing weight in fp32, rounds once and scatters each slot's row to its flat (token, choice) index.
#include <mutex>
#include <type_traits>

#include "async_copy.cuh"
#include "common.cuh"
#include "weight_only.cuh"

namespace fnn {
namespace {

constexpr int kMwThreads = 256;
constexpr int kMwChannels = 128;  // output channels per tile (64 packed rows)
constexpr int kMwKC = 128;        // k per stage
constexpr int kMwStages = 4;
constexpr int kMwXPitch = kMwKC * 2 + 16;  // bytes between two token rows of a stage (the odd 16 spreads them over banks)
constexpr int kMwWBytes = (kMwChannels / 2) * kMwKC;  // raw weight bytes of a stage

struct MoeW4Params {
  const void* a;
  int64_t lda;
  const uint8_t* b;     // [E, N/2, K] packed
  const void* scale;    // [E, N] or [E, N, K/group]
  const void* zp;       // nullptr or like scale
  const void* topk_w;   // [num_valid]
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* npp;
  void* out;
  int64_t ldo;
  int scale_dtype, topk_dtype;
  int N, K, EM, num_valid, top_k, block_m, tile_rows, tiles_per_block, mul_w, group, groups;
};

template <int TOK> struct MwSmem {
  static constexpr int kXBytes = TOK * kMwXPitch;
  static constexpr int kStageBytes = kXBytes + kMwWBytes;
  static constexpr int kRowOff = kMwStages * kStageBytes;  // int64 source offset (elements) per tile row, -1 = no token
  static constexpr int kBytes = kRowOff + TOK * 8;
};

__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gmem_src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes) : "memory");
}

__device__ __forceinline__ uint32_t mw_prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
template <typename T> struct MwNib;
template <> struct MwNib<__half> { static constexpr uint32_t magic = 0x64646464u, off = 0x64086408u, one2 = 0x3C003C00u; };          // 1024 + u; 1032
template <> struct MwNib<__nv_bfloat16> { static constexpr uint32_t magic = 0x43434343u, off = 0x43084308u, one2 = 0x3F803F80u; };  // 128 + u; 136
__device__ __forceinline__ uint32_t mw_sub2(uint32_t a, uint32_t b, __half) {
  __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t mw_sub2(uint32_t a, uint32_t b, __nv_bfloat16) {
  __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
// four packed bytes -> the A fragment of one 16-k step: a0 / a2 = low nibbles (row r) of bytes 0,1 / 2,3,
// a1 / a3 = high nibbles (row r + 8), as exact signed integers in T
template <typename T> __device__ __forceinline__ void mw_expand(uint32_t w, uint32_t (&a)[4]) {
  const uint32_t lo = (w & 0x0F0F0F0Fu) ^ 0x08080808u;
  const uint32_t hi = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
  a[0] = mw_sub2(mw_prmt(lo, MwNib<T>::magic, 0x4140), MwNib<T>::off, T());
  a[2] = mw_sub2(mw_prmt(lo, MwNib<T>::magic, 0x4342), MwNib<T>::off, T());
  a[1] = mw_sub2(mw_prmt(hi, MwNib<T>::magic, 0x4140), MwNib<T>::off, T());
  a[3] = mw_sub2(mw_prmt(hi, MwNib<T>::magic, 0x4342), MwNib<T>::off, T());
}

__device__ __forceinline__ void mw_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, __half) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mw_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, __nv_bfloat16) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// TOK: slots per tile (16, 32 or 64).  GRP: scales per K group ([E, N, K/group]) instead of per channel ([E, N]).
template <typename T, int TOK, bool GRP, bool HAS_ZP>
__global__ void __launch_bounds__(kMwThreads) moe_w4_kernel(const MoeW4Params p) {
  using L = MwSmem<TOK>;
  constexpr int NB = TOK / 8;
  extern __shared__ __align__(16) uint8_t mw_smem[];
  int64_t* row_src = reinterpret_cast<int64_t*>(mw_smem + L::kRowOff);

  // tile of this CTA: grouped ordering (8 slot tiles share a wave of channel tiles) so that the tiles of one expert
  // that run at the same time read the same weights
  const int tiles_n = (p.N + kMwChannels - 1) / kMwChannels;
  const int tiles_m = (p.EM / p.block_m) * p.tiles_per_block;
  constexpr int kGroupM = 8;
  const int pid = blockIdx.x;
  const int in_group = kGroupM * tiles_n;
  const int first_m = (pid / in_group) * kGroupM;
  const int gm = min(tiles_m - first_m, kGroupM);
  const int tm = first_m + (pid % in_group) % gm;
  const int tn = (pid % in_group) / gm;
  const int blk = tm / p.tiles_per_block;
  const int slot0 = blk * p.block_m + (tm % p.tiles_per_block) * p.tile_rows;
  if (slot0 >= __ldg(p.npp)) return;
  const int rows_valid = min(p.tile_rows, p.block_m - (tm % p.tiles_per_block) * p.tile_rows);
  const int expert = __ldg(p.expert_ids + blk);
  const int ch0 = tn * kMwChannels;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int j = lane >> 2, q = lane & 3;

  if (tid < TOK) {
    int64_t src = -1;
    if (tid < rows_valid) {
      const int flat = __ldg(p.sorted_ids + slot0 + tid);
      if (flat >= 0 && flat < p.num_valid) src = int64_t(flat / p.top_k) * p.lda;
    }
    row_src[tid] = src;
  }
  __syncthreads();

  const T* a = reinterpret_cast<const T*>(p.a);
  const uint8_t* wbase = p.b + (int64_t(expert) * (p.N / 2) + ch0 / 2) * int64_t(p.K);
  const int prow_valid = min(kMwChannels / 2, (p.N - ch0) / 2);  // packed rows of this tile that exist
  const int k_stages = (p.K + kMwKC - 1) / kMwKC;

  auto load_stage = [&](int ks, int slot) {
    uint8_t* sx = mw_smem + slot * L::kStageBytes;
    uint8_t* sw = sx + L::kXBytes;
    const int k0 = ks * kMwKC;
    // activations: TOK rows x 16 chunks of 8 elements
    for (int i = tid; i < TOK * 16; i += kMwThreads) {
      const int r = i >> 4, c = i & 15;
      const int64_t src = row_src[r];
      const bool ok = src >= 0 && k0 + c * 8 < p.K;
      cp_async16_zfill(sx + r * kMwXPitch + c * 16, ok ? static_cast<const void*>(a + src + k0 + c * 8) : p.a, ok);
    }
    // weights: 64 packed rows x 8 chunks of 16 bytes; chunk c of row r is stored at chunk c ^ (4 * (r & 1)), which
    // keeps the 16-byte reads of two adjacent rows on different banks
    for (int i = tid; i < (kMwChannels / 2) * 8; i += kMwThreads) {
      const int r = i >> 3, c = i & 7;
      const bool ok = r < prow_valid && k0 + c * 16 < p.K;
      cp_async16_zfill(sw + r * kMwKC + ((c ^ ((r & 1) << 2)) << 4), ok ? static_cast<const void*>(wbase + int64_t(r) * p.K + k0 + c * 16) : p.b, ok);
    }
  };

  float acc[NB][4];      // per-channel: the whole sum; per group: the group in flight
  float total[NB][4];    // per group only: the running total
  float ones[NB][4];     // with zero-points only: sum of the activations per token (same span as acc)
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nb][i] = total[nb][i] = ones[nb][i] = 0.f;

  // scale / zero-point of this lane's two channels (2j: accumulator rows r, 2j + 1: rows r + 8)
  const int ch_even = ch0 + warp * 16 + 2 * j;
  const bool ch_in = ch_even < p.N;  // N is even: the pair is in or out together
  const int64_t sidx = (int64_t(expert) * p.N + ch_even) * (GRP ? p.groups : 1);
  const int64_t sidx_odd = sidx + (GRP ? p.groups : 1);
  auto fold = [&](int g) {
    // total += s * (acc - zp * xsum) for the group that just ended
    const float s0 = ch_in ? load_as_f32(p.scale, p.scale_dtype, sidx + g) : 0.f;
    const float s1 = ch_in ? load_as_f32(p.scale, p.scale_dtype, sidx_odd + g) : 0.f;
    float z0 = 0.f, z1 = 0.f;
    if (HAS_ZP && ch_in) {
      z0 = load_as_f32(p.zp, p.scale_dtype, sidx + g);
      z1 = load_as_f32(p.zp, p.scale_dtype, sidx_odd + g);
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float v0 = acc[nb][0], v1 = acc[nb][1], v2 = acc[nb][2], v3 = acc[nb][3];
      if (HAS_ZP) {
        v0 = fmaf(-z0, ones[nb][0], v0); v1 = fmaf(-z0, ones[nb][1], v1);
        v2 = fmaf(-z1, ones[nb][2], v2); v3 = fmaf(-z1, ones[nb][3], v3);
      }
      if (GRP) {
        total[nb][0] = fmaf(s0, v0, total[nb][0]); total[nb][1] = fmaf(s0, v1, total[nb][1]);
        total[nb][2] = fmaf(s1, v2, total[nb][2]); total[nb][3] = fmaf(s1, v3, total[nb][3]);
      } else {
        total[nb][0] = s0 * v0; total[nb][1] = s0 * v1; total[nb][2] = s1 * v2; total[nb][3] = s1 * v3;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nb][i] = ones[nb][i] = 0.f;
    }
  };

  // prologue: fill the ring
#pragma unroll
  for (int s = 0; s < kMwStages - 1; ++s) {
    if (s < k_stages) load_stage(s, s);
    cp_async_commit();
  }
  const uint32_t one2 = MwNib<T>::one2;
  const uint32_t ones_a[4] = {one2, one2, one2, one2};
  const int prow = warp * 8 + j;  // this lane's packed row within the tile
  for (int ks = 0; ks < k_stages; ++ks) {
    cp_async_wait<kMwStages - 2>();
    __syncthreads();
    {  // refill the slot freed by the previous iteration
      const int nxt = ks + kMwStages - 1;
      if (nxt < k_stages) load_stage(nxt, nxt % kMwStages);
      cp_async_commit();
    }
    const uint8_t* sx = mw_smem + (ks % kMwStages) * L::kStageBytes;
    const uint8_t* sw = sx + L::kXBytes;
#pragma unroll
    for (int c = 0; c < kMwKC / 64; ++c) {
      const int kdone = ks * kMwKC + c * 64;  // k before this 64-k block
      if (kdone < p.K) {
        const int chunk = c * 4 + q;  // the lane's 16 bytes: k = kdone + 16 q .. + 15 of its packed row
        const uint4 wv = *reinterpret_cast<const uint4*>(sw + prow * kMwKC + ((chunk ^ ((prow & 1) << 2)) << 4));
        uint32_t af[4][4];
        mw_expand<T>(wv.x, af[0]);
        mw_expand<T>(wv.y, af[1]);
        mw_expand<T>(wv.z, af[2]);
        mw_expand<T>(wv.w, af[3]);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          // token nb * 8 + j, the same 16 k as the weight bytes: 32 bytes = four steps of (b0, b1)
          const uint8_t* xr = sx + (nb * 8 + j) * kMwXPitch + (c * 64 + q * 16) * 2;
          const uint4 x0 = *reinterpret_cast<const uint4*>(xr);
          const uint4 x1 = *reinterpret_cast<const uint4*>(xr + 16);
          mw_mma(acc[nb], af[0], x0.x, x0.y, T());
          mw_mma(acc[nb], af[1], x0.z, x0.w, T());
          mw_mma(acc[nb], af[2], x1.x, x1.y, T());
          mw_mma(acc[nb], af[3], x1.z, x1.w, T());
          if (HAS_ZP) {
            mw_mma(ones[nb], ones_a, x0.x, x0.y, T());
            mw_mma(ones[nb], ones_a, x0.z, x0.w, T());
            mw_mma(ones[nb], ones_a, x1.x, x1.y, T());
            mw_mma(ones[nb], ones_a, x1.z, x1.w, T());
          }
        }
        if (GRP && (kdone + 64) % p.group == 0) fold((kdone + 64) / p.group - 1);
      }
    }
  }
  cp_async_wait<0>();
  if (!GRP) fold(0);

  // epilogue: x routing weight, one rounding, scatter.  Accumulator columns 2q, 2q + 1 are tokens nb * 8 + 2q, + 1;
  // registers (0, 2) / (1, 3) are the channel pair (2j, 2j + 1) of those two tokens.
  T* out = reinterpret_cast<T*>(p.out);
  const bool pair_ok = (p.ldo % 2 == 0) && (reinterpret_cast<uintptr_t>(out) % 4 == 0);
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int t = nb * 8 + 2 * q + h;
      if (t >= rows_valid || !ch_in) continue;
      const int flat = __ldg(p.sorted_ids + slot0 + t);
      if (flat < 0 || flat >= p.num_valid) continue;
      float v0 = total[nb][h], v1 = total[nb][2 + h];
      if (p.mul_w) {
        const float rw = load_as_f32(p.topk_w, p.topk_dtype, flat);
        v0 *= rw;
        v1 *= rw;
      }
      T* o = out + int64_t(flat) * p.ldo + ch_even;
      if (pair_ok) {
        *reinterpret_cast<uint32_t*>(o) = pack2<T>(v0, v1);
      } else {
        o[0] = from_f32<T>(v0);
        o[1] = from_f32<T>(v1);
      }
    }
  }
}

template <typename T, int TOK, bool GRP, bool HAS_ZP>
int launch_moe_w4(const MoeW4Params& p, cudaStream_t st) {
  using L = MwSmem<TOK>;
  auto kern = moe_w4_kernel<T, TOK, GRP, HAS_ZP>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::call_once(once[dev], [&] { attr_err[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes); });
  if (attr_err[dev] != cudaSuccess) return check_cuda(attr_err[dev], "cudaFuncSetAttribute(fused moe a16w4)");
  const int64_t tiles = int64_t(p.EM / p.block_m) * p.tiles_per_block * ((p.N + kMwChannels - 1) / kMwChannels);
  if (tiles > INT32_MAX) return fail(FNN_ERR_SHAPE, "fused_moe_a16w4: too many tiles");
  kern<<<unsigned(tiles), kMwThreads, L::kBytes, st>>>(p);
  return check_cuda(cudaGetLastError(), "fused moe a16w4 launch");
}

template <typename T, int TOK>
int dispatch_moe_w4(const MoeW4Params& p, cudaStream_t st) {
  const bool grp = p.group > 0, zp = p.zp != nullptr;
  if (grp) return zp ? launch_moe_w4<T, TOK, true, true>(p, st) : launch_moe_w4<T, TOK, true, false>(p, st);
  return zp ? launch_moe_w4<T, TOK, false, true>(p, st) : launch_moe_w4<T, TOK, false, false>(p, st);
}

}  // namespace
}  // namespace fnn

namespace fnn {
namespace {
int fused_moe_a16w4_impl(const void* a, int a_dtype, int64_t lda, const void* b, int64_t E, int64_t N, int64_t K,
                         const void* scale, const void* zero_points, int scale_dtype, int64_t group_size,
                         const void* topk_weights, int topk_dtype, const int32_t* sorted_token_ids, int64_t EM,
                         const int32_t* expert_ids, const int32_t* num_tokens_post_padded,
                         int64_t num_valid_tokens, int top_k, int block_m, int mul_routed_weight, void* out,
                         int out_dtype, int64_t ldo, void* workspace, size_t workspace_bytes, void* stream) {
  if (E <= 0 || N < 0 || K <= 0 || EM < 0 || lda < K || ldo < N || num_valid_tokens < 0 || top_k <= 0 || block_m <= 0 || group_size < 0)
    return fail(FNN_ERR_SHAPE, "fused_moe_a16w4: E=%lld N=%lld K=%lld EM=%lld lda=%lld ldo=%lld top_k=%d block_m=%d group=%lld",
                (long long)E, (long long)N, (long long)K, (long long)EM, (long long)lda, (long long)ldo, top_k, block_m, (long long)group_size);
  if (E * N > INT32_MAX || K > INT32_MAX || EM > INT32_MAX || num_valid_tokens > INT32_MAX)
    return fail(FNN_ERR_SHAPE, "fused_moe_a16w4: sizes must be below 2^31");
  if (N % 2 != 0) return fail(FNN_ERR_SHAPE, "fused_moe_a16w4: packed int4 needs an even N (got %lld)", (long long)N);
  if (EM % block_m != 0) return fail(FNN_ERR_SHAPE, "fused_moe_a16w4: %lld sorted slots are not a multiple of block_m=%d", (long long)EM, block_m);
  if (block_m > 64 && block_m % 64 != 0)
    return fail(FNN_ERR_UNSUPPORTED, "fused_moe_a16w4: block_m must be at most 64 or a multiple of 64 (got %d)", block_m);
  if (group_size > 0 && (group_size % 64 != 0 || K % group_size != 0))
    return fail(FNN_ERR_UNSUPPORTED, "fused_moe_a16w4: the group size must be a multiple of 64 that divides K (got %lld, K=%lld)",
                (long long)group_size, (long long)K);
  if (a_dtype != FNN_F16 && a_dtype != FNN_BF16) return fail(FNN_ERR_DTYPE, "fused_moe_a16w4: tokens must be f16 or bf16");
  if (out_dtype != a_dtype) return fail(FNN_ERR_DTYPE, "fused_moe_a16w4: output dtype must equal the token dtype");
  if (scale_dtype < FNN_F16 || scale_dtype > FNN_F32) return fail(FNN_ERR_DTYPE, "fused_moe_a16w4: scales must be f16, bf16 or f32");
  if (mul_routed_weight && (topk_dtype < FNN_F16 || topk_dtype > FNN_F32)) return fail(FNN_ERR_DTYPE, "fused_moe_a16w4: routing weights must be f16, bf16 or f32");
  if (EM == 0 || N == 0 || num_valid_tokens == 0) return FNN_OK;
  if (!a || !b || !scale || !sorted_token_ids || !expert_ids || !num_tokens_post_padded || !out || (mul_routed_weight && !topk_weights))
    return fail(FNN_ERR_NULL_POINTER, "fused_moe_a16w4: null tensor pointer");
  if (K % 16 != 0 || reinterpret_cast<uintptr_t>(a) % 16 != 0 || lda % 8 != 0 || reinterpret_cast<uintptr_t>(b) % 16 != 0)
    return fail(FNN_ERR_ALIGNMENT, "fused_moe_a16w4: K must be a multiple of 16, lda of 8, and the operands 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Blocks of 256 slots (or a multiple) with a tile for every CTA pair and a workspace for the expert-sorted copy of the
  // token rows: the tcgen05 prefill kernels of the weight-only GEMM in their fused-MoE mode.
  if (workspace && block_m % 256 == 0 && (EM / 256) * ((N + 255) / 256) >= sm_count() / 2) {
    const int r = weight_only_moe_prefill(a, a_dtype, lda, b, int(E), int(N), int(K), scale, zero_points, scale_dtype,
                                          int(group_size), topk_weights, topk_dtype, sorted_token_ids, int(EM), expert_ids,
                                          num_tokens_post_padded, int(num_valid_tokens), top_k, block_m,
                                          mul_routed_weight ? 1 : 0, out, ldo, workspace, workspace_bytes, st);
    if (r >= 0) return r;
  }
  MoeW4Params p{};
  p.a = a; p.lda = lda; p.b = static_cast<const uint8_t*>(b); p.scale = scale; p.zp = zero_points; p.topk_w = topk_weights;
  p.sorted_ids = sorted_token_ids; p.expert_ids = expert_ids; p.npp = num_tokens_post_padded; p.out = out; p.ldo = ldo;
  p.scale_dtype = scale_dtype; p.topk_dtype = topk_dtype; p.N = int(N); p.K = int(K); p.EM = int(EM);
  p.num_valid = int(num_valid_tokens); p.top_k = top_k; p.block_m = block_m; p.mul_w = mul_routed_weight ? 1 : 0;
  p.group = int(group_size); p.groups = group_size > 0 ? int(K / group_size) : 1;
  p.tile_rows = block_m < 64 ? block_m : 64;
  p.tiles_per_block = (block_m + p.tile_rows - 1) / p.tile_rows;
#define FNN_MOE_W4(T)                                                  \
  do {                                                                 \
    if (p.tile_rows <= 16) return dispatch_moe_w4<T, 16>(p, st);       \
    if (p.tile_rows <= 32) return dispatch_moe_w4<T, 32>(p, st);       \
    return dispatch_moe_w4<T, 64>(p, st);                              \
  } while (0)
  if (a_dtype == FNN_F16) FNN_MOE_W4(__half);
  FNN_MOE_W4(__nv_bfloat16);
#undef FNN_MOE_W4
}
}  // namespace
}  // namespace fnn

extern "C" int fnn_fused_moe_a16w4(const void* a, int a_dtype, int64_t lda, const void* b, int64_t E, int64_t N, int64_t K,
                                   const void* scale, const void* zero_points, int scale_dtype, int64_t group_size,
                                   const void* topk_weights, int topk_dtype, const int32_t* sorted_token_ids, int64_t EM,
                                   const int32_t* expert_ids, const int32_t* num_tokens_post_padded,
                                   int64_t num_valid_tokens, int top_k, int block_m, int mul_routed_weight, void* out,
                                   int out_dtype, int64_t ldo, void* stream) {
  return fnn::fused_moe_a16w4_impl(a, a_dtype, lda, b, E, N, K, scale, zero_points, scale_dtype, group_size, topk_weights,
                                   topk_dtype, sorted_token_ids, EM, expert_ids, num_tokens_post_padded, num_valid_tokens,
                                   top_k, block_m, mul_routed_weight, out, out_dtype, ldo, nullptr, 0, stream);
}

extern "C" size_t fnn_fused_moe_a16w4_workspace_bytes(int64_t EM, int64_t K, int64_t group_size, int has_zero_points,
                                                      int block_m) {
  if (EM <= 0 || K <= 0 || block_m <= 0 || block_m % 256 != 0) return 0;
  return fnn::weight_only_moe_prefill_workspace(EM, K, group_size, has_zero_points != 0);
}

extern "C" int fnn_fused_moe_a16w4_ws(const void* a, int a_dtype, int64_t lda, const void* b, int64_t E, int64_t N, int64_t K,
                                      const void* scale, const void* zero_points, int scale_dtype, int64_t group_size,
                                      const void* topk_weights, int topk_dtype, const int32_t* sorted_token_ids, int64_t EM,
                                      const int32_t* expert_ids, const int32_t* num_tokens_post_padded,
                                      int64_t num_valid_tokens, int top_k, int block_m, int mul_routed_weight, void* out,
                                      int out_dtype, int64_t ldo, void* workspace, size_t workspace_bytes, void* stream) {
  return fnn::fused_moe_a16w4_impl(a, a_dtype, lda, b, E, N, K, scale, zero_points, scale_dtype, group_size, topk_weights,
                                   topk_dtype, sorted_token_ids, EM, expert_ids, num_tokens_post_padded, num_valid_tokens,
                                   top_k, block_m, mul_routed_weight, out, out_dtype, ldo, workspace, workspace_bytes, stream);
}
