// Prefill-shaped weight-only GEMM (M > 16), per-channel scales: fp16/bf16 activations x int8 or
// packed-int4 weights on the tcgen05 tensor cores (kind::f16, fp32 accumulators in TMEM).
//
// The weights stay packed in HBM and on the way into the SM.  Per K block of 64:
//   warp 0       TMA: this CTA's 128 activation rows (16-bit, 128-byte swizzle) and the raw weight bytes
//                of this CTA's 128 output channels (int8: 128 rows x 64 B, int4: 64 packed rows x 64 B)
//   warps 6-9    converters: raw bytes -> exact 16-bit integers (PRMT / LOP3 magic numbers, no int->float
//                instructions), written into the K-major 128-byte-swizzled operand tile the MMA reads
//   warp 1       MMA issuer (leader CTA of the pair): tcgen05.mma.cta_group::2, M = 256 tokens, N = 256
//                channels, four K = 16 steps per block
//   warps 2-5    epilogue: out = acc * s[n] - xsum[m] * s[n] zp[n] + bias[n], rounded once to 16 bits
// The dequantised weight is the exact integer, the channel scale is applied to the fp32 accumulator, so
// w*s is never rounded to 16 bits.  Zero-points are applied through the row sums of the activations
// (xsum, a small prologue kernel into caller-provided scratch).
//
// Two rings: a deep one filled by TMA (activations + raw weight bytes, 24 KB per stage, hides the HBM/L2
// latency) and one of converted weight tiles (16 KB per stage, filled locally; its depth has to cover the
// commit -> converter -> MMA round trip across the CTA pair, which is several K blocks long).  Barriers:
// raw_full (local, TMA bytes), conv_full (in the leader: its 4 converter warps + one relayed arrival for the
// peer's 4, which meet on the peer's conv_done), empty and conv_empty (local, from the leader's tcgen05.commit
// with a two-CTA mask); tmem_full / tmem_empty as in the A8W8 pair kernel.  Every wait is bounded.
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace fnn {
namespace {

constexpr int kTM = 128;        // tokens per CTA tile (256 per pair)
constexpr int kTN = 256;        // channels per pair tile (128 converted per CTA)
constexpr int kTK = 64;         // K per stage: 128 bytes of 16-bit operand
constexpr int kPfThreads = 320; // 10 warps
constexpr int kPfStages = 5;      // TMA ring: activations + raw weight bytes
constexpr int kPfConvStages = 5;  // ring of converted weight tiles
constexpr int kPfGroupM = 16;

struct PfParams {
  const void* scale;  // [N], or [K / group, N] for group-wise scales
  const void* zp;     // nullptr or like scale
  const void* bias;   // nullptr or [N]
  const float* xsum;  // [M] row sums of the activations (only with zero-points)
  void* out;
  int64_t ldo;
  int scale_dtype, bias_dtype;
  int M, N, K;
  int group;  // 0: per-channel scales; else the K-group size (a multiple of the 64-wide K block)
  int tiles_m, tiles_n, k_blocks;
  int* status;
};

template <int BITS> struct PfSmem {
  static constexpr int kXBytes = kTM * kTK * 2;                                      // 16 KB activations
  static constexpr int kRawBytes = (BITS == 8) ? (kTN / 2) * kTK : (kTN / 4) * kTK;  // 8 KB / 4 KB raw weights
  static constexpr int kWBytes = (kTN / 2) * kTK * 2;                                // 16 KB converted weights
  static constexpr int kStageBytes = kXBytes + kRawBytes;                            // one TMA stage
  static constexpr int kConvOff = kPfStages * kStageBytes;                           // converted-tile ring
  static constexpr int kVecOff = kConvOff + kPfConvStages * kWBytes;                 // [4 warps][3][kTN] float
  static constexpr int kBarOff = kVecOff + 4 * 3 * kTN * 4;
  static constexpr int kNumBars = 2 * kPfStages + 3 * kPfConvStages + 4 + 1;
  static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
  static constexpr int kAbortOff = kTmemSlotOff + 8;
  static constexpr int kTotal = kAbortOff + 8;
  static constexpr int kDynamicBytes = kTotal + 1024;
};

__device__ __forceinline__ void pf_tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
  const int group_sz = kPfGroupM * tiles_n;
  const int gid = t / group_sz;
  const int first_m = gid * kPfGroupM;
  const int gm = min(tiles_m - first_m, kPfGroupM);
  const int r = t - gid * group_sz;
  mb = first_m + r % gm;
  nb = r / gm;
}

__device__ __forceinline__ void pf_report(int* status, volatile int* abort_flag, int code) {
  *abort_flag = code;
  if (status) atomicCAS(status, 0, code);
}

__device__ __forceinline__ uint32_t pf_prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t pf_sub2(uint32_t a, uint32_t b, __half) {
  __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t pf_sub2(uint32_t a, uint32_t b, __nv_bfloat16) {
  __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ uint32_t pf_mul2(uint32_t a, uint32_t b, __half) {
  __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t pf_mul2(uint32_t a, uint32_t b, __nv_bfloat16) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
// group-wise dequantisation of two exact integer values: T((n - zp) * s), the value the reference's torch path
// stores (flashnn/quant_gemm.py:20-36); n - zp is exact for integer zero-points, so this is one rounding
template <typename T> __device__ __forceinline__ uint32_t pf_dequant2(uint32_t n2, uint32_t s2, uint32_t z2, bool has_zp) {
  if (has_zp) n2 = pf_sub2(n2, z2, T());
  return pf_mul2(n2, s2, T());
}

// four int8 -> four exact T values (two registers, k order preserved)
template <typename T> __device__ __forceinline__ void cvt_int8x4(uint32_t w, uint32_t& r01, uint32_t& r23);
template <> __device__ __forceinline__ void cvt_int8x4<__half>(uint32_t w, uint32_t& r01, uint32_t& r23) {
  const uint32_t u = w ^ 0x80808080u;  // b + 128 under a 0x64 high byte = 1024 + (b + 128)
  r01 = pf_sub2(pf_prmt(u, 0x64646464u, 0x4140), 0x64806480u, __half());
  r23 = pf_sub2(pf_prmt(u, 0x64646464u, 0x4342), 0x64806480u, __half());
}
template <> __device__ __forceinline__ void cvt_int8x4<__nv_bfloat16>(uint32_t w, uint32_t& r01, uint32_t& r23) {
  const uint32_t u = w ^ 0x80808080u;  // through fp32: (2^23 + u) - (2^23 + 128)
  const float f0 = __uint_as_float(pf_prmt(u, 0x4B000000u, 0x7650)) - 8388736.f;
  const float f1 = __uint_as_float(pf_prmt(u, 0x4B000000u, 0x7651)) - 8388736.f;
  const float f2 = __uint_as_float(pf_prmt(u, 0x4B000000u, 0x7652)) - 8388736.f;
  const float f3 = __uint_as_float(pf_prmt(u, 0x4B000000u, 0x7653)) - 8388736.f;
  r01 = pack2<__nv_bfloat16>(f0, f1);
  r23 = pack2<__nv_bfloat16>(f2, f3);
}
// four packed bytes -> low nibbles (lo01, lo23) and high nibbles (hi01, hi23) as exact signed T values
template <typename T> struct Nib;
template <> struct Nib<__half> { static constexpr uint32_t magic = 0x64646464u, off = 0x64086408u; };         // 1024 + u, 1032
template <> struct Nib<__nv_bfloat16> { static constexpr uint32_t magic = 0x43434343u, off = 0x43084308u; };  // 128 + u, 136
template <typename T>
__device__ __forceinline__ void cvt_int4x8(uint32_t w, uint32_t& lo01, uint32_t& lo23, uint32_t& hi01, uint32_t& hi23) {
  const uint32_t lo = (w & 0x0F0F0F0Fu) ^ 0x08080808u;
  const uint32_t hi = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
  lo01 = pf_sub2(pf_prmt(lo, Nib<T>::magic, 0x4140), Nib<T>::off, T());
  lo23 = pf_sub2(pf_prmt(lo, Nib<T>::magic, 0x4342), Nib<T>::off, T());
  hi01 = pf_sub2(pf_prmt(hi, Nib<T>::magic, 0x4140), Nib<T>::off, T());
  hi23 = pf_sub2(pf_prmt(hi, Nib<T>::magic, 0x4342), Nib<T>::off, T());
}

// D[tmem of both CTAs] (+)= A[smem of both CTAs] * B[smem halves of both CTAs]^T, 16-bit -> fp32, M = 256
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// byte offset of 16-byte chunk `kc` (0..7) of row `row` in a K-major tile with 128-byte rows and 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t kc) { return row * 128u + ((kc ^ (row & 7u)) << 4); }

// GRP: group-wise scales.  The converter warps then write T((n - zp) * s[k / group, n]) instead of the bare integer
// and the epilogue only adds the bias.
template <typename T, int BITS, bool GRP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPfThreads, 1)
wo_umma_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                    const PfParams p) {
  using L = PfSmem<BITS>;
  constexpr int STAGES = kPfStages;
  constexpr int CSTAGES = kPfConvStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* vec_smem = reinterpret_cast<float*>(smem + L::kVecOff);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* raw_full = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* conv_full = bars + 2 * STAGES;
  uint64_t* conv_empty = bars + 2 * STAGES + CSTAGES;
  uint64_t* conv_done = bars + 2 * STAGES + 2 * CSTAGES;  // peer CTA only: its four converter warps
  uint64_t* tmem_full_bar = bars + 2 * STAGES + 3 * CSTAGES;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint64_t* drain_bar = tmem_full_bar + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlotOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;
  constexpr uint32_t kTmemCols = 2 * kTN;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < CSTAGES; ++s) {
      mbar_init(&conv_full[s], 5);  // leader: its 4 converter warps + the peer's relay
      mbar_init(&conv_done[s], 4);
      mbar_init(&conv_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 8);
    }
    mbar_init(drain_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    const bool leader_lane = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    long long issued = 0;
    bool ok = true;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
      int mb, nb;
      pf_tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
      const int w_row = (BITS == 8) ? nb * kTN + int(rank) * (kTN / 2) : (nb * kTN + int(rank) * (kTN / 2)) / 2;
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (leader_lane) pf_report(p.status, abort_flag, DEV_TIMEOUT_PRODUCER);
          break;
        }
        if (leader_lane) {
          uint8_t* sx = smem + stage * L::kStageBytes;
          mbar_expect_tx(&raw_full[stage], L::kXBytes + L::kRawBytes);
          tma_load_2d(sx, &tmap_x, &raw_full[stage], kb * kTK, mb * 256 + int(rank) * kTM);
          tma_load_2d(sx + L::kXBytes, &tmap_w, &raw_full[stage], kb * kTK, w_row);
          ++issued;
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    if (leader_lane) {  // the last stages issued have been consumed (or the CTA is aborting) before exit
      const long long first = issued > STAGES ? issued - STAGES : 0;
      for (long long i = first; i < issued; ++i)
        if (!mbar_wait_bounded(&empty_bar[i % STAGES], uint32_t((i / STAGES) & 1), abort_flag)) break;
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader only) -------------------------------
    const bool leader_lane = elect_one();
    if (rank == 0) {
      constexpr uint32_t idesc = umma_idesc(/*f32*/ 1, std::is_same<T, __half>::value ? 0u : 1u, 256, kTN);
      int stage = 0, cstage = 0;
      uint32_t phase = 0, cphase = 0;
      int local = 0;
      bool ok = true;
      bool issued_any = false;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs, ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        ok = mbar_wait_bounded(&tmem_empty_bar[buf], acc_phase ^ 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (leader_lane) pf_report(p.status, abort_flag, DEV_TIMEOUT_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kTN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          ok = mbar_wait_bounded(&conv_full[cstage], cphase, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (leader_lane) pf_report(p.status, abort_flag, DEV_TIMEOUT_MMA);
            break;
          }
          tc_fence_after();
          if (leader_lane) {
            const uint32_t sx = smem_u32(smem + stage * L::kStageBytes);
            const uint32_t sw = smem_u32(smem + L::kConvOff + cstage * L::kWBytes);
#pragma unroll
            for (int k = 0; k < kTK / 16; ++k)
              umma_f16_pair(tmem_d, umma_desc_k_sw128(sx + k * 32), umma_desc_k_sw128(sw + k * 32), idesc,
                            (kb | k) != 0 ? 1u : 0u);
            tc_commit_pair(&empty_bar[stage], 0x3);     // activations + raw bytes of this stage, both CTAs
            tc_commit_pair(&conv_empty[cstage], 0x3);   // converted tile, both CTAs
            issued_any = true;
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (++cstage == CSTAGES) { cstage = 0; cphase ^= 1; }
        }
        if (ok && leader_lane) tc_commit_pair(&tmem_full_bar[buf], 0x3);
        __syncwarp();
      }
      if (leader_lane && issued_any) {
        int none = 0;
        tc_commit_pair(drain_bar, 0x1);
        if (!mbar_wait_bounded(drain_bar, 0, &none)) pf_report(p.status, abort_flag, DEV_TIMEOUT_DRAIN);
      }
    } else {
      // peer CTA: relay "this CTA's converted tile is ready" to the leader's barrier, one remote arrive per
      // K block, so the converter warps themselves only ever signal locally
      int cstage = 0;
      uint32_t cphase = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          ok = mbar_wait_bounded(&conv_done[cstage], cphase, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (leader_lane) pf_report(p.status, abort_flag, DEV_TIMEOUT_MMA);
            break;
          }
          if (leader_lane) mbar_arrive_cluster(map_to_cta(smem_u32(&conv_full[cstage]), 0));
          __syncwarp();
          if (++cstage == CSTAGES) { cstage = 0; cphase ^= 1; }
        }
      }
    }
  } else if (warp < 6) {
    // -------------------------------- epilogue (both CTAs) --------------------------------
    const int quarter = warp & 3;
    float* cs = vec_smem + quarter * 3 * kTN;  // scale, scale*zp, bias of this tile's channels (private copy)
    float* cz = cs + kTN;
    float* cb = cz + kTN;
    T* out = reinterpret_cast<T*>(p.out);
    const bool vec_ok = (p.ldo % 8 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0);
    int local = 0;
    bool ok = true;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs, ++local) {
      int mb, nb;
      pf_tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int row = mb * 256 + int(rank) * kTM + quarter * 32 + lane;
      const int n0 = nb * kTN;
      for (int j = lane; j < kTN; j += 32) {
        const bool in = n0 + j < p.N;
        const float s = GRP ? 1.f : (in ? load_as_f32(p.scale, p.scale_dtype, n0 + j) : 0.f);
        cs[j] = s;
        cz[j] = (!GRP && in && p.zp) ? s * load_as_f32(p.zp, p.scale_dtype, n0 + j) : 0.f;
        cb[j] = (in && p.bias) ? load_as_f32(p.bias, p.bias_dtype, n0 + j) : 0.f;
      }
      const float xs = (!GRP && p.zp && row < p.M) ? p.xsum[row] : 0.f;
      __syncwarp();

      ok = mbar_wait_bounded(&tmem_full_bar[buf], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) pf_report(p.status, abort_flag, DEV_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * kTN;
#pragma unroll 1
      for (int c = 0; c < kTN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tc_wait_ld();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = fmaf(__uint_as_float(r[j]), cs[c * 32 + j], fmaf(-xs, cz[c * 32 + j], cb[c * 32 + j]));
          T* orow = out + int64_t(row) * p.ldo + col0;
          if (col0 + 32 <= p.N && vec_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8)
              *reinterpret_cast<uint4*>(orow + j) =
                  make_uint4(pack2<T>(v[j], v[j + 1]), pack2<T>(v[j + 2], v[j + 3]), pack2<T>(v[j + 4], v[j + 5]),
                             pack2<T>(v[j + 6], v[j + 7]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) orow[j] = from_f32<T>(v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[buf]), 0));
    }
  } else {
    // -------------------------------- converters (both CTAs) --------------------------------
    const int ct = threadIdx.x - 6 * 32;  // 0..127
    int stage = 0, cstage = 0;
    uint32_t phase = 0, cphase = 0;
    bool ok = true;
    // group-wise scales: packed (s, s) and (zp, zp) of the four channels this thread converts, reloaded per K group
    uint32_t gs2[4] = {0, 0, 0, 0}, gz2[4] = {0, 0, 0, 0};
    const bool has_zp = p.zp != nullptr;
    const int kb_per_group = GRP ? p.group / kTK : 1;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
      int mb_c, nb_c;
      pf_tile_coords(t, p.tiles_m, p.tiles_n, mb_c, nb_c);
      const int ch_base = nb_c * kTN + int(rank) * (kTN / 2);  // first channel of this CTA's half of the tile
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (GRP && kb % kb_per_group == 0) {
          const int64_t grow = int64_t(kb / kb_per_group) * p.N;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // int8: rows ct/4 + 32 i; int4: packed rows ct/4 + 32 (i / 2), channel 2 * prow + (i & 1)
            const int ch = ch_base + ((BITS == 8) ? (ct >> 2) + 32 * i : 2 * ((ct >> 2) + 32 * (i >> 1)) + (i & 1));
            const float sv = ch < p.N ? load_as_f32(p.scale, p.scale_dtype, grow + ch) : 0.f;
            const float zv = (has_zp && ch < p.N) ? load_as_f32(p.zp, p.scale_dtype, grow + ch) : 0.f;
            gs2[i] = pack2<T>(sv, sv);
            gz2[i] = pack2<T>(zv, zv);
          }
        }
        ok = mbar_wait_bounded(&conv_empty[cstage], cphase ^ 1, abort_flag) &&
             mbar_wait_bounded(&raw_full[stage], phase, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) pf_report(p.status, abort_flag, DEV_TIMEOUT_EPILOGUE);
          break;
        }
        uint8_t* sw = smem + L::kConvOff + cstage * L::kWBytes;                // converted tile: 128 rows x 128 B, swizzled
        const uint8_t* raw = smem + stage * L::kStageBytes + L::kXBytes;       // raw tile: rows of 64 B, not swizzled
        if (BITS == 8) {
          // 128 rows x 4 chunks of 16 bytes; chunk id -> (row = id / 4, c = id % 4): 16 k -> 32 bytes out
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int id = ct + i * 128;
            const uint32_t row = id >> 2, c = id & 3;
            const uint4 w = *reinterpret_cast<const uint4*>(raw + id * 16);
            uint4 o0, o1;
            cvt_int8x4<T>(w.x, o0.x, o0.y);
            cvt_int8x4<T>(w.y, o0.z, o0.w);
            cvt_int8x4<T>(w.z, o1.x, o1.y);
            cvt_int8x4<T>(w.w, o1.z, o1.w);
            if (GRP) {
              o0.x = pf_dequant2<T>(o0.x, gs2[i], gz2[i], has_zp); o0.y = pf_dequant2<T>(o0.y, gs2[i], gz2[i], has_zp);
              o0.z = pf_dequant2<T>(o0.z, gs2[i], gz2[i], has_zp); o0.w = pf_dequant2<T>(o0.w, gs2[i], gz2[i], has_zp);
              o1.x = pf_dequant2<T>(o1.x, gs2[i], gz2[i], has_zp); o1.y = pf_dequant2<T>(o1.y, gs2[i], gz2[i], has_zp);
              o1.z = pf_dequant2<T>(o1.z, gs2[i], gz2[i], has_zp); o1.w = pf_dequant2<T>(o1.w, gs2[i], gz2[i], has_zp);
            }
            *reinterpret_cast<uint4*>(sw + sw128(row, 2 * c)) = o0;
            *reinterpret_cast<uint4*>(sw + sw128(row, 2 * c + 1)) = o1;
          }
        } else {
          // 64 packed rows x 4 chunks; packed row j carries channel rows 2j (low nibbles) and 2j+1 (high)
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int id = ct + i * 128;
            const uint32_t prow = id >> 2, c = id & 3;
            const uint4 w = *reinterpret_cast<const uint4*>(raw + id * 16);
            uint4 l0, l1, h0, h1;
            cvt_int4x8<T>(w.x, l0.x, l0.y, h0.x, h0.y);
            cvt_int4x8<T>(w.y, l0.z, l0.w, h0.z, h0.w);
            cvt_int4x8<T>(w.z, l1.x, l1.y, h1.x, h1.y);
            cvt_int4x8<T>(w.w, l1.z, l1.w, h1.z, h1.w);
            if (GRP) {
              const uint32_t sl = gs2[2 * i], zl = gz2[2 * i], sh = gs2[2 * i + 1], zh = gz2[2 * i + 1];
              l0.x = pf_dequant2<T>(l0.x, sl, zl, has_zp); l0.y = pf_dequant2<T>(l0.y, sl, zl, has_zp);
              l0.z = pf_dequant2<T>(l0.z, sl, zl, has_zp); l0.w = pf_dequant2<T>(l0.w, sl, zl, has_zp);
              l1.x = pf_dequant2<T>(l1.x, sl, zl, has_zp); l1.y = pf_dequant2<T>(l1.y, sl, zl, has_zp);
              l1.z = pf_dequant2<T>(l1.z, sl, zl, has_zp); l1.w = pf_dequant2<T>(l1.w, sl, zl, has_zp);
              h0.x = pf_dequant2<T>(h0.x, sh, zh, has_zp); h0.y = pf_dequant2<T>(h0.y, sh, zh, has_zp);
              h0.z = pf_dequant2<T>(h0.z, sh, zh, has_zp); h0.w = pf_dequant2<T>(h0.w, sh, zh, has_zp);
              h1.x = pf_dequant2<T>(h1.x, sh, zh, has_zp); h1.y = pf_dequant2<T>(h1.y, sh, zh, has_zp);
              h1.z = pf_dequant2<T>(h1.z, sh, zh, has_zp); h1.w = pf_dequant2<T>(h1.w, sh, zh, has_zp);
            }
            *reinterpret_cast<uint4*>(sw + sw128(2 * prow, 2 * c)) = l0;
            *reinterpret_cast<uint4*>(sw + sw128(2 * prow, 2 * c + 1)) = l1;
            *reinterpret_cast<uint4*>(sw + sw128(2 * prow + 1, 2 * c)) = h0;
            *reinterpret_cast<uint4*>(sw + sw128(2 * prow + 1, 2 * c + 1)) = h1;
          }
        }
        fence_proxy_async_smem();  // the tensor core reads these bytes through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(rank == 0 ? &conv_full[cstage] : &conv_done[cstage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
        if (++cstage == CSTAGES) { cstage = 0; cphase ^= 1; }
      }
    }
  }

  // -------------------------------- teardown --------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// xsum[m] = sum_k x[m, k] in fp32, one warp per row
template <typename T>
__global__ void row_sum_kernel(const T* __restrict__ act, int64_t lda, float* __restrict__ xsum, int M, int K) {
  const int64_t row = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const T* x = act + row * lda;
  float s = 0.f;
  for (int i = lane; i < K; i += 32) s += to_f32(x[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) xsum[row] = s;
}

template <typename T, int BITS, bool GRP>
int launch_prefill_g(const T* act, int64_t lda, const uint8_t* qw, PfParams p, float* xsum_ws, cudaStream_t st) {
  using L = PfSmem<BITS>;
  static_assert(L::kDynamicBytes <= 227 * 1024, "shared memory budget");
  static_assert(L::kStageBytes % 1024 == 0 && L::kWBytes % 1024 == 0 && L::kConvOff % 1024 == 0, "tile alignment");
  auto kern = wo_umma_pair_kernel<T, BITS, GRP>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];  // per device, so that a failure is reported on every call and not only the first
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  });
  if (attr_err[dev] != cudaSuccess) return check_cuda(attr_err[dev], "cudaFuncSetAttribute(weight-only prefill)");
  if (p.zp && !GRP) {
    row_sum_kernel<T><<<unsigned((int64_t(p.M) * 32 + 255) / 256), 256, 0, st>>>(act, lda, xsum_ws, p.M, p.K);
    if (int e = check_cuda(cudaGetLastError(), "row_sum launch")) return e;
    p.xsum = xsum_ws;
  }
  CUtensorMap tx, tw;
  if (int e = make_tmap_2d(&tx, 2, act, p.M, p.K, lda * 2, kTK, kTM, true)) return e;
  const int64_t w_rows = (BITS == 8) ? p.N : p.N / 2;
  if (int e = make_tmap_2d(&tw, 1, qw, w_rows, p.K, p.K, kTK, (BITS == 8) ? kTN / 2 : kTN / 4, false)) return e;
  p.tiles_m = (p.M + 255) / 256;
  p.tiles_n = (p.N + kTN - 1) / kTN;
  p.k_blocks = (p.K + kTK - 1) / kTK;
  const int tiles = p.tiles_m * p.tiles_n;
  const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  kern<<<2 * pairs, kPfThreads, L::kDynamicBytes, st>>>(tx, tw, p);
  return check_cuda(cudaGetLastError(), "weight-only prefill launch");
}

template <typename T, int BITS>
int launch_prefill(const T* act, int64_t lda, const uint8_t* qw, PfParams p, float* xsum_ws, cudaStream_t st) {
  return p.group > 0 ? launch_prefill_g<T, BITS, true>(act, lda, qw, p, xsum_ws, st)
                     : launch_prefill_g<T, BITS, false>(act, lda, qw, p, xsum_ws, st);
}

}  // namespace

// Entry used by fnn_gemm_weight_only for M > 16 with per-channel scales.  Returns -1 when the operands do
// not meet the TMA path's alignment rules (the caller then takes the generic kernel).
int weight_only_prefill(const void* act, int act_dtype, int64_t lda, const void* qweight, int bits, const void* scale,
                        const void* zp, int scale_dtype, int group, const void* bias, int bias_dtype, void* out,
                        int64_t ldo, int M, int N, int K, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (group > 0 && (group % kTK != 0 || K % group != 0)) return -1;  // a K block must lie inside one scale group
  if (reinterpret_cast<uintptr_t>(act) % 16 != 0 || (lda * 2) % 16 != 0) return -1;
  if (reinterpret_cast<uintptr_t>(qweight) % 16 != 0 || K % 16 != 0) return -1;
  if (bits == 4 && N % 2 != 0) return -1;
  float* xsum = nullptr;
  if (zp && group == 0) {
    const size_t need = size_t(M) * sizeof(float);
    if (!workspace || workspace_bytes < need)
      return fail(FNN_ERR_WORKSPACE, "gemm_weight_only: zero-points need %zu bytes of workspace, got %zu", need, workspace_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return fail(FNN_ERR_ALIGNMENT, "gemm_weight_only: workspace must be 256-byte aligned");
    xsum = static_cast<float*>(workspace);
  }
  PfParams p{};
  p.scale = scale; p.zp = zp; p.bias = bias; p.xsum = nullptr; p.out = out; p.ldo = ldo;
  p.scale_dtype = scale_dtype; p.bias_dtype = bias_dtype; p.M = M; p.N = N; p.K = K; p.group = group;
  p.status = device_status_word();
  const uint8_t* qw = static_cast<const uint8_t*>(qweight);
  if (act_dtype == FNN_F16) {
    const __half* a = static_cast<const __half*>(act);
    return bits == 8 ? launch_prefill<__half, 8>(a, lda, qw, p, xsum, st) : launch_prefill<__half, 4>(a, lda, qw, p, xsum, st);
  }
  const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(act);
  return bits == 8 ? launch_prefill<__nv_bfloat16, 8>(a, lda, qw, p, xsum, st) : launch_prefill<__nv_bfloat16, 4>(a, lda, qw, p, xsum, st);
}

}  // namespace fnn

// ---------------------------------------------------------------------------
// Entry point that allocates nothing: the row-sum scratch lives in the library image.
// ---------------------------------------------------------------------------
namespace fnn {
namespace {

constexpr int kStaticRows = 65536;  // most activation rows (tokens) one call may bring

// Row sums of the activations for the zero-point term; 256 KB on every GPU that loads the library, for as
// long as the process lives.  In host code this name is only a handle for the runtime, not a device address.
static __device__ __align__(256) float g_static_row_sums[kStaticRows];

float* g_static_row_sums_addr[64];
std::once_flag g_static_once[64];
cudaError_t g_static_err[64];

}  // namespace
}  // namespace fnn

extern "C" int fnn_gemm_weight_only_prefill_static(const void* act, int act_dtype, int64_t lda, const void* qweight,
                                                   int weight_bits, const void* scale, const void* zero_points,
                                                   int scale_dtype, const void* bias, int bias_dtype, void* out,
                                                   int out_dtype, int64_t ldo, int64_t M, int64_t N, int64_t K,
                                                   void* stream) {
  using namespace fnn;
  if (M < 0 || N < 0 || K <= 0 || lda < K || ldo < N)
    return fail(FNN_ERR_SHAPE, "gemm_weight_only_prefill_static: M=%lld N=%lld K=%lld lda=%lld ldo=%lld", (long long)M,
                (long long)N, (long long)K, (long long)lda, (long long)ldo);
  if (M > kStaticRows)
    return fail(FNN_ERR_WORKSPACE, "gemm_weight_only_prefill_static: M=%lld exceeds the %d rows the built-in scratch holds; "
                "use fnn_gemm_weight_only with a caller-provided workspace", (long long)M, kStaticRows);
  if (N > INT32_MAX || K > INT32_MAX) return fail(FNN_ERR_SHAPE, "gemm_weight_only_prefill_static: sizes must be below 2^31");
  if (weight_bits != 4 && weight_bits != 8) return fail(FNN_ERR_UNSUPPORTED, "gemm_weight_only_prefill_static: weight_bits must be 4 or 8 (got %d)", weight_bits);
  if (weight_bits == 4 && (N % 2) != 0) return fail(FNN_ERR_SHAPE, "gemm_weight_only_prefill_static: packed int4 needs an even N");
  if (act_dtype != FNN_F16 && act_dtype != FNN_BF16) return fail(FNN_ERR_DTYPE, "gemm_weight_only_prefill_static: activations must be f16 or bf16");
  if (out_dtype != act_dtype) return fail(FNN_ERR_DTYPE, "gemm_weight_only_prefill_static: output dtype must equal the activation dtype");
  if (scale_dtype < FNN_F16 || scale_dtype > FNN_F32) return fail(FNN_ERR_DTYPE, "gemm_weight_only_prefill_static: bad scale dtype code %d", scale_dtype);
  if (bias && (bias_dtype < FNN_F16 || bias_dtype > FNN_F32)) return fail(FNN_ERR_DTYPE, "gemm_weight_only_prefill_static: bad bias dtype code %d", bias_dtype);
  if (M == 0 || N == 0) return FNN_OK;
  if (!act || !qweight || !scale || !out) return fail(FNN_ERR_NULL_POINTER, "gemm_weight_only_prefill_static: null tensor pointer");

  // Set-up, once per device and with that device current: ask the runtime where this device's copy of the
  // array lives.  (The array's name itself must never be handed to a kernel from host code.)
  int dev = 0;
  if (int e = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return e;
  if (dev < 0 || dev >= 64) return fail(FNN_ERR_UNSUPPORTED, "gemm_weight_only_prefill_static: device index %d is out of range", dev);
  std::call_once(g_static_once[dev], [dev] {
    float* ptr = nullptr;
    g_static_err[dev] = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_row_sums);
    g_static_row_sums_addr[dev] = (g_static_err[dev] == cudaSuccess) ? ptr : nullptr;
  });
  if (g_static_err[dev] != cudaSuccess || !g_static_row_sums_addr[dev])
    return check_cuda(g_static_err[dev] != cudaSuccess ? g_static_err[dev] : cudaErrorInvalidSymbol,
                      "cudaGetSymbolAddress(row-sum scratch)");

  // Every element the kernel reads (rows 0..M-1) is rewritten by the row-sum kernel of this same call, so nothing
  // left over from an earlier call is ever used and nothing has to be cleared.
  const int r = weight_only_prefill(act, act_dtype, lda, qweight, weight_bits, scale, zero_points, scale_dtype, 0, bias,
                                    bias_dtype, out, ldo, int(M), int(N), int(K), g_static_row_sums_addr[dev],
                                    sizeof(float) * kStaticRows, static_cast<cudaStream_t>(stream));
  if (r < 0)
    return fail(FNN_ERR_ALIGNMENT, "gemm_weight_only_prefill_static: act and qweight must be 16-byte aligned, lda a multiple "
                "of 8 elements and K a multiple of 16");
  return r;
}
