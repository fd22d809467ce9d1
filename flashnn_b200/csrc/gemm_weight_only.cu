// Prefill-shaped weight-only GEMM (M > 16): fp16/bf16 activations x int8 or packed-int4 weights on the tcgen05
// tensor cores (kind::f16, fp32 accumulators in TMEM), per-channel scales (described here) or group-wise scales
// (second kernel, described where it is defined).
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
// Per-channel kernel: warps 0-3 TMA, MMA and two idle ones; 4-7 epilogue; 8-15 converters.  Whole warpgroups, so that
// each role sizes its registers with setmaxnreg (40 / 200 / 72).  Eight converter warps: with four, a device-side
// timeline showed them, not the MMAs, setting the pace (0.51 us per K block against 0.34 us); twelve or sixteen are
// no faster than eight.
constexpr int kPfConvWarps = 8;
// The converter warps take the K blocks in this many teams, in turn.  Measured: int4 weights (two iterations per thread
// and block, four shared-memory stores each) gain 5 % from two teams of four warps (1319 -> 1390 TFLOP/s at
// 2048 x 28672 x 8192), int8 weights are the same either way, the group-wise kernel's four warps lose 4 % as two teams.
template <int BITS> constexpr int pf_conv_teams() { return BITS == 4 ? 2 : 1; }
constexpr int kPgConvTeams = 1;
constexpr int kPfThreads = (8 + kPfConvWarps) * 32;
constexpr int kPfConvRegs = 72;
constexpr int kPfStages = 5;      // TMA ring: activations + raw weight bytes
constexpr int kPfConvStages = 5;  // ring of converted weight tiles
constexpr int kPfGroupM = 16;
constexpr int kPgScaleStages = 4;  // group-wise kernel: scale groups staged ahead of the epilogue

struct PfParams {
  const void* scale;  // [N], or [K / group, N] for group-wise scales
  const void* zp;     // nullptr or like scale
  const void* bias;   // nullptr or [N]
  const float* xsum;  // row sums of the activations (only with zero-points): [M], or [K / group, M] per scale group
  void* out;
  int64_t ldo;
  int scale_dtype, bias_dtype;
  int M, N, K;
  int group;  // 0: per-channel scales; else the K-group size (a multiple of the 64-wide K block)
  int tiles_m, tiles_n, k_blocks;
  int moe;  // fused-MoE mode, see PfMoe
  int* status;
};

// Fused MoE (PfParams::moe != 0): the activations are the expert-sorted copy of the token rows [EM, K] (M = EM), a
// 256-row tile is one block of sorted slots (block_m is a multiple of 256) whose expert picks the weight rows and the
// scales ([E, N], or [E, N, K / group] for group-wise ones); the epilogue multiplies by the routing weight and scatters
// each slot's row to its flat (token, choice) index.  Row tiles past the slots in use are left out by every role
// alike.  A kernel parameter of its own: the dense kernels' parameter block stays as small as it was
// (growing it cost the group-wise kernel 4 % through local-memory copies of the block).
struct PfMoe {
  int num_experts, top_k, num_valid, mul_w, block_m, topk_dtype;
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* npp;
  const void* topk_w;
};

// Expert of the row tile mb, or -1 where the tile lies past the slots in use (or names no expert).
__device__ __forceinline__ int pf_moe_expert(const PfMoe& m, int mb) {
  if (mb * 256 >= __ldg(m.npp)) return -1;
  const int e = __ldg(m.expert_ids + (mb * 256) / m.block_m);
  return (e >= 0 && e < m.num_experts) ? e : -1;
}

template <int BITS> struct PfSmem {
  static constexpr int kXBytes = kTM * kTK * 2;                                      // 16 KB activations
  static constexpr int kRawBytes = (BITS == 8) ? (kTN / 2) * kTK : (kTN / 4) * kTK;  // 8 KB / 4 KB raw weights
  static constexpr int kWBytes = (kTN / 2) * kTK * 2;                                // 16 KB converted weights
  static constexpr int kStageBytes = kXBytes + kRawBytes;                            // one TMA stage
  static constexpr int kConvOff = kPfStages * kStageBytes;                           // converted-tile ring
  static constexpr int kVecOff = kConvOff + kPfConvStages * kWBytes;                 // [4 warps][3][kTN] float (group-wise kernel: scale ring [2][kPgScaleStages][kTN] + bias [2][kTN])
  static constexpr int kBarOff = kVecOff + 4 * 3 * kTN * 4;
  static constexpr int kNumBars = 2 * kPfStages + 3 * kPfConvStages + 8 + 1 + 2 * kPgScaleStages;
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

// ---------------------------------------------------------------------------------------------------------
// Roles shared by the per-channel kernel and the group-wise kernel.  `bars` layout: raw_full[S], empty[S],
// conv_full[C], conv_empty[C], conv_done[C], tmem_full[4], tmem_empty[4], drain, then (group-wise kernel only)
// scale_full[kPgScaleStages], scale_empty[kPgScaleStages].
// ---------------------------------------------------------------------------------------------------------
struct PfBars {
  uint64_t *raw_full, *empty, *conv_full, *conv_empty, *conv_done, *tmem_full, *tmem_empty, *drain, *scale_full, *scale_empty;
};
__device__ __forceinline__ PfBars pf_bars(uint64_t* bars) {
  PfBars b;
  b.raw_full = bars;
  b.empty = bars + kPfStages;
  b.conv_full = bars + 2 * kPfStages;
  b.conv_empty = b.conv_full + kPfConvStages;
  b.conv_done = b.conv_empty + kPfConvStages;  // peer CTA only: its four converter warps
  b.tmem_full = b.conv_done + kPfConvStages;
  b.tmem_empty = b.tmem_full + 4;
  b.drain = b.tmem_full + 8;
  b.scale_full = b.tmem_full + 9;
  b.scale_empty = b.scale_full + kPgScaleStages;
  return b;
}

// Thread 0 of each CTA: barrier counts.  `epi_arrivals` = epilogue warps of both CTAs that free an accumulator.
__device__ __forceinline__ void pf_init_bars(const PfBars& b, int epi_arrivals, bool grp, int conv_warps = 4) {
  for (int s = 0; s < kPfStages; ++s) {
    mbar_init(&b.raw_full[s], 1);
    mbar_init(&b.empty[s], 1);
  }
  for (int s = 0; s < kPfConvStages; ++s) {
    mbar_init(&b.conv_full[s], conv_warps + 1);  // leader: its converter warps + the peer's relay
    mbar_init(&b.conv_done[s], conv_warps);
    mbar_init(&b.conv_empty[s], 1);
  }
  for (int i = 0; i < 4; ++i) {  // up to four accumulators (512 TMEM columns / tile width)
    mbar_init(&b.tmem_full[i], 1);
    mbar_init(&b.tmem_empty[i], epi_arrivals);
  }
  mbar_init(b.drain, 1);
  if (grp)
    for (int i = 0; i < kPgScaleStages; ++i) {
      mbar_init(&b.scale_full[i], 2);   // the two staging warps, one per column half
      mbar_init(&b.scale_empty[i], 8);  // the eight epilogue warps
    }
  mbar_fence_init();
}

// Fused MoE: is the row tile of tile t in use?  (Every role leaves out the same tiles, so the rings stay in step.)
__device__ __forceinline__ bool pf_tile_in_use(const PfMoe* moe, const PfParams& p, int t) {
  if (!moe) return true;
  int mb, nb;
  pf_tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
  return pf_moe_expert(*moe, mb) >= 0;
}

// warp 0 of both CTAs: TMA loads of this CTA's 128 activation rows and its raw weight bytes, one K block per stage
template <int BITS, int BN = kTN, bool MOE = false>
__device__ __forceinline__ void pf_producer(uint8_t* smem, const PfBars& b, const CUtensorMap* tmap_x,
                                            const CUtensorMap* tmap_w, const PfParams& p, uint32_t rank, int pair_id,
                                            int num_pairs, volatile int* abort_flag, const PfMoe* moe = nullptr) {
  using L = PfSmem<BITS>;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const bool leader_lane = elect_one();
  int stage = 0;
  uint32_t phase = 0;
  long long issued = 0;
  bool ok = true;
  for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
    int mb, nb;
    pf_tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
    int w_row = (BITS == 8) ? nb * BN + int(rank) * (BN / 2) : (nb * BN + int(rank) * (BN / 2)) / 2;
    if (MOE) {  // the expert's rows of the weight stack; a tile that is not in use is left out
      const int e = pf_moe_expert(*moe, mb);
      if (e < 0) continue;
      w_row += e * ((BITS == 8) ? p.N : p.N / 2);
    }
    for (int kb = 0; kb < p.k_blocks; ++kb) {
      ok = mbar_wait_bounded(&b.empty[stage], phase ^ 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (leader_lane) pf_report(p.status, abort_flag, DEV_TIMEOUT_PRODUCER);
        break;
      }
      if (leader_lane) {
        uint8_t* sx = smem + stage * L::kStageBytes;
        mbar_expect_tx(&b.raw_full[stage], L::kXBytes + ((BITS == 8) ? (BN / 2) * kTK : (BN / 4) * kTK));
        tma_load_2d(sx, tmap_x, &b.raw_full[stage], kb * kTK, mb * 256 + int(rank) * kTM);
        tma_load_2d(sx + L::kXBytes, tmap_w, &b.raw_full[stage], kb * kTK, w_row);
        ++issued;
      }
      __syncwarp();
      if (++stage == kPfStages) { stage = 0; phase ^= 1; }
    }
  }
  if (leader_lane) {  // the last stages issued have been consumed (or the CTA is aborting) before exit
    const long long first = issued > kPfStages ? issued - kPfStages : 0;
    for (long long i = first; i < issued; ++i)
      if (!mbar_wait_bounded(&b.empty[i % kPfStages], uint32_t((i / kPfStages) & 1), abort_flag)) break;
  }
}

// warp 1 of the leader CTA: issues the MMAs of both CTAs.  An accumulator (one of the two TMEM buffers) collects
// `kb_per_acc` K blocks and is then handed to the epilogue: the whole K range for per-channel scales, one scale
// group for group-wise scales.
template <typename T, int BITS, int BN = kTN, int NBUF = 2, int ACC_STRIDE = kTN>
__device__ __forceinline__ void pf_mma(uint8_t* smem, const PfBars& b, const PfParams& p, uint32_t tmem_base, int pair_id,
                                       int num_pairs, int kb_per_acc, volatile int* abort_flag, const PfMoe* moe = nullptr) {
  using L = PfSmem<BITS>;
  constexpr uint32_t idesc = umma_idesc(/*f32*/ 1, std::is_same<T, __half>::value ? 0u : 1u, 256, BN);
  const int num_tiles = p.tiles_m * p.tiles_n;
  const bool leader_lane = elect_one();
  int stage = 0, cstage = 0;
  uint32_t cphase = 0;
  int seg = 0;  // accumulators started so far
  bool ok = true;
  bool issued_any = false;
  for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
    if (!pf_tile_in_use(moe, p, t)) continue;
    for (int kb0 = 0; kb0 < p.k_blocks && ok; kb0 += kb_per_acc, ++seg) {
      const int buf = seg % NBUF;
      const uint32_t acc_phase = (seg / NBUF) & 1;
      ok = mbar_wait_bounded(&b.tmem_empty[buf], acc_phase ^ 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (leader_lane) pf_report(p.status, abort_flag, DEV_TIMEOUT_MMA);
        break;
      }
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + buf * ACC_STRIDE;
      const int kb1 = min(kb0 + kb_per_acc, p.k_blocks);
      for (int kb = kb0; kb < kb1; ++kb) {
        ok = mbar_wait_bounded(&b.conv_full[cstage], cphase, abort_flag);
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
                          (kb != kb0 || k != 0) ? 1u : 0u);
          tc_commit_pair(&b.empty[stage], 0x3);        // activations + raw bytes of this stage, both CTAs
          tc_commit_pair(&b.conv_empty[cstage], 0x3);  // converted tile, both CTAs
          issued_any = true;
        }
        __syncwarp();
        if (++stage == kPfStages) stage = 0;
        if (++cstage == kPfConvStages) { cstage = 0; cphase ^= 1; }
      }
      if (ok && leader_lane) tc_commit_pair(&b.tmem_full[buf], 0x3);
      __syncwarp();
    }
  }
  if (leader_lane && issued_any) {
    int none = 0;
    tc_commit_pair(b.drain, 0x1);
    if (!mbar_wait_bounded(b.drain, 0, &none)) pf_report(p.status, abort_flag, DEV_TIMEOUT_DRAIN);
  }
}

// warp 1 of the peer CTA: relays "this CTA's converted tile is ready" to the leader's barrier, one remote arrive per
// K block, so the converter warps themselves only ever signal locally
__device__ __forceinline__ void pf_relay(const PfBars& b, const PfParams& p, int pair_id, int num_pairs,
                                         volatile int* abort_flag, const PfMoe* moe = nullptr) {
  const int num_tiles = p.tiles_m * p.tiles_n;
  const bool leader_lane = elect_one();
  int cstage = 0;
  uint32_t cphase = 0;
  bool ok = true;
  for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
    if (!pf_tile_in_use(moe, p, t)) continue;
    for (int kb = 0; kb < p.k_blocks; ++kb) {
      ok = mbar_wait_bounded(&b.conv_done[cstage], cphase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (leader_lane) pf_report(p.status, abort_flag, DEV_TIMEOUT_MMA);
        break;
      }
      if (leader_lane) mbar_arrive_cluster(map_to_cta(smem_u32(&b.conv_full[cstage]), 0));
      __syncwarp();
      if (++cstage == kPfConvStages) { cstage = 0; cphase ^= 1; }
    }
  }
}

// converter warps of both CTAs: raw bytes of a K block -> exact 16-bit integers in the K-major 128-byte-swizzled
// operand tile.  The warps form TEAMS teams of CT threads (ct = 0..CT-1 within a team); the K blocks go to the teams
// in turn, so a team has TEAMS blocks' time for one block's conversion and its fixed cost (two barrier waits, the
// proxy fence, the arrive), which is what sets the pace when a block is short.
template <typename T, int BITS, int BN = kTN, int CT = 128, int TEAMS = 1>
__device__ __forceinline__ void pf_converters(uint8_t* smem, const PfBars& b, const PfParams& p, uint32_t rank, int pair_id,
                                              int num_pairs, int ct, volatile int* abort_flag, int team = 0,
                                              const PfMoe* moe = nullptr) {
  using L = PfSmem<BITS>;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int lane = ct & 31;
  int stage = 0, cstage = 0, turn = 0;  // ring positions of the current K block; whose turn it is
  uint32_t phase = 0, cphase = 0;
  bool ok = true;
  auto advance = [&]() {
    if (++stage == kPfStages) { stage = 0; phase ^= 1; }
    if (++cstage == kPfConvStages) { cstage = 0; cphase ^= 1; }
    if (++turn == TEAMS) turn = 0;
  };
  for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
    if (!pf_tile_in_use(moe, p, t)) continue;
    for (int kb = 0; kb < p.k_blocks; ++kb, advance()) {
      if (TEAMS > 1 && turn != team) continue;
      ok = mbar_wait_bounded(&b.conv_empty[cstage], cphase ^ 1, abort_flag) &&
           mbar_wait_bounded(&b.raw_full[stage], phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) pf_report(p.status, abort_flag, DEV_TIMEOUT_EPILOGUE);
        break;
      }
      uint8_t* sw = smem + L::kConvOff + cstage * L::kWBytes;           // converted tile: 128 rows x 128 B, swizzled
      const uint8_t* raw = smem + stage * L::kStageBytes + L::kXBytes;  // raw tile: rows of 64 B, not swizzled
      if (BITS == 8) {
        // 128 rows x 4 chunks of 16 bytes; chunk id -> (row = id / 4, c = id % 4): 16 k -> 32 bytes out
#pragma unroll
        for (int id = ct; id < 512; id += CT) {
          const uint32_t row = id >> 2, c = id & 3;
          if (BN < kTN && row >= BN / 2) continue;  // a narrower tile brings fewer weight rows
          const uint4 w = *reinterpret_cast<const uint4*>(raw + id * 16);
          uint4 o0, o1;
          cvt_int8x4<T>(w.x, o0.x, o0.y);
          cvt_int8x4<T>(w.y, o0.z, o0.w);
          cvt_int8x4<T>(w.z, o1.x, o1.y);
          cvt_int8x4<T>(w.w, o1.z, o1.w);
          *reinterpret_cast<uint4*>(sw + sw128(row, 2 * c)) = o0;
          *reinterpret_cast<uint4*>(sw + sw128(row, 2 * c + 1)) = o1;
        }
      } else {
        // 64 packed rows x 4 chunks; packed row j carries channel rows 2j (low nibbles) and 2j+1 (high)
#pragma unroll
        for (int id = ct; id < 256; id += CT) {
          const uint32_t prow = id >> 2, c = id & 3;
          if (BN < kTN && prow >= BN / 4) continue;
          const uint4 w = *reinterpret_cast<const uint4*>(raw + id * 16);
          uint4 l0, l1, h0, h1;
          cvt_int4x8<T>(w.x, l0.x, l0.y, h0.x, h0.y);
          cvt_int4x8<T>(w.y, l0.z, l0.w, h0.z, h0.w);
          cvt_int4x8<T>(w.z, l1.x, l1.y, h1.x, h1.y);
          cvt_int4x8<T>(w.w, l1.z, l1.w, h1.z, h1.w);
          *reinterpret_cast<uint4*>(sw + sw128(2 * prow, 2 * c)) = l0;
          *reinterpret_cast<uint4*>(sw + sw128(2 * prow, 2 * c + 1)) = l1;
          *reinterpret_cast<uint4*>(sw + sw128(2 * prow + 1, 2 * c)) = h0;
          *reinterpret_cast<uint4*>(sw + sw128(2 * prow + 1, 2 * c + 1)) = h1;
        }
      }
      fence_proxy_async_smem();  // the tensor core reads these bytes through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(rank == 0 ? &b.conv_full[cstage] : &b.conv_done[cstage]);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Per-channel scales: sixteen warps (TMA, MMA, two idle, four epilogue, eight converters); the accumulator of a tile is read
// once, out = acc * s[n] - xsum[m] * s[n] zp[n] + bias[n].
// ---------------------------------------------------------------------------------------------------------
// BN: channels per pair tile (256, or narrower where that fills the last wave better; the shared-memory and TMEM
// layout stays that of 256, a narrower tile simply uses fewer rows / columns of it).
template <typename T, int BITS, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPfThreads, 1)
wo_umma_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                    const PfParams p, const __grid_constant__ PfMoe moe) {
  using L = PfSmem<BITS>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* vec_smem = reinterpret_cast<float*>(smem + L::kVecOff);
  const PfBars b = pf_bars(reinterpret_cast<uint64_t*>(smem + L::kBarOff));
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
    pf_init_bars(b, 8, false, kPfConvWarps / pf_conv_teams<BITS>());
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

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      if (p.moe) pf_producer<BITS, BN, true>(smem, b, &tmap_x, &tmap_w, p, rank, pair_id, num_pairs, abort_flag, &moe);
      else pf_producer<BITS, BN, false>(smem, b, &tmap_x, &tmap_w, p, rank, pair_id, num_pairs, abort_flag);
    } else if (warp == 1) {
      const PfMoe* in_use = p.moe ? &moe : nullptr;
      if (rank == 0) pf_mma<T, BITS, BN>(smem, b, p, tmem_base, pair_id, num_pairs, p.k_blocks, abort_flag, in_use);
      else pf_relay(b, p, pair_id, num_pairs, abort_flag, in_use);
    }
  } else if (warp < 8) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    // -------------------------------- epilogue (both CTAs) --------------------------------
    const int quarter = warp & 3;
    float* cs = vec_smem + quarter * 3 * kTN;  // scale, scale*zp, bias of this tile's channels (private copy)
    float* cz = cs + kTN;
    float* cb = cz + kTN;
    T* out = reinterpret_cast<T*>(p.out);
    const bool vec_ok = (p.ldo % 8 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0);
    int local = 0;
    bool ok = true;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
      int mb, nb;
      pf_tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
      const int expert = p.moe ? pf_moe_expert(moe, mb) : 0;
      if (expert < 0) continue;  // fused MoE: a row tile past the slots in use
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ++local;
      const int row = mb * 256 + int(rank) * kTM + quarter * 32 + lane;
      const int n0 = nb * BN;
      const int64_t sbase = int64_t(expert < 0 ? 0 : expert) * p.N;  // fused MoE: the expert's scales
      for (int j = lane; j < BN; j += 32) {
        const bool in = n0 + j < p.N && expert >= 0;
        const float s = in ? load_as_f32(p.scale, p.scale_dtype, sbase + n0 + j) : 0.f;
        cs[j] = s;
        cz[j] = (in && p.zp) ? s * load_as_f32(p.zp, p.scale_dtype, sbase + n0 + j) : 0.f;
        cb[j] = (in && p.bias) ? load_as_f32(p.bias, p.bias_dtype, n0 + j) : 0.f;
      }
      const float xs = (p.zp && row < p.M) ? p.xsum[row] : 0.f;
      // where this thread's row goes: its own row, or (fused MoE) the flat (token, choice) index of its slot
      int64_t out_row = row < p.M ? row : -1;
      float rw = 1.f;
      if (p.moe) {
        out_row = -1;
        if (expert >= 0) {
          const int flat = __ldg(moe.sorted_ids + row);
          if (flat >= 0 && flat < moe.num_valid) {
            out_row = flat;
            if (moe.mul_w) rw = load_as_f32(moe.topk_w, moe.topk_dtype, flat);
          }
        }
      }
      __syncwarp();

      ok = mbar_wait_bounded(&b.tmem_full[buf], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) pf_report(p.status, abort_flag, DEV_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * kTN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tc_wait_ld();
        const int col0 = n0 + c * 32;
        if (out_row >= 0 && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = rw * fmaf(__uint_as_float(r[j]), cs[c * 32 + j], fmaf(-xs, cz[c * 32 + j], cb[c * 32 + j]));
          T* orow = out + out_row * p.ldo + col0;
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
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&b.tmem_empty[buf]), 0));
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kPfConvRegs));
    constexpr int kTeamThreads = kPfConvWarps * 32 / pf_conv_teams<BITS>();
    pf_converters<T, BITS, BN, kTeamThreads, pf_conv_teams<BITS>()>(smem, b, p, rank, pair_id, num_pairs,
                                                           (threadIdx.x - 8 * 32) % kTeamThreads, abort_flag,
                                                           (threadIdx.x - 8 * 32) / kTeamThreads, p.moe ? &moe : nullptr);
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

// ---------------------------------------------------------------------------------------------------------
// Group-wise scales, exact in fp32.  The converted weight is the bare integer; the MMA warp gives every scale group
// (group / 64 K blocks) an accumulator of its own in one of the two TMEM buffers, and the epilogue warps promote it
// while the next group accumulates in the other buffer:
//     total[m, n] += s[g, n] * acc_g[m, n] - (s[g, n] zp[g, n]) * xsum_g[m]        (fp32 registers)
// so w * s is never rounded to 16 bits and the result differs from the fp32 dequant-matmul only by the order of
// fp32 additions.  A thread owns one token row and 128 channels (128 running sums), so the CTA needs eight
// epilogue warps (two per TMEM lane quarter, one per column half) and more registers per epilogue thread than an
// even split of the register file gives: sixteen warps, and the warpgroups re-balance their registers at the start
// (producer/MMA warpgroup 40, converter warpgroup 56, the two epilogue warpgroups 208 each: 512 x 128 in all).
//   warps 0-3   TMA producer, MMA issuer / relay, two idle        warps 4-7   converters
//   warps 8-15  epilogue: quarter = warp % 4, column half = (warp - 8) / 4
// Per group the 256 epilogue threads stage that group's 256 scales (and s * zp) as fp32 in shared memory, double
// buffered, handing over through an mbarrier per buffer and column half (every wait in this kernel is bounded).
// ---------------------------------------------------------------------------------------------------------
constexpr int kPgThreads = 512;

__device__ __forceinline__ void ffma2(uint64_t& d, uint32_t a0, uint32_t a1, float b0, float b1) {
  uint64_t a, b;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "r"(a0), "r"(a1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(b0), "f"(b1));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// BN: channels per pair tile, 256 or 128; the 512 TMEM columns hold NBUF = 512 / BN accumulators, so that many scale
// groups are in flight between the MMA warp and the epilogue warps.
template <typename T, int BITS, bool HAS_ZP, int BN, bool MOE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPgThreads, 1)
wo_umma_pair_group_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                          const PfParams p, const __grid_constant__ PfMoe moe) {
  using L = PfSmem<BITS>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* vec_smem = reinterpret_cast<float*>(smem + L::kVecOff);
  const PfBars b = pf_bars(reinterpret_cast<uint64_t*>(smem + L::kBarOff));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlotOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;
  constexpr uint32_t kTmemCols = 512;
  constexpr int NBUF = 512 / BN;
  constexpr int HC = BN / 2;  // columns of a tile that one epilogue thread folds (one column half)

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    pf_init_bars(b, 16, true, 4 / kPgConvTeams);
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
  const int kb_per_group = p.group / kTK;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      pf_producer<BITS, BN, MOE>(smem, b, &tmap_x, &tmap_w, p, rank, pair_id, num_pairs, abort_flag, &moe);
    } else if (warp == 1) {
      if (rank == 0) pf_mma<T, BITS, BN, NBUF, BN>(smem, b, p, tmem_base, pair_id, num_pairs, kb_per_group, abort_flag, MOE ? &moe : nullptr);
      else pf_relay(b, p, pair_id, num_pairs, abort_flag, MOE ? &moe : nullptr);
    } else {
      // ---- warps 2 and 3: stage the scales (and scale * zero-point, and with a tile's first group its bias) of the
      // coming groups as fp32 in a ring of kPgScaleStages slots, one column half each, CPL columns per lane, so that
      // the epilogue warps find them ready
      constexpr int CPL = HC / 32;
      const int half = warp - 2;
      const int c0 = half * HC + lane * CPL;
      float* sS = vec_smem;
      float* sZ = sS + kPgScaleStages * kTN;
      float* sB = sZ + kPgScaleStages * kTN;
      const int groups = p.K / p.group;
      int seg = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        int mb, nb;
        pf_tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
        const int n0 = nb * BN + c0;
        const int expert = MOE ? pf_moe_expert(moe, mb) : 0;
        if (expert < 0) continue;
        for (int g = 0; g < groups; ++g, ++seg) {
          const int slot = seg % kPgScaleStages;
          const uint32_t ph = (seg / kPgScaleStages) & 1;
          float sv[CPL], zv[CPL], bv[CPL];
#pragma unroll
          for (int j = 0; j < CPL; ++j) {
            const bool in = n0 + j < p.N && expert >= 0;
            // dense: [K / group, N]; fused MoE: [E, N, K / group]
            const int64_t at = MOE ? (int64_t(expert) * p.N + n0 + j) * groups + g : int64_t(g) * p.N + n0 + j;
            sv[j] = in ? load_as_f32(p.scale, p.scale_dtype, at) : 0.f;
            zv[j] = (HAS_ZP && in) ? sv[j] * load_as_f32(p.zp, p.scale_dtype, at) : 0.f;
            bv[j] = (g == 0 && p.bias && in) ? load_as_f32(p.bias, p.bias_dtype, n0 + j) : 0.f;
          }
          ok = mbar_wait_bounded(&b.scale_empty[slot], ph ^ 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (lane == 0) pf_report(p.status, abort_flag, DEV_TIMEOUT_PRODUCER);
            break;
          }
#pragma unroll
          for (int j = 0; j < CPL; ++j) {
            sS[slot * kTN + c0 + j] = sv[j];
            if (HAS_ZP) sZ[slot * kTN + c0 + j] = zv[j];
            if (g == 0) sB[slot * kTN + c0 + j] = bv[j];
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&b.scale_full[slot]);
        }
      }
    }
  } else if (warp < 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    pf_converters<T, BITS, BN, 128 / kPgConvTeams, kPgConvTeams>(smem, b, p, rank, pair_id, num_pairs,
                                                                 (threadIdx.x - 4 * 32) % (128 / kPgConvTeams), abort_flag,
                                                                 (threadIdx.x - 4 * 32) / (128 / kPgConvTeams), MOE ? &moe : nullptr);
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    // -------------------------------- epilogue (both CTAs) --------------------------------
    const int quarter = warp & 3;
    const int half = (warp - 8) >> 2;
    const float* sS = vec_smem;                       // [kPgScaleStages][kTN] scale of a group
    const float* sZ = sS + kPgScaleStages * kTN;      // scale * zero-point
    const float* sB = sZ + kPgScaleStages * kTN;      // bias, valid in the slot of a tile's first group
    T* out = reinterpret_cast<T*>(p.out);
    const bool vec_ok = (p.ldo % 8 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0);
    const int groups = p.K / p.group;
    uint64_t sum2[HC / 2];
#pragma unroll
    for (int i = 0; i < HC / 2; ++i) sum2[i] = 0ull;
    int seg = 0, local = 0;
    bool ok = true;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs, ++local) {
      int mb, nb;
      pf_tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
      const int row = mb * 256 + int(rank) * kTM + quarter * 32 + lane;
      const int n0 = nb * BN;
      // fused MoE: the flat (token, choice) index this thread's slot writes (-1: none) and its routing weight
      int moe_row = -1;
      float rw = 1.f;
      if (MOE) {
        if (pf_moe_expert(moe, mb) < 0) continue;  // a row tile past the slots in use
        const int flat = __ldg(moe.sorted_ids + row);
        if (flat >= 0 && flat < moe.num_valid) {
          moe_row = flat;
          if (moe.mul_w) rw = load_as_f32(moe.topk_w, moe.topk_dtype, flat);
        }
      }
      for (int g = 0; g < groups; ++g, ++seg) {
        const int buf = seg % NBUF;
        const uint32_t seg_phase = (seg / NBUF) & 1;
        const int slot = seg % kPgScaleStages;
        const uint32_t slot_phase = (seg / kPgScaleStages) & 1;
        float nxg = 0.f;
        if (HAS_ZP && row < p.M) nxg = -p.xsum[int64_t(g) * p.M + row];
        ok = mbar_wait_bounded(&b.scale_full[slot], slot_phase, abort_flag) &&
             mbar_wait_bounded(&b.tmem_full[buf], seg_phase, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) pf_report(p.status, abort_flag, DEV_TIMEOUT_EPILOGUE);
          break;
        }
        if (g == 0) {  // the sums of a tile start from its bias (they were left at zero)
          const float4* b4 = reinterpret_cast<const float4*>(sB + slot * kTN + half * HC);
#pragma unroll
          for (int i = 0; i < HC / 4; ++i) {
            const float4 bv = b4[i];
            asm("mov.b64 %0, {%1, %2};" : "=l"(sum2[2 * i]) : "f"(bv.x), "f"(bv.y));
            asm("mov.b64 %0, {%1, %2};" : "=l"(sum2[2 * i + 1]) : "f"(bv.z), "f"(bv.w));
          }
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * BN + half * HC;
        const float4* s4 = reinterpret_cast<const float4*>(sS + slot * kTN + half * HC);
        const float4* z4 = reinterpret_cast<const float4*>(sZ + slot * kTN + half * HC);
#pragma unroll
        for (int c = 0; c < HC / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 sv = s4[(c * 32 + j) >> 2];
            ffma2(sum2[(c * 32 + j) >> 1], r[j], r[j + 1], sv.x, sv.y);
            ffma2(sum2[((c * 32 + j) >> 1) + 1], r[j + 2], r[j + 3], sv.z, sv.w);
            if (HAS_ZP) {
              const float4 zv = z4[(c * 32 + j) >> 2];
              const uint32_t nx = __float_as_uint(nxg);
              ffma2(sum2[(c * 32 + j) >> 1], nx, nx, zv.x, zv.y);
              ffma2(sum2[((c * 32 + j) >> 1) + 1], nx, nx, zv.z, zv.w);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_cluster(map_to_cta(smem_u32(&b.tmem_empty[buf]), 0));
          mbar_arrive(&b.scale_empty[slot]);
        }
      }
      if (!ok) break;
      // the tile's sums are complete: round once, store, and clear the sums for the next tile
      const bool row_ok = MOE ? moe_row >= 0 : row < p.M;
      T* orow0 = out + int64_t(MOE ? (moe_row < 0 ? 0 : moe_row) : row) * p.ldo + n0 + half * HC;
#pragma unroll
      for (int c = 0; c < HC / 32; ++c) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          unpack2(sum2[(c * 32 + j) >> 1], v[j], v[j + 1]);
          if (MOE) {
            v[j] *= rw;
            v[j + 1] *= rw;
          }
          sum2[(c * 32 + j) >> 1] = 0ull;
        }
        const int col0 = n0 + half * HC + c * 32;
        if (row_ok && col0 < p.N) {
          T* orow = orow0 + c * 32;
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

// xsum[g, m] = sum of x[m, k] over the k of scale group g, in fp32; one warp per row, group after group
template <typename T>
__global__ void row_group_sum_kernel(const T* __restrict__ act, int64_t lda, float* __restrict__ xsum, int M, int K,
                                     int group) {
  const int64_t row = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const T* x = act + row * lda;
  for (int g = 0; g * group < K; ++g) {
    float s = 0.f;
    for (int i = lane; i < group; i += 32) s += to_f32(x[g * group + i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) xsum[int64_t(g) * M + row] = s;
  }
}

template <typename KernT>
int pf_configure(KernT kern, int bytes, cudaError_t (&attr_err)[64], std::once_flag (&once)[64]) {
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::call_once(once[dev], [&] { attr_err[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); });
  return attr_err[dev] == cudaSuccess ? FNN_OK : check_cuda(attr_err[dev], "cudaFuncSetAttribute(weight-only prefill)");
}

// Tile width of the per-channel kernel: waves x width x a small per-width cost (a narrower tile re-reads the
// activation rows for fewer channels); ties keep the wider tile.
inline int pf_pick_bn(int M, int N, int pairs) {
  const int widths[3] = {256, 224, 192};
  const double cost_of[3] = {1.0, 1.03, 1.06};
  const int tiles_m = (M + 255) / 256;
  int best = 256;
  double best_cost = 1e30;
  for (int i = 0; i < 3; ++i) {
    const long long tiles = 1ll * tiles_m * ((N + widths[i] - 1) / widths[i]);
    const double cost = double((tiles + pairs - 1) / pairs) * widths[i] * cost_of[i];
    if (cost < best_cost) { best_cost = cost; best = widths[i]; }
  }
  return best;
}

template <typename T, int BITS, int BN>
int launch_prefill_perch(const T* act, int64_t lda, const uint8_t* qw, PfParams p, const PfMoe& moe, cudaStream_t st) {
  using L = PfSmem<BITS>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];  // per device, so that a failure is reported on every call and not only the first
  if (int e = pf_configure(wo_umma_pair_kernel<T, BITS, BN>, L::kDynamicBytes, attr_err, once)) return e;
  CUtensorMap tx, tw;
  if (int e = make_tmap_2d(&tx, 2, act, p.M, p.K, lda * 2, kTK, kTM, true)) return e;
  const int64_t w_rows = int64_t((BITS == 8) ? p.N : p.N / 2) * (p.moe ? moe.num_experts : 1);
  if (int e = make_tmap_2d(&tw, 1, qw, w_rows, p.K, p.K, kTK, (BITS == 8) ? BN / 2 : BN / 4, false)) return e;
  p.tiles_m = (p.M + 255) / 256;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.k_blocks = (p.K + kTK - 1) / kTK;
  const int tiles = p.tiles_m * p.tiles_n;
  const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  wo_umma_pair_kernel<T, BITS, BN><<<2 * pairs, kPfThreads, L::kDynamicBytes, st>>>(tx, tw, p, moe);
  return check_cuda(cudaGetLastError(), "weight-only prefill launch");
}

// Tile width of the group-wise kernel.  128-wide tiles would keep four accumulators in flight instead of two, which
// hides the hand-over of a group's accumulator, but a K block of a 128-wide tile gives the four converter warps half
// the time for the same per-block barrier round: measured 676 against 865 TFLOP/s (A16W4, group 128, 2048 x 28672 x 8192).
constexpr int kPgTile = 256;

template <typename T, int BITS, bool HAS_ZP, int BN, bool MOE>
int launch_prefill_group(const T* act, int64_t lda, const uint8_t* qw, PfParams p, const PfMoe& moe, cudaStream_t st) {
  using L = PfSmem<BITS>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];  // per device, so that a failure is reported on every call and not only the first
  if (int e = pf_configure(wo_umma_pair_group_kernel<T, BITS, HAS_ZP, BN, MOE>, L::kDynamicBytes, attr_err, once)) return e;
  CUtensorMap tx, tw;
  if (int e = make_tmap_2d(&tx, 2, act, p.M, p.K, lda * 2, kTK, kTM, true)) return e;
  const int64_t w_rows = int64_t((BITS == 8) ? p.N : p.N / 2) * (p.moe ? moe.num_experts : 1);
  if (int e = make_tmap_2d(&tw, 1, qw, w_rows, p.K, p.K, kTK, (BITS == 8) ? BN / 2 : BN / 4, false)) return e;
  p.tiles_m = (p.M + 255) / 256;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.k_blocks = (p.K + kTK - 1) / kTK;
  const int tiles = p.tiles_m * p.tiles_n;
  const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  wo_umma_pair_group_kernel<T, BITS, HAS_ZP, BN, MOE><<<2 * pairs, kPgThreads, L::kDynamicBytes, st>>>(tx, tw, p, moe);
  return check_cuda(cudaGetLastError(), "weight-only prefill launch");
}

template <typename T, int BITS>
int launch_prefill(const T* act, int64_t lda, const uint8_t* qw, PfParams p, float* xsum_ws, cudaStream_t st,
                   const PfMoe& moe = PfMoe{}) {
  using L = PfSmem<BITS>;
  static_assert(L::kDynamicBytes <= 227 * 1024, "shared memory budget");
  static_assert(L::kStageBytes % 1024 == 0 && L::kWBytes % 1024 == 0 && L::kConvOff % 1024 == 0, "tile alignment");
  if (p.zp) {
    const unsigned blocks = unsigned((int64_t(p.M) * 32 + 255) / 256);
    if (p.group == 0) row_sum_kernel<T><<<blocks, 256, 0, st>>>(act, lda, xsum_ws, p.M, p.K);
    else row_group_sum_kernel<T><<<blocks, 256, 0, st>>>(act, lda, xsum_ws, p.M, p.K, p.group);
    if (int e = check_cuda(cudaGetLastError(), "row_sum launch")) return e;
    p.xsum = xsum_ws;
  }
  if (p.group == 0) {
    switch (pf_pick_bn(p.M, p.N, sm_count() / 2)) {
      case 224: return launch_prefill_perch<T, BITS, 224>(act, lda, qw, p, moe, st);
      case 192: return launch_prefill_perch<T, BITS, 192>(act, lda, qw, p, moe, st);
      default: return launch_prefill_perch<T, BITS, 256>(act, lda, qw, p, moe, st);
    }
  }
  if (BITS == 4 && p.moe) {  // fused MoE exists for packed int4 only
    if (p.zp) return launch_prefill_group<T, 4, true, kPgTile, true>(act, lda, qw, p, moe, st);
    return launch_prefill_group<T, 4, false, kPgTile, true>(act, lda, qw, p, moe, st);
  }
  if (p.zp) return launch_prefill_group<T, BITS, true, kPgTile, false>(act, lda, qw, p, moe, st);
  return launch_prefill_group<T, BITS, false, kPgTile, false>(act, lda, qw, p, moe, st);
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
  if (zp) {
    const size_t need = size_t(M) * sizeof(float) * (group == 0 ? 1 : size_t(K / group));
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

// Copies 16-bit token rows into expert-sorted order: slot s gets row sorted_ids[s] / top_k of A; slots that name no
// token get zeros, slots past the ones in use are left alone.  One warp per slot, 16 bytes per lane and step.
__global__ void moe_gather_rows16_kernel(const uint16_t* __restrict__ a, int64_t lda, const int32_t* __restrict__ sorted_ids,
                                         const int32_t* __restrict__ npp, int num_valid, int top_k,
                                         uint16_t* __restrict__ a_sorted, int K, int EM) {
  const int slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (slot >= EM || slot >= __ldg(npp)) return;
  const int lane = threadIdx.x & 31;
  const int flat = __ldg(sorted_ids + slot);
  const bool valid = flat >= 0 && flat < num_valid;
  const uint4* src = reinterpret_cast<const uint4*>(a + int64_t(valid ? flat / top_k : 0) * lda);
  uint4* dst = reinterpret_cast<uint4*>(a_sorted + int64_t(slot) * K);
  for (int i = lane; i < K / 8; i += 32) dst[i] = valid ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
}

size_t weight_only_moe_prefill_workspace(int64_t EM, int64_t K, int64_t group, bool zp) {
  size_t bytes = (size_t(EM) * size_t(K) * 2 + 255) / 256 * 256;
  if (zp) bytes += (size_t(EM) * sizeof(float) * (group > 0 ? size_t(K / group) : 1) + 255) / 256 * 256;
  return bytes;
}

// Fused MoE with packed-int4 expert weights on the prefill kernels: blocks of 256 sorted slots (or a multiple).
// Returns -1 when the operands are outside what these kernels take (the caller then runs its own kernel).
int weight_only_moe_prefill(const void* a, int a_dtype, int64_t lda, const void* b, int E, int N, int K, const void* scale,
                            const void* zp, int scale_dtype, int group, const void* topk_w, int topk_dtype,
                            const int32_t* sorted_ids, int EM, const int32_t* expert_ids, const int32_t* npp, int num_valid,
                            int top_k, int block_m, int mul_w, void* out, int64_t ldo, void* workspace,
                            size_t workspace_bytes, cudaStream_t st) {
  if (block_m % 256 != 0 || EM % 256 != 0) return -1;
  if (group > 0 && (group % kTK != 0 || K % group != 0)) return -1;
  if (K % 16 != 0 || N % 2 != 0 || reinterpret_cast<uintptr_t>(b) % 16 != 0 || reinterpret_cast<uintptr_t>(a) % 16 != 0 || lda % 8 != 0)
    return -1;
  if (int64_t(E) * (N / 2) > INT32_MAX) return -1;
  const size_t need = weight_only_moe_prefill_workspace(EM, K, group, zp != nullptr);
  if (!workspace || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return -1;
  uint16_t* a_sorted = static_cast<uint16_t*>(workspace);
  float* xsum = zp ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + (size_t(EM) * size_t(K) * 2 + 255) / 256 * 256) : nullptr;
  moe_gather_rows16_kernel<<<unsigned((EM + 7) / 8), 256, 0, st>>>(static_cast<const uint16_t*>(a), lda, sorted_ids, npp, num_valid,
                                                                   top_k, a_sorted, K, EM);
  if (int e = check_cuda(cudaGetLastError(), "fused moe a16w4 gather launch")) return e;
  PfParams p{};
  p.scale = scale; p.zp = zp; p.bias = nullptr; p.xsum = nullptr; p.out = out; p.ldo = ldo;
  p.scale_dtype = scale_dtype; p.bias_dtype = FNN_F32; p.M = EM; p.N = N; p.K = K; p.group = group;
  p.status = device_status_word();
  p.moe = 1;
  PfMoe moe{};
  moe.num_experts = E; moe.top_k = top_k; moe.num_valid = num_valid; moe.mul_w = mul_w; moe.block_m = block_m;
  moe.topk_dtype = topk_dtype; moe.sorted_ids = sorted_ids; moe.expert_ids = expert_ids; moe.npp = npp; moe.topk_w = topk_w;
  const uint8_t* qw = static_cast<const uint8_t*>(b);
  if (a_dtype == FNN_F16)
    return launch_prefill<__half, 4>(reinterpret_cast<const __half*>(a_sorted), K, qw, p, xsum, st, moe);
  return launch_prefill<__nv_bfloat16, 4>(reinterpret_cast<const __nv_bfloat16*>(a_sorted), K, qw, p, xsum, st, moe);
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
