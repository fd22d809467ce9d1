// A8W8 GEMM for sm_100a: int8 x int8 -> int32 on the 5th-generation tensor
// cores (tcgen05.mma kind::i8), operands staged by TMA, accumulators in TMEM,
// per-token x per-channel scaling fused into the epilogue.
//
// One persistent CTA per SM, six warps:
//   warp 0      TMA producer   (one elected lane issues the bulk tensor loads)
//   warp 1      MMA issuer     (one elected lane issues tcgen05.mma / commit; owns TMEM)
//   warps 2-5   epilogue       (tcgen05.ld -> scale -> 16-bit store), one TMEM lane
//                               quarter each (quarter = warp id % 4)
// Shared memory holds a STAGES-deep ring of {A 128x128 B, B BNx128 B} tiles in
// the 128-byte-swizzled K-major layout that both the TMA tensor map and the
// UMMA shared-memory descriptor name.  TMEM holds two BN-column accumulators so
// the epilogue of tile i overlaps the main loop of tile i+1.
//
// Every wait is bounded: a role that runs out of time records a code in the
// device status word, raises the CTA's abort flag, and all roles fall through to
// a common teardown that drains outstanding copies and MMAs and frees TMEM.
#include <atomic>
#include <chrono>
#include <mutex>

#include <type_traits>

#include "a8w8_plan.h"
#include "common.cuh"
#include "weight_only.cuh"

namespace fnn {
namespace {

constexpr int kBM = 128;       // rows of A per tile (UMMA M)
constexpr int kBK = 128;       // K bytes per stage = one 128-byte swizzle row
constexpr int kUmmaK = 32;     // K per tcgen05.mma for 8-bit operands
constexpr int kThreads = 192;  // 6 warps
// tiles along M that share a wave (L2 reuse of B); measured on the CTA-pair kernel: 8 is 2.5 % slower on the FFN
// gate/up projection and 8192^3, 4 is 8 % slower, 32 is 10 % slower
constexpr int kGroupM = 16;

struct A8W8Params {
  const void* alpha_row;
  const void* alpha_col;
  void* out;
  int32_t* acc_out;
  int64_t ldo, ldacc;
  int row_dtype, col_dtype;
  int M, N, K;
  int tiles_m, tiles_n, k_blocks;
  int* status;  // device status word
  int out_tma;  // CTA-pair kernel: the output goes through shared memory and TMA stores (out and its pitch are 16-byte aligned)
  unsigned long long wait_ns;  // longest time one wait may take (single-CTA kernel; kWaitLimitNs unless a test shortened it)
  int skip_kb;                 // -1, or (test hook) the K block of a CTA's first tile whose loads are left out
  // Fused-MoE mode (kernel template flag MOE): A is the expert-sorted copy of the token rows [EM, K], B is the
  // stack of expert weights seen as [E * N, K]; a tile is `tile_rows` sorted slots of one expert x BN channels.
  const int32_t* sorted_ids;       // [EM] flat (token * top_k + choice) index per slot, >= num_valid for padding
  const int32_t* expert_ids;       // [EM / block_m] expert of each block of block_m slots
  const int32_t* num_post_padded;  // [1] slots in use (a multiple of block_m)
  const void* topk_w;              // [num_valid] routing weights
  int topk_w_dtype, top_k, block_m, tile_rows, num_valid, mul_w;
  int64_t col_stride_e;            // elements between two experts' rows of alpha_col
  // K-balanced mode of the CTA-pair kernel (template flag SK): the sk_tiles tiles of the ragged round are shared.
  // Pair i < sk_tiles computes K blocks [0, sk_units) of tile i; the other pairs share the tails [sk_units, k_blocks)
  // evenly (sk_tail_units consecutive blocks of the concatenated tails each), leave the int32 partial sums of each
  // piece in a slot of sk_partials and raise the slot's flags to sk_epoch; the pair that holds a tile's head adds them.
  unsigned long long* sk_flags;    // [slots][8] one word per epilogue warp of a pair
  int32_t* sk_partials;            // [slots][256 * 256]
  unsigned long long sk_epoch;     // never 0, different for every launch
  int sk_tiles, sk_units, sk_tail_units, sk_slots;  // sk_slots: slots reserved per tail-sharing pair
};

// AROWS: rows of A one stage holds (16, 32, 64 or 128).  Decode shapes are bound by the weight stream, and what
// bounds that is the bytes a CTA keeps in flight, so their stages carry only the rows of A that exist and there are
// more of them.  The tensor core still reads 128 rows from the A base (what lies behind the real rows belongs to the
// following buffers; the accumulator rows it produces are never stored), so the last stage is followed by padding.
template <int BN, int STAGES, int AROWS = kBM> struct SmemLayout {
  static constexpr int kABytes = AROWS * kBK;
  static constexpr int kBBytes = BN * kBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTailPad = (kBM * kBK > kStageBytes) ? kBM * kBK - kStageBytes : 0;
  static constexpr int kColScaleOff = STAGES * kStageBytes + kTailPad;  // [4][BN] float
  static constexpr int kBarOff = kColScaleOff + 4 * BN * 4;          // barriers
  static constexpr int kNumBars = 2 * STAGES + 4 + 1;                // full, empty, tmem full/empty x2, drain
  static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
  static constexpr int kAbortOff = kTmemSlotOff + 8;
  static constexpr int kTotal = kAbortOff + 8;
  static constexpr int kDynamicBytes = kTotal + 1024;  // slack for manual 1024-byte alignment
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
  const int group_sz = kGroupM * tiles_n;
  const int gid = t / group_sz;
  const int first_m = gid * kGroupM;
  const int gm = min(tiles_m - first_m, kGroupM);
  const int r = t - gid * group_sz;
  mb = first_m + r % gm;
  nb = r / gm;
}

__device__ __forceinline__ void report(int* status, volatile int* abort_flag, int code) {
  *abort_flag = code;
  if (status) atomicCAS(status, 0, code);
}

// Epilogue of 32 accumulator columns of one output row: optional raw int32 copy, then
// out = fl32(float(acc) * s) with s = row scale * column scale (rounded to the scales' dtype when
// both scales share a 16-bit dtype), rounded once to OutT.
__device__ __forceinline__ void store_acc_chunk(const uint32_t (&r)[32], int row, int col0, const A8W8Params& p,
                                                bool acc_vec_ok) {
  if (!p.acc_out || row >= p.M || col0 >= p.N) return;
  int32_t* arow = p.acc_out + int64_t(row) * p.ldacc + col0;
  if (col0 + 32 <= p.N && acc_vec_ok) {
#pragma unroll
    for (int j = 0; j < 32; j += 4)
      *reinterpret_cast<uint4*>(arow + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.N) arow[j] = int32_t(r[j]);
  }
}

// s = fl32(row scale * column scale) (rounded to the scales' dtype when both share a 16-bit one), v = fl32(acc * s):
// four column scales per shared-memory read, two products per packed fp32 multiply
__device__ __forceinline__ void scale_chunk(const uint32_t (&r)[32], float rs, const float* cs, bool same16,
                                            const A8W8Params& p, float (&v)[32]) {
  const uint64_t rs2 = pack_f32x2(rs, rs);
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 c4 = *reinterpret_cast<const float4*>(cs + j);
    float s0, s1, s2, s3;
    unpack_f32x2(fmul2_rn(rs2, pack_f32x2(c4.x, c4.y)), s0, s1);
    unpack_f32x2(fmul2_rn(rs2, pack_f32x2(c4.z, c4.w)), s2, s3);
    if (same16) {
      s0 = round_through(s0, p.row_dtype); s1 = round_through(s1, p.row_dtype);
      s2 = round_through(s2, p.row_dtype); s3 = round_through(s3, p.row_dtype);
    }
    unpack_f32x2(fmul2_rn(pack_f32x2(float(int32_t(r[j])), float(int32_t(r[j + 1]))), pack_f32x2(s0, s1)), v[j], v[j + 1]);
    unpack_f32x2(fmul2_rn(pack_f32x2(float(int32_t(r[j + 2])), float(int32_t(r[j + 3]))), pack_f32x2(s2, s3)), v[j + 2], v[j + 3]);
  }
}

template <typename OutT>
__device__ __forceinline__ void store_chunk(const uint32_t (&r)[32], int row, int col0, float rs, const float* cs,
                                            bool same16, const A8W8Params& p, bool vec_ok, bool acc_vec_ok) {
  if (row >= p.M || col0 >= p.N) return;
  const bool full = col0 + 32 <= p.N;
  store_acc_chunk(r, row, col0, p, acc_vec_ok);
  float v[32];
  scale_chunk(r, rs, cs, same16, p, v);
  OutT* orow = reinterpret_cast<OutT*>(p.out) + int64_t(row) * p.ldo + col0;
  if (full && vec_ok) {
#pragma unroll
    for (int j = 0; j < 32; j += 8)
      *reinterpret_cast<uint4*>(orow + j) =
          make_uint4(pack2<OutT>(v[j], v[j + 1]), pack2<OutT>(v[j + 2], v[j + 3]),
                     pack2<OutT>(v[j + 4], v[j + 5]), pack2<OutT>(v[j + 6], v[j + 7]));
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.N) orow[j] = from_f32<OutT>(v[j]);
  }
}

// Fused-MoE epilogue of 32 accumulator columns of one sorted slot, in the order of the reference kernel
// (flashnn/triton_kernels/fused_moe_a8w8.py:155-170): acc * alpha_row, * alpha_col, * routing weight, cast to fp16,
// then to the output dtype.
template <typename OutT>
__device__ __forceinline__ void store_chunk_moe(const uint32_t (&r)[32], int64_t out_row, int col0, float rs, float rw,
                                                bool mul_w, const float* cs, const A8W8Params& p, bool vec_ok) {
  if (col0 >= p.N) return;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float t = __fmul_rn(__fmul_rn(float(int32_t(r[j])), rs), cs[j]);
    if (mul_w) t = __fmul_rn(t, rw);
    // the reference kernel casts its accumulator to fp16 whatever the output tensor's dtype is
    // (fused_moe_a8w8.py:165) and the store converts again: a bf16 output is rounded twice
    v[j] = std::is_same<OutT, __half>::value ? t : __half2float(__float2half_rn(t));
  }
  OutT* orow = reinterpret_cast<OutT*>(p.out) + out_row * p.ldo + col0;
  if (col0 + 32 <= p.N && vec_ok) {
#pragma unroll
    for (int j = 0; j < 32; j += 8)
      *reinterpret_cast<uint4*>(orow + j) =
          make_uint4(pack2<OutT>(v[j], v[j + 1]), pack2<OutT>(v[j + 2], v[j + 3]),
                     pack2<OutT>(v[j + 4], v[j + 5]), pack2<OutT>(v[j + 6], v[j + 7]));
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.N) orow[j] = from_f32<OutT>(v[j]);
  }
}

template <typename OutT, int BN, int STAGES, bool MOE, int AROWS>
__global__ void __launch_bounds__(kThreads, 1)
a8w8_umma_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const A8W8Params p) {
  using L = SmemLayout<BN, STAGES, AROWS>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* col_scale_smem = reinterpret_cast<float*>(smem + L::kColScaleOff);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full_bar = bars + 2 * STAGES;
  uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2;
  uint64_t* drain_bar = bars + 2 * STAGES + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlotOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  constexpr uint32_t kTmemCols = 2 * BN;
  // fused MoE: row tiles past the slots in use are skipped by every role alike
  const int rows_in_use = MOE ? __ldg(p.num_post_padded) : 0;
  const int tile_rows = MOE ? p.tile_rows : kBM;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 4);
    }
    mbar_init(drain_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    const bool leader = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    long long issued = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int mb, nb;
      tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
      if (MOE && mb * tile_rows >= rows_in_use) continue;
      // fused MoE: the tile's weights are rows [e * N + nb * BN, ...) of the expert stack
      const int b_row = nb * BN + (MOE ? __ldg(p.expert_ids + (mb * tile_rows) / p.block_m) * p.N : 0);
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, p.wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (leader) report(p.status, abort_flag, DEV_TIMEOUT_PRODUCER);
          break;
        }
        if (leader && !(kb == p.skip_kb && t == int(blockIdx.x))) {  // (test hook: one K block's loads left out)
          uint8_t* sa = smem + stage * L::kStageBytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * kBK, mb * tile_rows);
          tma_load_2d(sa + L::kABytes, &tmap_b, &full_bar[stage], kb * kBK, b_row);
          ++issued;
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    // Wait (bounded) until the last copies issued have landed, so that nothing
    // writes this CTA's shared memory after it has exited, even after an abort.
    if (leader) {
      int none = 0;
      const long long first = issued > STAGES ? issued - STAGES : 0;
      for (long long i = first; i < issued; ++i)
        if (!mbar_wait_bounded(&full_bar[i % STAGES], uint32_t((i / STAGES) & 1), &none, p.wait_ns)) {
          report(p.status, abort_flag, DEV_TIMEOUT_DRAIN);
          break;
        }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    const bool leader = elect_one();
    constexpr uint32_t idesc = umma_idesc(/*s32*/ 2, /*signed 8-bit*/ 1, kBM, BN);
    int stage = 0;
    uint32_t phase = 0;
    int local = 0;
    bool ok = true;
    bool issued_any = false;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      if (MOE) {
        int mb, nb;
        tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
        if (mb * tile_rows >= rows_in_use) continue;
      }
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ++local;
      ok = mbar_wait_bounded(&tmem_empty_bar[buf], acc_phase ^ 1, abort_flag, p.wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (leader) report(p.status, abort_flag, DEV_TIMEOUT_MMA);
        break;
      }
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + buf * BN;
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        ok = mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (leader) report(p.status, abort_flag, DEV_TIMEOUT_MMA);
          break;
        }
        tc_fence_after();
        if (leader) {
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_i8(tmem_d, umma_desc_k_sw128(sa + k * kUmmaK), umma_desc_k_sw128(sb + k * kUmmaK),
                    idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs have read it
          issued_any = true;
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (ok && leader) tc_commit(&tmem_full_bar[buf]);  // accumulator complete
      __syncwarp();
    }
    // Wait (bounded) for every MMA issued before TMEM is freed, even after an abort.
    if (leader && issued_any) {
      int none = 0;
      tc_commit(drain_bar);
      if (!mbar_wait_bounded(drain_bar, 0, &none, p.wait_ns)) report(p.status, abort_flag, DEV_TIMEOUT_DRAIN);
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quarter = warp & 3;
    float* cs = col_scale_smem + quarter * BN;  // this warp's private copy
    const bool same16 = (p.row_dtype == p.col_dtype) && (p.row_dtype != FNN_F32);
    const bool vec_ok = (p.ldo % 8 == 0) && (reinterpret_cast<uintptr_t>(p.out) % 16 == 0);
    const bool acc_vec_ok = p.acc_out && (p.ldacc % 4 == 0) && (reinterpret_cast<uintptr_t>(p.acc_out) % 16 == 0);
    int local = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int mb, nb;
      tile_coords(t, p.tiles_m, p.tiles_n, mb, nb);
      if (MOE && mb * tile_rows >= rows_in_use) continue;
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ++local;
      const int row = mb * tile_rows + quarter * 32 + lane;
      const int n0 = nb * BN;
      // column scales of this tile -> this warp's smem copy (fp32); row scale -> register
      const int64_t col_base = MOE ? int64_t(__ldg(p.expert_ids + (mb * tile_rows) / p.block_m)) * p.col_stride_e : 0;
      for (int j = lane; j < BN; j += 32)
        cs[j] = (n0 + j < p.N) ? load_as_f32(p.alpha_col, p.col_dtype, col_base + n0 + j) : 0.f;
      float rs = 0.f, rw = 1.f;
      int64_t out_row = -1;  // fused MoE: the flat (token, choice) index this slot writes, or -1
      if (MOE) {
        if (quarter * 32 + lane < tile_rows) {
          const int flat = __ldg(p.sorted_ids + row);
          if (flat >= 0 && flat < p.num_valid) {
            out_row = flat;
            rs = load_as_f32(p.alpha_row, p.row_dtype, flat / p.top_k);
            if (p.mul_w) rw = load_as_f32(p.topk_w, p.topk_w_dtype, flat);
          }
        }
      } else {
        rs = (row < p.M) ? load_as_f32(p.alpha_row, p.row_dtype, row) : 0.f;
      }
      __syncwarp();

      ok = mbar_wait_bounded(&tmem_full_bar[buf], acc_phase, abort_flag, p.wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, abort_flag, DEV_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tc_wait_ld();
        if (MOE) {
          if (out_row >= 0) store_chunk_moe<OutT>(r, out_row, n0 + c * 32, rs, rw, p.mul_w != 0, cs + c * 32, p, vec_ok);
        } else {
          store_chunk<OutT>(r, row, n0 + c * 32, rs, cs + c * 32, same16, p, vec_ok, acc_vec_ok);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
    }
  }

  // -------------------------------- teardown --------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// CTA-pair variant (cluster of 2, tcgen05 cta_group::2): one 256 x BN output tile per pair (BN = 256 unless a
// narrower tile fills the last wave better, see pick_pair_bn).
// CTA r of the pair loads rows [128 r, 128 r + 128) of the A tile and its half of the B tile's rows (no multicast:
// every CTA fetches exactly the bytes that end up in its own shared memory), so each stage is
// 32 KB per CTA for the same MMA work that takes 48 KB in the single-CTA kernel: a third less
// L2->SM traffic and a deeper ring in the same shared memory.  The leader CTA (rank 0) issues
// the MMAs for both; each CTA's TMEM holds its own 128 accumulator rows and each CTA runs its
// own epilogue.  Barriers:
//   full[s]        in the leader; the leader's producer expects the bytes of both CTAs, both CTAs'
//                  TMA loads complete on it
//   empty[s]       in each CTA; signalled by the leader's tcgen05.commit with a two-CTA mask
//   tmem_full[b]   in each CTA; signalled the same way when a tile's accumulator is complete
//   tmem_empty[b]  in the leader; 8 arrivals (4 epilogue warps of each CTA, the peer's remotely)
// ---------------------------------------------------------------------------
// Work list of one CTA pair; its three roles walk the same list.  Plain mode: whole tiles pair_id, pair_id +
// num_pairs, ...  K-balanced mode: the tiles of the ragged round (the first sk_tiles) come first.  Pair i < sk_tiles
// takes the head [0, sk_units) of tile i, so all heads advance through K in step, like whole tiles do (which is what
// keeps the operand re-reads in L2); the remaining pairs walk their share of the tails and hand each piece over.
// The whole rounds follow, for every pair alike, and hide the longer epilogue of a head behind their MMAs.
template <bool SK, bool MOE = false> struct PairWork {
  int tile, kb0, kb1;  // the current piece: K blocks [kb0, kb1) of a tile
  int slot;            // workspace slot a tail piece is handed over in, -1 for any other piece
  bool head;           // head of a shared tile: its epilogue adds the tail pieces
  int next_plain, step, num_tiles, k_blocks;
  int pair, units, tail, pos, pos_end, next_slot;
  int tiles_m, tiles_n, rows_in_use;  // fused MoE: row tiles past the slots in use are left out
  bool head_pending;
  __device__ __forceinline__ PairWork(const A8W8Params& p, int pair_id, int num_pairs) {
    k_blocks = p.k_blocks;
    num_tiles = p.tiles_m * p.tiles_n;
    tiles_m = p.tiles_m;
    tiles_n = p.tiles_n;
    rows_in_use = MOE ? __ldg(p.num_post_padded) : 0;
    step = num_pairs;
    next_plain = pair_id;
    tile = kb0 = kb1 = 0;
    slot = -1;
    head = head_pending = false;
    pair = pair_id;
    units = tail = pos = pos_end = next_slot = 0;
    if (SK) {
      next_plain += p.sk_tiles;
      units = p.sk_units;
      tail = k_blocks - units;
      if (pair_id < p.sk_tiles) {
        head_pending = true;
      } else {
        const int h = pair_id - p.sk_tiles;
        pos = min(p.sk_tiles * tail, h * p.sk_tail_units);
        pos_end = min(p.sk_tiles * tail, pos + p.sk_tail_units);
        next_slot = h * p.sk_slots;
      }
    }
  }
  __device__ __forceinline__ bool next() {
    slot = -1;
    head = false;
    if (SK && head_pending) {
      head_pending = false;
      tile = pair;
      kb0 = 0;
      kb1 = units;
      head = tail > 0;
      return true;
    }
    if (SK && pos < pos_end) {
      tile = pos / tail;
      const int off = pos - tile * tail;
      const int len = min(tail - off, pos_end - pos);
      kb0 = units + off;
      kb1 = kb0 + len;
      pos += len;
      slot = next_slot++;
      return true;
    }
    kb0 = 0;
    kb1 = k_blocks;
    while (true) {
      tile = next_plain;
      next_plain += step;
      if (tile >= num_tiles) return false;
      if (!MOE) return true;
      int mb, nb;
      tile_coords(tile, tiles_m, tiles_n, mb, nb);
      if (mb * 256 < rows_in_use) return true;
    }
  }
};

__device__ __forceinline__ void flag_store_release(unsigned long long* f, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(f), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long flag_load_acquire(const unsigned long long* f) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(f) : "memory");
  return v;
}
// Bounded wait (one lane) until *f == want; false when the limit ran out or another role reported a failure.
__device__ __forceinline__ bool flag_wait_bounded(const unsigned long long* f, unsigned long long want,
                                                  volatile int* abort_flag) {
  if (flag_load_acquire(f) == want) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (flag_load_acquire(f) == want) return true;
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) return false;
    }
  }
}

template <int BN, int STAGES, int EPI = 4> struct PairSmem {
  static constexpr int kBN = BN;                        // output columns of a pair tile (a multiple of 32, at most 256)
  static constexpr int kABytes = kBM * kBK;             // this CTA's 128 rows of A
  static constexpr int kBBytes = (kBN / 2) * kBK;       // this CTA's BN / 2 rows of B
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kOutOff = STAGES * kStageBytes;        // [EPI epilogue warps][2][32 rows x 64 B] output staging
  static constexpr int kOutBufs = EPI == 4 ? 2 : 1;           // staging buffers per epilogue warp
  static constexpr int kOutBytes = EPI * kOutBufs * 2048;
  static constexpr int kColScaleOff = kOutOff + kOutBytes;    // [EPI][kBN] float
  static constexpr int kBarOff = kColScaleOff + EPI * kBN * 4;
  static constexpr int kNumBars = 2 * STAGES + 4 + 1;
  static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
  static constexpr int kAbortOff = kTmemSlotOff + 8;
  static constexpr int kTotal = kAbortOff + 8;
  static constexpr int kDynamicBytes = kTotal + 1024;
};

// MOE: fused-MoE mode for blocks of 256 sorted slots (A8W8Params, "Fused-MoE mode"): a pair tile is one block, whose
// expert picks the weight rows and column scales; the epilogue scatters each slot's row to its (token, choice) index.
// EPI: epilogue warps per CTA, 4 or 8.  With 8 (the plain mode's default), two warps share a TMEM lane quarter and
// split a tile's column chunks, and each has one output staging buffer instead of two.
template <typename OutT, int BN, int STAGES, bool SK, bool MOE = false, int EPI = 4>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((2 + EPI) * 32, 1)
a8w8_umma_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_out, const A8W8Params p) {
  using L = PairSmem<BN, STAGES, EPI>;
  static_assert(EPI == 4 || (EPI == 8 && !SK && !MOE), "eight epilogue warps exist for the plain mode only");
  constexpr int kAccStride = 256;  // TMEM columns between the two accumulators (512 are allocated whatever BN is)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* col_scale_smem = reinterpret_cast<float*>(smem + L::kColScaleOff);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full_bar = bars + 2 * STAGES;
  uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2;
  uint64_t* drain_bar = bars + 2 * STAGES + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlotOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  constexpr uint32_t kTmemCols = 2 * kAccStride;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 2 * EPI);
    }
    mbar_init(drain_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.out_tma) tma_prefetch_desc(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything crosses the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    const bool leader_lane = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    long long issued = 0;
    bool ok = true;
    PairWork<SK, MOE> w(p, pair_id, num_pairs);
    while (ok && w.next()) {
      int mb, nb;
      tile_coords(w.tile, p.tiles_m, p.tiles_n, mb, nb);
      // fused MoE: the tile's weights are rows [e * N + nb * BN, ...) of the expert stack
      const int b_row = nb * BN + int(rank) * (BN / 2) + (MOE ? __ldg(p.expert_ids + (mb * 256) / p.block_m) * p.N : 0);
      for (int kb = w.kb0; kb < w.kb1; ++kb) {
        ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (leader_lane) report(p.status, abort_flag, DEV_TIMEOUT_PRODUCER);
          break;
        }
        if (leader_lane) {
          uint8_t* sa = smem + stage * L::kStageBytes;
          const uint32_t full_in_leader = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
          tma_load_2d_pair(sa, &tmap_a, full_in_leader, kb * kBK, mb * 256 + int(rank) * 128);
          tma_load_2d_pair(sa + L::kABytes, &tmap_b, full_in_leader, kb * kBK, b_row);
          ++issued;
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    // Wait (bounded, cut short by an abort) until the MMAs have consumed the last stages issued:
    // nothing is still being written into this CTA's shared memory when it exits.
    if (leader_lane) {
      const long long first = issued > STAGES ? issued - STAGES : 0;
      for (long long i = first; i < issued; ++i)
        if (!mbar_wait_bounded(&empty_bar[i % STAGES], uint32_t((i / STAGES) & 1), abort_flag)) break;
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader only) -------------------------------
    const bool leader_lane = elect_one();
    if (rank == 0) {
      constexpr uint32_t idesc = umma_idesc(/*s32*/ 2, /*signed 8-bit*/ 1, 256, BN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      bool issued_any = false;
      PairWork<SK, MOE> w(p, pair_id, num_pairs);
      for (; ok && w.next(); ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        ok = mbar_wait_bounded(&tmem_empty_bar[buf], acc_phase ^ 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (leader_lane) report(p.status, abort_flag, DEV_TIMEOUT_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * kAccStride;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          ok = mbar_wait_bounded(&full_bar[stage], phase, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (leader_lane) report(p.status, abort_flag, DEV_TIMEOUT_MMA);
            break;
          }
          tc_fence_after();
          if (leader_lane) {
            const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
            const uint32_t sb = sa + L::kABytes;
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k)
              umma_i8_pair(tmem_d, umma_desc_k_sw128(sa + k * kUmmaK), umma_desc_k_sw128(sb + k * kUmmaK), idesc,
                           (kb != w.kb0 || k != 0) ? 1u : 0u);
            tc_commit_pair(&empty_bar[stage], 0x3);  // frees this stage in both CTAs
            issued_any = true;
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok && leader_lane) tc_commit_pair(&tmem_full_bar[buf], 0x3);  // accumulator complete, both CTAs
        __syncwarp();
      }
      // Wait (bounded) for every MMA issued before TMEM is freed, even after an abort.
      if (leader_lane && issued_any) {
        int none = 0;
        tc_commit_pair(drain_bar, 0x1);
        if (!mbar_wait_bounded(drain_bar, 0, &none)) report(p.status, abort_flag, DEV_TIMEOUT_DRAIN);
      }
    }
  } else {
    // -------------------------------- epilogue (both CTAs) --------------------------------
    const int quarter = warp & 3;
    const int ewarp = warp - 2;                  // 0 .. EPI-1
    constexpr int NC = BN / 32;                  // column chunks of a tile
    const int c_begin = (EPI == 8 && ewarp >= 4) ? (NC + 1) / 2 : 0;  // with eight warps the second four take the upper chunks
    const int c_end = (EPI == 8 && ewarp < 4) ? (NC + 1) / 2 : NC;
    float* cs = col_scale_smem + ewarp * BN;  // this warp's private copy
    const bool same16 = (p.row_dtype == p.col_dtype) && (p.row_dtype != FNN_F32);
    const bool vec_ok = (p.ldo % 8 == 0) && (reinterpret_cast<uintptr_t>(p.out) % 16 == 0);
    const bool acc_vec_ok = p.acc_out && (p.ldacc % 4 == 0) && (reinterpret_cast<uintptr_t>(p.acc_out) % 16 == 0);
    int local = 0;
    bool ok = true;
    PairWork<SK, MOE> w(p, pair_id, num_pairs);
    uint8_t* out_stage = smem + L::kOutOff + ewarp * (L::kOutBufs * 2048);  // this warp's output staging buffer(s)
    int out_buf = 0;
    const int my_flag = int(rank) * 4 + quarter;                        // this warp's flag word within a pair's eight
    const int my_row = int(rank) * 128 + quarter * 32 + lane;           // this thread's row within a tile
    for (; ok && w.next(); ++local) {
      int mb, nb;
      tile_coords(w.tile, p.tiles_m, p.tiles_n, mb, nb);
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const int row = mb * 256 + my_row;
      // K-balanced mode: a tail piece is handed over; a head adds the pieces of its tile's tail, which lie in the
      // slots of the tail-sharing pairs first_h .. last_h
      const bool hands_over = SK && w.slot >= 0;
      const bool adds = SK && w.head;
      const int tail_blocks = p.k_blocks - p.sk_units;
      const int first_h = adds ? (w.tile * tail_blocks) / p.sk_tail_units : 0;
      const int last_h = adds ? ((w.tile + 1) * tail_blocks - 1) / p.sk_tail_units : -1;
      // slot of the piece of this tile that tail-sharing pair h computed: its pieces are of consecutive tiles
      auto slot_of = [&](int h) { return h * p.sk_slots + (w.tile - (h * p.sk_tail_units) / tail_blocks); };
      const int n0 = nb * BN;
      const int64_t col_base = MOE ? int64_t(__ldg(p.expert_ids + (mb * 256) / p.block_m)) * p.col_stride_e : 0;
      for (int j = c_begin * 32 + lane; j < c_end * 32; j += 32)
        cs[j] = (n0 + j < p.N) ? load_as_f32(p.alpha_col, p.col_dtype, col_base + n0 + j) : 0.f;
      float rs = 0.f, rw = 1.f;
      int64_t out_row = -1;  // fused MoE: the flat (token, choice) index this slot writes, or -1
      if (MOE) {
        const int flat = __ldg(p.sorted_ids + row);
        if (flat >= 0 && flat < p.num_valid) {
          out_row = flat;
          rs = load_as_f32(p.alpha_row, p.row_dtype, flat / p.top_k);
          if (p.mul_w) rw = load_as_f32(p.topk_w, p.topk_w_dtype, flat);
        }
      } else {
        rs = (row < p.M) ? load_as_f32(p.alpha_row, p.row_dtype, row) : 0.f;
      }
      __syncwarp();

      ok = mbar_wait_bounded(&tmem_full_bar[buf], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, abort_flag, DEV_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      if (adds) {
        // wait (bounded) until every piece of the tail has been delivered for this warp's rows
        for (int h = first_h; h <= last_h && ok; ++h) {
          if (lane == 0) ok = flag_wait_bounded(p.sk_flags + slot_of(h) * 8 + my_flag, p.sk_epoch, abort_flag);
          ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
        }
        __syncwarp();  // lane 0's acquire orders the other lanes' reads of the sums as well
        if (!ok) {
          if (lane == 0) report(p.status, abort_flag, DEV_TIMEOUT_EPILOGUE);
          break;
        }
      }
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * kAccStride;
      // Partial sums in the workspace: slot of a pair = [chunk of 32 columns][epilogue warp of the pair][j][lane]
      // 16-byte words, word j of a lane holding its row's columns 4j .. 4j+3 of the chunk: every warp access is 512
      // contiguous bytes, and the warp that reads a word is the one (same CTA rank, same quarter) that wrote it.
      auto slot_word = [&](int slot, int c) {
        return reinterpret_cast<uint4*>(p.sk_partials + size_t(slot) * 256 * 256) + ((c * 8 + my_flag) * 8) * 32 + lane;
      };
      uint4 ahead[8];  // the first tail piece's sums of the chunk after the current one, fetched a chunk early
      if (adds) {
        const uint4* src = slot_word(slot_of(first_h), 0);
#pragma unroll
        for (int j = 0; j < 8; ++j) ahead[j] = __ldcg(src + j * 32);  // written by another SM in this launch: read through L2
      }
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        uint4 cur[8];
        if (adds) {
#pragma unroll
          for (int j = 0; j < 8; ++j) cur[j] = ahead[j];
          if (c + 1 < BN / 32) {
            const uint4* src = slot_word(slot_of(first_h), c + 1);
#pragma unroll
            for (int j = 0; j < 8; ++j) ahead[j] = __ldcg(src + j * 32);
          }
        }
        tc_wait_ld();
        if (hands_over) {
          uint4* dst = slot_word(w.slot, c);  // the raw sums
#pragma unroll
          for (int j = 0; j < 8; ++j) dst[j * 32] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          continue;
        }
        if (adds) {
          // int32 sums: exact in any order
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            r[4 * j] += cur[j].x; r[4 * j + 1] += cur[j].y; r[4 * j + 2] += cur[j].z; r[4 * j + 3] += cur[j].w;
          }
          for (int h = first_h + 1; h <= last_h; ++h) {  // a tail cut into more than one piece
            const uint4* src = slot_word(slot_of(h), c);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint4 v = __ldcg(src + j * 32);
              r[4 * j] += v.x; r[4 * j + 1] += v.y; r[4 * j + 2] += v.z; r[4 * j + 3] += v.w;
            }
          }
        }
        if (MOE) {
          if (out_row >= 0) store_chunk_moe<OutT>(r, out_row, n0 + c * 32, rs, rw, p.mul_w != 0, cs + c * 32, p, vec_ok);
        } else if (p.out_tma) {
          // The 32 x 32 block of outputs goes through shared memory and leaves as one TMA store: whole 64-byte row
          // pieces instead of 16 bytes per lane and row.  Rows of 64 bytes in the 64-byte swizzle pattern (16-byte
          // piece j of row l sits at piece j ^ ((l >> 1) & 3)), so the 32 lanes' stores spread over all banks; the
          // store leaves out what lies beyond M or N.  Two buffers per warp: before one is written again, the store
          // that read it two chunks ago has finished reading.
          store_acc_chunk(r, row, n0 + c * 32, p, acc_vec_ok);
          float v[32];
          scale_chunk(r, rs, cs + c * 32, same16, p, v);
          if (lane == 0) tma_store_wait_read<L::kOutBufs - 1>();
          __syncwarp();
          uint8_t* buf_out = out_stage + out_buf * 2048;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(buf_out + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
                make_uint4(pack2<OutT>(v[8 * j], v[8 * j + 1]), pack2<OutT>(v[8 * j + 2], v[8 * j + 3]),
                           pack2<OutT>(v[8 * j + 4], v[8 * j + 5]), pack2<OutT>(v[8 * j + 6], v[8 * j + 7]));
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && n0 + c * 32 < p.N && mb * 256 + int(rank) * 128 + quarter * 32 < p.M) {
            tma_store_2d(&tmap_out, buf_out, n0 + c * 32, mb * 256 + int(rank) * 128 + quarter * 32);
            tma_store_commit();
          }
          if (L::kOutBufs == 2) out_buf ^= 1;
        } else {
          store_chunk<OutT>(r, row, n0 + c * 32, rs, cs + c * 32, same16, p, vec_ok, acc_vec_ok);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[buf]), 0));  // the accumulator is free again
      if (hands_over) {
        // the warp's stores are ordered before lane 0 by the barrier above, and its release makes them visible
        // device-wide before the flag says so
        if (lane == 0) flag_store_release(p.sk_flags + w.slot * 8 + my_flag, p.sk_epoch);
      } else if (adds && lane == 0) {
        // consumed: the words go back to 0, so that a replay of this launch (same epoch) waits again
        for (int h = first_h; h <= last_h; ++h)
          *reinterpret_cast<volatile unsigned long long*>(p.sk_flags + slot_of(h) * 8 + my_flag) = 0ull;
      }
    }
    if (lane == 0) tma_store_wait_all<0>();  // this warp's output stores have left shared memory and are complete
  }

  // -------------------------------- teardown --------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still touch its memory or barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// Any alignment, any strides: one thread per output element (correctness path
// for operands the TMA path cannot address; also covers K == 0).
template <typename OutT>
__global__ void a8w8_generic_kernel(const int8_t* __restrict__ a, int64_t lda, const int8_t* __restrict__ b,
                                    int64_t ldb, const A8W8Params p) {
  const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= int64_t(p.M) * p.N) return;
  const int m = int(idx / p.N), n = int(idx % p.N);
  const int8_t* ar = a + m * lda;
  const int8_t* br = b + n * ldb;
  int acc = 0;
  for (int k = 0; k < p.K; ++k) acc += int(ar[k]) * int(br[k]);
  if (p.acc_out) p.acc_out[m * p.ldacc + n] = acc;
  const bool same16 = (p.row_dtype == p.col_dtype) && (p.row_dtype != FNN_F32);
  float s = __fmul_rn(load_as_f32(p.alpha_row, p.row_dtype, m), load_as_f32(p.alpha_col, p.col_dtype, n));
  if (same16) s = round_through(s, p.row_dtype);
  reinterpret_cast<OutT*>(p.out)[m * p.ldo + n] = from_f32<OutT>(__fmul_rn(float(acc), s));
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
// int8 [rows, K] row-major (pitch `ld` bytes) -> tensor map with a {128 B, box_rows} box, 128-byte swizzle
int make_tmap_i8(CUtensorMap* m, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows) {
  return make_tmap_2d(m, /*elem_bytes=*/1, base, rows, K, ld, kBK, box_rows, /*swizzle128=*/true);
}

template <typename OutT, int BN, int STAGES, int AROWS>
int launch_umma(const int8_t* a, int64_t lda, const int8_t* b, int64_t ldb, A8W8Params p, cudaStream_t st) {
  using L = SmemLayout<BN, STAGES, AROWS>;
  static_assert(L::kDynamicBytes <= 227 * 1024, "shared memory budget");
  static_assert(L::kStageBytes % 1024 == 0 && L::kABytes % 1024 == 0, "tiles must stay 1024-byte aligned");
  auto kern = a8w8_umma_kernel<OutT, BN, STAGES, false, AROWS>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];  // per device, so that a failure is reported on every call and not only the first
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  });
  if (attr_err[dev] != cudaSuccess) return check_cuda(attr_err[dev], "cudaFuncSetAttribute(a8w8)");
  CUtensorMap ta, tb;
  if (int e = make_tmap_i8(&ta, a, p.M, p.K, lda, AROWS)) return e;
  if (int e = make_tmap_i8(&tb, b, p.N, p.K, ldb, BN)) return e;
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.k_blocks = (p.K + kBK - 1) / kBK;
  if (const int stall_us = opt_test_stall_us()) {  // test hook: make one wait run out quickly
    p.wait_ns = 1000ull * unsigned(stall_us);
    p.skip_kb = p.k_blocks > 1 ? 1 : 0;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kThreads, L::kDynamicBytes, st>>>(ta, tb, p);
  return check_cuda(cudaGetLastError(), "a8w8 tcgen05 launch");
}

// Tile width BN with the stage count that fills shared memory for the rows of A a stage has to hold.
template <typename OutT, int BN>
int launch_umma_rows(const int8_t* a, int64_t lda, const int8_t* b, int64_t ldb, const A8W8Params& p, cudaStream_t st) {
  constexpr int kBudget = 210 * 1024;
  if (p.M <= 16) return launch_umma<OutT, BN, kBudget / ((16 + BN) * kBK), 16>(a, lda, b, ldb, p, st);
  if (p.M <= 64) return launch_umma<OutT, BN, kBudget / ((64 + BN) * kBK), 64>(a, lda, b, ldb, p, st);
  return launch_umma<OutT, BN, kBudget / ((kBM + BN) * kBK) < 8 ? kBudget / ((kBM + BN) * kBK) : 8, kBM>(a, lda, b, ldb, p, st);
}

// Geometry of the K-balanced mode for `tiles` 256-wide tiles of `kbs` K blocks on `pairs` CTA pairs.
struct SkSplit {
  int tiles;       // shared tiles: the ragged round
  int units;       // K blocks of a head
  int tail_units;  // K blocks of the concatenated tails per tail-sharing pair
  int slots;       // pieces a tail-sharing pair may hand over
  bool valid;
};
inline SkSplit sk_split(long long tiles, int kbs, int pairs) {
  SkSplit s{0, 0, 0, 0, false};
  const int ragged = int(tiles % pairs);
  if (ragged == 0 || kbs < 2) return s;
  s.tiles = ragged;
  // A pair that walks tail pieces is slower than one that computes a head: its operands are not being read by
  // other pairs at the same moment (the heads advance through K together and meet in L2), and every piece has an
  // epilogue of its own.  Measured: about 0.85 of the heads' rate, and 8 K blocks' time per share (less for short K).  The heads take
  // that much more, so that both kinds finish together.
  const int helpers = pairs - ragged;
  const double head = (double(ragged) * kbs + helpers * (kbs < 64 ? kbs / 8.0 : 8.0)) / (ragged + helpers * 0.85);
  s.units = int(head + 0.999);
  if (s.units >= kbs) return s;
  const int tail = kbs - s.units;
  s.tail_units = int((1ll * ragged * tail + helpers - 1) / helpers);
  s.slots = (s.tail_units + tail - 1) / tail + 1;
  s.valid = true;
  return s;
}

// Bytes of scratch the K-balanced mode needs: eight flag words and a 256 x 256 int32 slot per piece that can be
// handed over; fewer than two pieces per CTA pair whatever the shape.
constexpr size_t kSkFlagBytes = 16384;
inline int sk_max_slots(int sms) { return 2 * (sms / 2); }
inline size_t sk_workspace_bytes(int sms) { return kSkFlagBytes + size_t(sk_max_slots(sms)) * 256 * 256 * 4; }

inline unsigned long long next_sk_epoch() {
  static std::atomic<unsigned long long> epoch{
      (static_cast<unsigned long long>(std::chrono::steady_clock::now().time_since_epoch().count()) * 0x9E3779B97F4A7C15ull) | 1ull};
  unsigned long long e = epoch.fetch_add(2, std::memory_order_relaxed);  // stays odd: never 0
  return e;
}

template <typename OutT, int BN, bool SK = false, int EPI = 4>
int launch_pair(const int8_t* a, int64_t lda, const int8_t* b, int64_t ldb, A8W8Params p, cudaStream_t st,
                void* workspace = nullptr) {
  // for the operand ring; the output staging buffers and the column scales of the epilogue warps take the rest
  constexpr int kBudget = (EPI == 4 ? 196 : 194) * 1024;
  constexpr int STAGES = kBudget / (kBM * kBK + (BN / 2) * kBK) < 8 ? kBudget / (kBM * kBK + (BN / 2) * kBK) : 8;
  using L = PairSmem<BN, STAGES, EPI>;
  static_assert(L::kDynamicBytes <= 227 * 1024, "shared memory budget");
  static_assert(L::kStageBytes % 1024 == 0 && L::kABytes % 1024 == 0 && L::kOutOff % 1024 == 0, "tiles must stay 1024-byte aligned");
  static_assert(BN % 32 == 0 && BN <= 256, "pair tile width");
  auto kern = a8w8_umma_pair_kernel<OutT, BN, STAGES, SK, false, EPI>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];  // per device, so that a failure is reported on every call and not only the first
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  });
  if (attr_err[dev] != cudaSuccess) return check_cuda(attr_err[dev], "cudaFuncSetAttribute(a8w8 pair)");
  CUtensorMap ta, tb, tout;
  if (int e = make_tmap_i8(&ta, a, p.M, p.K, lda, kBM)) return e;
  if (int e = make_tmap_i8(&tb, b, p.N, p.K, ldb, BN / 2)) return e;
  // output blocks of 32 rows x 32 columns (64 bytes per row) for the epilogue's TMA stores, where the output allows it
  p.out_tma = (reinterpret_cast<uintptr_t>(p.out) % 16 == 0) && ((p.ldo * int64_t(sizeof(OutT))) % 16 == 0);
  if (p.out_tma) {
    if (int e = make_tmap_2d(&tout, int(sizeof(OutT)), p.out, p.M, p.N, p.ldo * int64_t(sizeof(OutT)), 32, 32, /*swizzle=*/2)) return e;
  } else {
    tout = ta;  // never used
  }
  p.tiles_m = (p.M + 255) / 256;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.k_blocks = (p.K + kBK - 1) / kBK;
  const int tiles = p.tiles_m * p.tiles_n;
  int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  if (SK) {
    pairs = sm_count() / 2;
    const SkSplit split = sk_split(tiles, p.k_blocks, pairs);
    if (!split.valid || (pairs - split.tiles) * split.slots > sk_max_slots(sm_count()))
      return fail(FNN_ERR_UNSUPPORTED, "a8w8: the K-balanced mode does not apply to this shape");
    p.sk_tiles = split.tiles;
    p.sk_units = split.units;
    p.sk_tail_units = split.tail_units;
    p.sk_slots = split.slots;
    p.sk_flags = static_cast<unsigned long long*>(workspace);
    p.sk_partials = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(workspace) + kSkFlagBytes);
    p.sk_epoch = next_sk_epoch();
  }
  kern<<<2 * pairs, (2 + EPI) * 32, L::kDynamicBytes, st>>>(ta, tb, tout, p);
  return check_cuda(cudaGetLastError(), "a8w8 tcgen05 (CTA pair) launch");
}

// ---------------------------------------------------------------------------
// Shape -> kernel and tile (the static counterpart of the reference's autotune cache,
// flashnn/triton_kernels/triton_utils.py:84-151).  Both tensor-core kernels are persistent, so the time of a launch
// is waves x time of one tile; the plan with the least column-work per SM wins:
//   CTA pair, tile 256 x BN, BN in kPairWidths:  ceil(tiles / (SMs / 2)) * BN * kPairColumnCost[BN]
//   single CTA, tile 128 x BN, BN in {256, 128, 64}:  ceil(tiles / SMs) * BN * kSingleCtaPenalty
// The constants are measured (a8w8_plan.h, generated by flashnn_b200/tune_a8w8.py): a narrower pair tile re-reads
// the A rows for fewer output columns, and the single-CTA kernel moves half as many output columns per byte of
// operand traffic; it wins where the problem is too small to give every CTA pair a tile.  Problems of at
// most 128 rows are bound by the weight stream instead and keep their own rule.
// ---------------------------------------------------------------------------
struct A8W8Plan {
  bool pair;
  int bn;
  double cost;  // column-work per SM, in columns of a 128-row tile
  bool balanced = false;  // CTA-pair kernel in its K-balanced mode (needs the workspace)
};

// K-balanced mode: 256-wide pair tiles, the (tile, K block) units dealt out evenly, so the cost is the exact share
// of one pair plus what the hand-over of one partial tile costs, expressed in K blocks.
constexpr int kSkMinKBlocks = 128;
constexpr double kSkHandOverBlocks = 8.0;
constexpr int kSkMinTailBlocks = 24;
constexpr double kSkMinGain = 0.95;  // taken when at least 5 % cheaper than the best whole-tile plan

A8W8Plan plan_a8w8(int M, int N, int sms);

A8W8Plan plan_a8w8(int M, int N, int K, int sms, int balanced_mode /* 0 auto, 1 always where possible, 2 never */) {
  A8W8Plan best = plan_a8w8(M, N, sms);
  const int kbs = (K + kBK - 1) / kBK;
  if (M <= kBM || balanced_mode == 2 || kbs < (balanced_mode == 1 ? 2 : kSkMinKBlocks)) return best;
  const int pairs = sms / 2;
  const long long tiles = 1ll * ((M + 255) / 256) * ((N + 255) / 256);
  if (tiles * kbs > INT32_MAX) return best;
  const SkSplit split = sk_split(tiles, kbs, pairs);
  if (!split.valid || (pairs - split.tiles) * split.slots > sk_max_slots(sms)) return best;
  // short tails make pieces whose hand-over takes longer than their MMAs, short heads make tails that are cut into
  // many pieces, and with less than one whole round nothing follows the heads to hide their longer epilogue behind:
  // left to the forced mode
  if (balanced_mode != 1 && (kbs - split.units < kSkMinTailBlocks || split.units * 3 < kbs || tiles < pairs)) return best;
  const double blocks = double(tiles / pairs) * kbs + double(split.units) + kSkHandOverBlocks;
  const double cost = blocks / kbs * 256.0;
  if (balanced_mode == 1 || cost < best.cost * kSkMinGain) return A8W8Plan{true, 256, cost, true};
  return best;
}

A8W8Plan plan_a8w8(int M, int N, int sms) {
  A8W8Plan best{false, 64, 1e30};
  const int tiles_m1 = (M + kBM - 1) / kBM;
  if (M <= kBM) {
    // one row of tiles (decode shapes): bound by the weight stream, not by the tensor pipe.  The persistent CTAs walk
    // the tiles in rounds, so the time goes with rounds x tile width; ties keep the wider tile (more bytes in flight per
    // CTA), and 64-wide tiles carry a measured 20 % penalty (64 x 57344 x 8192: 0.098 ms with 256-wide tiles in two
    // rounds, 0.115 ms with 64-wide ones in seven; 64 x 14336 x 8192: 0.037 ms with 128-wide tiles in one round,
    // 0.041 ms with 64-wide ones in two).
    int best_bn = 256;
    double best_cost = 1e30;
    for (int bn : {256, 128, 64}) {
      const long long tiles = (N + bn - 1) / bn;
      const double cost = double((tiles + sms - 1) / sms) * bn * (bn == 64 ? 1.2 : 1.0);
      if (cost < best_cost) { best_cost = cost; best_bn = bn; }
    }
    return A8W8Plan{false, best_bn, 0.0};
  }
  for (int bn : {256, 128, 64}) {
    const long long tiles = 1ll * tiles_m1 * ((N + bn - 1) / bn);
    const double cost = double((tiles + sms - 1) / sms) * bn * kSingleCtaPenalty;
    if (cost < best.cost) best = A8W8Plan{false, bn, cost};
  }
  if (M > kBM) {
    const int pairs = sms / 2;
    const int tiles_m2 = (M + 255) / 256;
    for (int i = 0; i < 5; ++i) {
      const int bn = kPairWidths[i];
      const long long tiles = 1ll * tiles_m2 * ((N + bn - 1) / bn);
      const double cost = double((tiles + pairs - 1) / pairs) * bn * kPairColumnCost[i];
      if (cost < best.cost) best = A8W8Plan{true, bn, cost};  // ties keep the wider tile (listed first)
    }
  }
  return best;
}

template <typename OutT>
int dispatch(const int8_t* a, int64_t lda, const int8_t* b, int64_t ldb, const A8W8Params& p, cudaStream_t st,
             void* workspace, size_t workspace_bytes) {
  const bool tma_ok = p.K > 0 && (reinterpret_cast<uintptr_t>(a) % 16 == 0) && (reinterpret_cast<uintptr_t>(b) % 16 == 0) &&
                      (lda % 16 == 0) && (ldb % 16 == 0);
  if (!tma_ok) {
    const int64_t total = int64_t(p.M) * p.N;
    a8w8_generic_kernel<OutT><<<unsigned((total + 255) / 256), 256, 0, st>>>(a, lda, b, ldb, p);
    return check_cuda(cudaGetLastError(), "a8w8 generic launch");
  }
  // Up to 8 tokens: the weight stream is all that matters, and the per-lane streaming kernel of the weight-only
  // decode path moves it faster than tile copies do: 6-10 % on wide matrices, and 2-3x on narrow, long ones
  // (N = 1024 .. 4096 at K = 28672: 57 us -> 16 .. 33 us), where 64-column tiles leave most SMs without work while
  // the streaming kernel has a CTA per 16 channels.  It declines shapes it does not cover (K not a multiple of its
  // block, activations that do not fit its shared memory).
  if (p.M <= 8 && p.N >= 512 && opt_test_stall_us() == 0) {
    const int r = gemv_a8w8_imma(a, lda, b, ldb, p.alpha_row, p.row_dtype, p.alpha_col, p.col_dtype, p.out,
                                 std::is_same<OutT, __half>::value ? FNN_F16 : FNN_BF16, p.ldo, p.M, p.N, p.K, p.acc_out,
                                 p.ldacc, st);
    if (r >= 0) return r;
  }
  // the K-balanced mode needs scratch: without it (or with a misaligned one) the best whole-tile plan runs instead
  const bool ws_ok = workspace && workspace_bytes >= sk_workspace_bytes(sm_count()) && reinterpret_cast<uintptr_t>(workspace) % 256 == 0;
  A8W8Plan plan = opt_test_stall_us() != 0 ? A8W8Plan{false, 64, 0.0}
                                           : plan_a8w8(p.M, p.N, p.K, sm_count(), ws_ok ? opt_a8w8_balanced() : 2);
  if (const int forced = opt_a8w8_pair_tile()) {  // tuning hook: a given pair-tile width wherever the pair kernel can run
    if (p.M > kBM) plan = A8W8Plan{true, forced, 0.0};
  }
  if (plan.balanced) return launch_pair<OutT, 256, true>(a, lda, b, ldb, p, st, workspace);
  if (plan.pair && opt_a8w8_epilogue_warps() != 4) {
    // Eight epilogue warps per CTA (one output staging buffer each, so the operand ring keeps its depth).  With short K
    // a tile's MMAs take less time than four warps need to write it out: measured four -> eight warps, K = 1664
    // 2037 -> 3003 TOPS, 2048 2051 -> 2766, 3328 3273 -> 3344, 4096 3322 -> 3370, 8192 the same.
    switch (plan.bn) {
      case 256: return launch_pair<OutT, 256, false, 8>(a, lda, b, ldb, p, st);
      case 224: return launch_pair<OutT, 224, false, 8>(a, lda, b, ldb, p, st);
      case 192: return launch_pair<OutT, 192, false, 8>(a, lda, b, ldb, p, st);
      case 160: return launch_pair<OutT, 160, false, 8>(a, lda, b, ldb, p, st);
      default: return launch_pair<OutT, 128, false, 8>(a, lda, b, ldb, p, st);
    }
  }
  if (plan.pair) {
    switch (plan.bn) {
      case 256: return launch_pair<OutT, 256>(a, lda, b, ldb, p, st);
      case 224: return launch_pair<OutT, 224>(a, lda, b, ldb, p, st);
      case 192: return launch_pair<OutT, 192>(a, lda, b, ldb, p, st);
      case 160: return launch_pair<OutT, 160>(a, lda, b, ldb, p, st);
      default: return launch_pair<OutT, 128>(a, lda, b, ldb, p, st);
    }
  }
  if (plan.bn == 256) return launch_umma_rows<OutT, 256>(a, lda, b, ldb, p, st);
  if (plan.bn == 128) return launch_umma_rows<OutT, 128>(a, lda, b, ldb, p, st);
  return launch_umma_rows<OutT, 64>(a, lda, b, ldb, p, st);
}

// ---------------------------------------------------------------------------
// fused MoE (expert-sorted grouped GEMM)
// ---------------------------------------------------------------------------
// Copies token rows into expert-sorted order: slot s gets row sorted_ids[s] / top_k of A, padding slots get zeros.
// One warp per slot, 16 bytes per lane and step (K % 16 == 0).
__global__ void moe_gather_rows_kernel(const int8_t* __restrict__ a, int64_t lda, const int32_t* __restrict__ sorted_ids,
                                       const int32_t* __restrict__ num_post_padded, int num_valid, int top_k,
                                       int8_t* __restrict__ a_sorted, int K, int EM) {
  const int slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (slot >= EM || slot >= __ldg(num_post_padded)) return;
  const int lane = threadIdx.x & 31;
  const int flat = __ldg(sorted_ids + slot);
  const bool valid = flat >= 0 && flat < num_valid;
  const uint4* src = reinterpret_cast<const uint4*>(a + int64_t(valid ? flat / top_k : 0) * lda);
  uint4* dst = reinterpret_cast<uint4*>(a_sorted + int64_t(slot) * K);
  for (int i = lane; i < K / 16; i += 32) dst[i] = valid ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
}

template <typename OutT, int BN, int STAGES, int AROWS>
int launch_moe(const int8_t* a_sorted, int64_t EM, const int8_t* b, int64_t E, A8W8Params p, cudaStream_t st) {
  using L = SmemLayout<BN, STAGES, AROWS>;
  static_assert(L::kDynamicBytes <= 227 * 1024, "shared memory budget");
  auto kern = a8w8_umma_kernel<OutT, BN, STAGES, true, AROWS>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];  // per device, so that a failure is reported on every call and not only the first
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  });
  if (attr_err[dev] != cudaSuccess) return check_cuda(attr_err[dev], "cudaFuncSetAttribute(fused moe a8w8)");
  CUtensorMap ta, tb;
  if (int e = make_tmap_i8(&ta, a_sorted, EM, p.K, p.K, AROWS)) return e;  // a block's own slots (and a few more)
  if (int e = make_tmap_i8(&tb, b, E * p.N, p.K, p.K, BN)) return e;
  p.tiles_m = int(EM / p.tile_rows);
  p.tiles_n = (p.N + BN - 1) / BN;
  p.k_blocks = (p.K + kBK - 1) / kBK;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kThreads, L::kDynamicBytes, st>>>(ta, tb, p);
  return check_cuda(cudaGetLastError(), "fused moe a8w8 launch");
}

template <typename OutT, int BN>
int launch_moe_rows(const int8_t* a_sorted, int64_t EM, const int8_t* b, int64_t E, const A8W8Params& p, cudaStream_t st) {
  constexpr int kBudget = 210 * 1024;
  if (p.tile_rows <= 16) return launch_moe<OutT, BN, kBudget / ((16 + BN) * kBK), 16>(a_sorted, EM, b, E, p, st);
  if (p.tile_rows <= 64) return launch_moe<OutT, BN, kBudget / ((64 + BN) * kBK), 64>(a_sorted, EM, b, E, p, st);
  return launch_moe<OutT, BN, kBudget / ((kBM + BN) * kBK) < 8 ? kBudget / ((kBM + BN) * kBK) : 8, kBM>(a_sorted, EM, b, E, p, st);
}

// Blocks of 256 sorted slots (or a multiple): one block is one 256-row tile of the CTA-pair kernel.
template <typename OutT>
int launch_moe_pair(const int8_t* a_sorted, int64_t EM, const int8_t* b, int64_t E, A8W8Params p, cudaStream_t st) {
  constexpr int BN = 256;
  constexpr int kBudget = 196 * 1024;
  constexpr int STAGES = kBudget / (kBM * kBK + (BN / 2) * kBK);
  using L = PairSmem<BN, STAGES>;
  static_assert(L::kDynamicBytes <= 227 * 1024, "shared memory budget");
  auto kern = a8w8_umma_pair_kernel<OutT, BN, STAGES, false, true>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];  // per device, so that a failure is reported on every call and not only the first
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  });
  if (attr_err[dev] != cudaSuccess) return check_cuda(attr_err[dev], "cudaFuncSetAttribute(fused moe a8w8, CTA pair)");
  CUtensorMap ta, tb;
  if (int e = make_tmap_i8(&ta, a_sorted, EM, p.K, p.K, kBM)) return e;
  if (int e = make_tmap_i8(&tb, b, E * p.N, p.K, p.K, BN / 2)) return e;
  p.tiles_m = int(EM / 256);
  p.tiles_n = (p.N + BN - 1) / BN;
  p.k_blocks = (p.K + kBK - 1) / kBK;
  p.out_tma = 0;
  const int tiles = p.tiles_m * p.tiles_n;
  const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  kern<<<2 * pairs, kThreads, L::kDynamicBytes, st>>>(ta, tb, ta, p);
  return check_cuda(cudaGetLastError(), "fused moe a8w8 (CTA pair) launch");
}

template <typename OutT>
int dispatch_moe(const int8_t* a_sorted, int64_t EM, const int8_t* b, int64_t E, const A8W8Params& p, cudaStream_t st) {
  // the widest tile that still gives every SM work; small problems stream the expert weights with 64-wide tiles
  const int sms = sm_count();
  // blocks of 256 slots with enough tiles for every CTA pair: the CTA-pair kernel (a third less operand traffic per MMA)
  if (p.block_m % 256 == 0 && (EM / 256) * ((p.N + 255) / 256) >= sms / 2)
    return launch_moe_pair<OutT>(a_sorted, EM, b, E, p, st);
  const int64_t tiles_m = EM / p.tile_rows;
  if (tiles_m * ((p.N + 255) / 256) >= sms) return launch_moe_rows<OutT, 256>(a_sorted, EM, b, E, p, st);
  if (tiles_m * ((p.N + 127) / 128) >= sms) return launch_moe_rows<OutT, 128>(a_sorted, EM, b, E, p, st);
  return launch_moe_rows<OutT, 64>(a_sorted, EM, b, E, p, st);
}

}  // namespace
}  // namespace fnn

extern "C" size_t fnn_fused_moe_a8w8_workspace_bytes(int64_t EM, int64_t K) {
  if (EM <= 0 || K <= 0) return 0;
  return (size_t(EM) * size_t(K) + 255) / 256 * 256;  // the expert-sorted copy of the token rows
}

extern "C" int fnn_fused_moe_a8w8(const int8_t* a, int64_t lda, const int8_t* b, int64_t E, int64_t N, int64_t K,
                                  const void* alpha_row, int row_dtype, const void* alpha_col, int col_dtype,
                                  const void* topk_weights, int topk_dtype, const int32_t* sorted_token_ids, int64_t EM,
                                  const int32_t* expert_ids, const int32_t* num_tokens_post_padded,
                                  int64_t num_valid_tokens, int top_k, int block_m, int mul_routed_weight, void* out,
                                  int out_dtype, int64_t ldo, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace fnn;
  if (E <= 0 || N < 0 || K <= 0 || EM < 0 || lda < K || ldo < N || num_valid_tokens < 0 || top_k <= 0 || block_m <= 0)
    return fail(FNN_ERR_SHAPE, "fused_moe_a8w8: E=%lld N=%lld K=%lld EM=%lld lda=%lld ldo=%lld top_k=%d block_m=%d", (long long)E,
                (long long)N, (long long)K, (long long)EM, (long long)lda, (long long)ldo, top_k, block_m);
  if (E * N > INT32_MAX || K > INT32_MAX || EM > INT32_MAX || num_valid_tokens > INT32_MAX)
    return fail(FNN_ERR_SHAPE, "fused_moe_a8w8: sizes must be below 2^31");
  if (EM % block_m != 0) return fail(FNN_ERR_SHAPE, "fused_moe_a8w8: %lld sorted slots are not a multiple of block_m=%d", (long long)EM, block_m);
  if (block_m > kBM && block_m % kBM != 0)
    return fail(FNN_ERR_UNSUPPORTED, "fused_moe_a8w8: block_m must be at most %d or a multiple of it (got %d)", kBM, block_m);
  if (out_dtype != FNN_F16 && out_dtype != FNN_BF16) return fail(FNN_ERR_DTYPE, "fused_moe_a8w8: output must be f16 or bf16");
  if (row_dtype < FNN_F16 || row_dtype > FNN_F32 || col_dtype < FNN_F16 || col_dtype > FNN_F32)
    return fail(FNN_ERR_DTYPE, "fused_moe_a8w8: scales must be f16, bf16 or f32");
  if (mul_routed_weight && (topk_dtype < FNN_F16 || topk_dtype > FNN_F32)) return fail(FNN_ERR_DTYPE, "fused_moe_a8w8: routing weights must be f16, bf16 or f32");
  if (EM == 0 || N == 0 || num_valid_tokens == 0) return FNN_OK;
  if (!a || !b || !alpha_row || !alpha_col || !sorted_token_ids || !expert_ids || !num_tokens_post_padded || !out ||
      (mul_routed_weight && !topk_weights))
    return fail(FNN_ERR_NULL_POINTER, "fused_moe_a8w8: null tensor pointer");
  if (K % 16 != 0 || reinterpret_cast<uintptr_t>(a) % 16 != 0 || lda % 16 != 0 || reinterpret_cast<uintptr_t>(b) % 16 != 0)
    return fail(FNN_ERR_ALIGNMENT, "fused_moe_a8w8: K and lda must be multiples of 16 and the operands 16-byte aligned");
  const size_t need = fnn_fused_moe_a8w8_workspace_bytes(EM, K);
  if (!workspace || workspace_bytes < need) return fail(FNN_ERR_WORKSPACE, "fused_moe_a8w8: needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return fail(FNN_ERR_ALIGNMENT, "fused_moe_a8w8: workspace must be 256-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int8_t* a_sorted = static_cast<int8_t*>(workspace);
  moe_gather_rows_kernel<<<unsigned((EM + 7) / 8), 256, 0, st>>>(a, lda, sorted_token_ids, num_tokens_post_padded,
                                                                 int(num_valid_tokens), top_k, a_sorted, int(K), int(EM));
  if (int e = check_cuda(cudaGetLastError(), "fused moe gather launch")) return e;
  A8W8Params p{};
  p.alpha_row = alpha_row; p.alpha_col = alpha_col; p.out = out; p.acc_out = nullptr;
  p.ldo = ldo; p.ldacc = 0; p.row_dtype = row_dtype; p.col_dtype = col_dtype;
  p.M = int(num_valid_tokens); p.N = int(N); p.K = int(K);
  p.status = device_status_word();
  p.wait_ns = kWaitLimitNs; p.skip_kb = -1;
  p.sorted_ids = sorted_token_ids; p.expert_ids = expert_ids; p.num_post_padded = num_tokens_post_padded;
  p.topk_w = topk_weights; p.topk_w_dtype = topk_dtype; p.top_k = top_k; p.block_m = block_m;
  p.tile_rows = block_m < kBM ? block_m : kBM; p.num_valid = int(num_valid_tokens); p.mul_w = mul_routed_weight ? 1 : 0;
  p.col_stride_e = N;
  if (out_dtype == FNN_F16) return dispatch_moe<__half>(a_sorted, EM, b, E, p, st);
  return dispatch_moe<__nv_bfloat16>(a_sorted, EM, b, E, p, st);
}

extern "C" size_t fnn_gemm_a8w8_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  using namespace fnn;
  if (M <= 0 || N <= 0 || K <= 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return 0;
  if (opt_test_stall_us() != 0 || opt_a8w8_pair_tile() != 0) return 0;
  return plan_a8w8(int(M), int(N), int(K), sm_count(), opt_a8w8_balanced()).balanced ? sk_workspace_bytes(sm_count()) : 0;
}

extern "C" int fnn_gemm_a8w8_plan(int64_t M, int64_t N, int64_t K, int* kernel, int* tile_n) {
  using namespace fnn;
  if (!kernel || !tile_n) return fail(FNN_ERR_NULL_POINTER, "gemm_a8w8_plan: null output pointer");
  if (M <= 0 || N <= 0 || K <= 0 || M > INT32_MAX || N > INT32_MAX) return fail(FNN_ERR_SHAPE, "gemm_a8w8_plan: M, N, K must be positive");
  if (M <= 8 && N >= 512 && N % 16 == 0 && K % 4096 == 0) {  // the streaming decode kernel takes these when its own shape rules hold
    *kernel = 2;
    *tile_n = 16;
    return FNN_OK;
  }
  const A8W8Plan plan = plan_a8w8(int(M), int(N), int(K > INT32_MAX ? INT32_MAX : K), sm_count(), opt_a8w8_balanced());
  *kernel = plan.balanced ? 3 : plan.pair ? 1 : 0;
  *tile_n = plan.bn;
  return FNN_OK;
}

extern "C" int fnn_gemm_a8w8(const int8_t* a, int64_t lda, const int8_t* b, int64_t ldb, const void* alpha_row,
                             int row_dtype, const void* alpha_col, int col_dtype, void* out, int out_dtype,
                             int64_t ldo, int64_t M, int64_t N, int64_t K, int32_t* acc_out, int64_t ldacc,
                             void* workspace, size_t workspace_bytes, void* stream) {
  using namespace fnn;
  if (M < 0 || N < 0 || K < 0 || lda < K || ldb < K || ldo < N || (acc_out && ldacc < N))
    return fail(FNN_ERR_SHAPE, "gemm_a8w8: M=%lld N=%lld K=%lld lda=%lld ldb=%lld ldo=%lld", (long long)M,
                (long long)N, (long long)K, (long long)lda, (long long)ldb, (long long)ldo);
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(FNN_ERR_SHAPE, "gemm_a8w8: sizes must be below 2^31");
  if (out_dtype != FNN_F16 && out_dtype != FNN_BF16) return fail(FNN_ERR_DTYPE, "gemm_a8w8: output must be f16 or bf16 (got dtype code %d)", out_dtype);
  if (row_dtype < FNN_F16 || row_dtype > FNN_F32 || col_dtype < FNN_F16 || col_dtype > FNN_F32)
    return fail(FNN_ERR_DTYPE, "gemm_a8w8: scales must be f16, bf16 or f32 (got dtype codes %d, %d)", row_dtype, col_dtype);
  if (M == 0 || N == 0) return FNN_OK;
  if (!a || !b || !alpha_row || !alpha_col || !out) return fail(FNN_ERR_NULL_POINTER, "gemm_a8w8: null tensor pointer");
  A8W8Params p{};
  p.alpha_row = alpha_row; p.alpha_col = alpha_col; p.out = out; p.acc_out = acc_out;
  p.ldo = ldo; p.ldacc = ldacc; p.row_dtype = row_dtype; p.col_dtype = col_dtype;
  p.M = int(M); p.N = int(N); p.K = int(K);
  p.status = device_status_word();
  p.wait_ns = kWaitLimitNs; p.skip_kb = -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == FNN_F16) return dispatch<__half>(a, lda, b, ldb, p, st, workspace, workspace_bytes);
  return dispatch<__nv_bfloat16>(a, lda, b, ldb, p, st, workspace, workspace_bytes);
}
