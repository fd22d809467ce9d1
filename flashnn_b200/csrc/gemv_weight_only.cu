// Weight-only GEMV / skinny GEMM for decode shapes (M <= 16): fp16/bf16
// activations x int8 or packed-int4 weights, per-channel or group-wise scales.
//
// The op is HBM-bound (every weight byte is read exactly once), so the kernel is
// built around 128-bit weight loads that go straight into registers:
//   - a CTA owns 16 output channels (8 packed rows for int4, 16 rows for int8)
//     and its 8 warps split K;
//   - each lane expands its weight bytes to exact 16-bit integers with
//     PRMT/LOP3 bit tricks (no int->float conversions) and uses them as the
//     16 x 16 operand of mma.sync.m16n8k16; the activations are the narrow
//     16 x 8 operand, so one weight fragment serves up to 8 tokens (two MMAs
//     for 9..16 tokens);
//   - the MMA accumulates x*w in fp32 over one scale group; the group scale
//     (and zero-point) is applied to that partial sum in fp32, so w*s is never
//     rounded to 16 bits;
//   - partial sums of the 8 warps meet in shared memory; bias is added in fp32
//     and the result is rounded once.
// Zero-points are applied as  -zp * s * sum_k x  per group, with the per-group
// activation sums produced by a small prologue kernel in caller-provided scratch.
#include "common.cuh"

namespace fnn {
namespace {

constexpr int kGemvWarps = 8;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kStepK = 64;   // K covered by one warp-wide 128-bit load per row (4 lanes x 16 B)
constexpr int kBatch = 4;    // loads in flight per lane

struct WoParams {
  const void* act;      // [M, K] T
  const uint8_t* qw;    // int8 [N, K] or packed [N/2, K]
  const void* scale;    // [N] or [G, N]
  const void* zp;       // nullptr or like scale
  const void* bias;     // nullptr or [N]
  const float* xsum;    // [M, G] activation sums per group (only with zero-points)
  void* out;
  int64_t lda, ldo;
  int scale_dtype, bias_dtype;
  int M, N, K;
  int group;  // 0 = per channel
  int G;      // number of groups along K (1 when per channel)
};

template <typename T> struct Mma;
template <> struct Mma<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct Mma<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b, __half) {
  __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b, __nv_bfloat16) {
  __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

// Four packed bytes (4 consecutive k of one packed row) -> the MMA A fragment:
//   a[0] = low nibbles  (channel 2j)   at k0, k0+1      a[1] = high nibbles (channel 2j+1) at k0, k0+1
//   a[2] = low nibbles  (channel 2j)   at k0+2, k0+3    a[3] = high nibbles (channel 2j+1) at k0+2, k0+3
// each as an exact signed integer in T.
template <typename T> __device__ __forceinline__ void dequant_int4(uint32_t w, uint32_t (&a)[4]);
template <> __device__ __forceinline__ void dequant_int4<__nv_bfloat16>(uint32_t w, uint32_t (&a)[4]) {
  // byte = 0x80 | ((n ^ 8) << 3) under a 0x41 high byte is the bf16 value 16 + (n ^ 8) = n_signed + 24
  const uint32_t lo = ((w << 3) & 0x78787878u) ^ 0xC0C0C0C0u;
  const uint32_t hi = ((w >> 1) & 0x78787878u) ^ 0xC0C0C0C0u;
  const uint32_t m = 0x41414141u, off = 0x41C041C0u;  // 24.0 twice
  a[0] = sub2(prmt(lo, m, 0x4140), off, __nv_bfloat16());
  a[1] = sub2(prmt(hi, m, 0x4140), off, __nv_bfloat16());
  a[2] = sub2(prmt(lo, m, 0x4342), off, __nv_bfloat16());
  a[3] = sub2(prmt(hi, m, 0x4342), off, __nv_bfloat16());
}
template <> __device__ __forceinline__ void dequant_int4<__half>(uint32_t w, uint32_t (&a)[4]) {
  // byte = n ^ 8 under a 0x64 high byte is the fp16 value 1024 + (n ^ 8) = n_signed + 1032
  const uint32_t lo = (w & 0x0F0F0F0Fu) ^ 0x08080808u;
  const uint32_t hi = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
  const uint32_t m = 0x64646464u, off = 0x64086408u;  // 1032.0 twice
  a[0] = sub2(prmt(lo, m, 0x4140), off, __half());
  a[1] = sub2(prmt(hi, m, 0x4140), off, __half());
  a[2] = sub2(prmt(lo, m, 0x4342), off, __half());
  a[3] = sub2(prmt(hi, m, 0x4342), off, __half());
}

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

template <typename T, int BITS, int NT>
__global__ void __launch_bounds__(kGemvThreads)
gemv_mma_kernel(const WoParams p) {
  __shared__ float red[kGemvWarps][NT][4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int ch_base = blockIdx.x * 16;
  // channels behind accumulator registers {0,1} and {2,3}
  const int ch_a = (BITS == 4) ? ch_base + 2 * g : ch_base + g;
  const int ch_b = (BITS == 4) ? ch_a + 1 : ch_a + 8;
  // weight rows this lane streams (clamped; out-of-range channels are never stored)
  const int64_t last_row = (BITS == 4 ? p.N / 2 : p.N) - 1;
  const int64_t row_a = min(int64_t(BITS == 4 ? ch_base / 2 + g : ch_a), last_row);
  const int64_t row_b = min(int64_t(ch_b), last_row);  // int8 only
  const uint8_t* wa = p.qw + row_a * p.K + tig * 16;
  const uint8_t* wb = p.qw + row_b * p.K + tig * 16;
  const T* act = reinterpret_cast<const T*>(p.act);

  // K range of this warp, in units of one scale group (or of 64 when per channel)
  const int unit = p.group > 0 ? p.group : kStepK;
  const int units = p.K / unit;
  const int u0 = int(int64_t(units) * warp / kGemvWarps), u1 = int(int64_t(units) * (warp + 1) / kGemvWarps);
  const int steps_per_unit = unit / kStepK;

  float tot[NT][4], acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) tot[t][i] = acc[t][i] = 0.f;

  const bool tok_ok[2] = {g < p.M, g + 8 < p.M};
  const int total_steps = (u1 - u0) * steps_per_unit;
  int k = u0 * unit;
  int step_in_unit = 0;
  int grp = u0;

  // scale / zero-point of the current group for the two channels of this lane
  auto finish_group = [&](int gi) {
    float sa = 1.f, sb = 1.f, za = 0.f, zb = 0.f;
    if (p.group > 0) {
      const int64_t o = int64_t(gi) * p.N;
      if (ch_a < p.N) { sa = load_as_f32(p.scale, p.scale_dtype, o + ch_a); if (p.zp) za = load_as_f32(p.zp, p.scale_dtype, o + ch_a); }
      if (ch_b < p.N) { sb = load_as_f32(p.scale, p.scale_dtype, o + ch_b); if (p.zp) zb = load_as_f32(p.zp, p.scale_dtype, o + ch_b); }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      float x0 = 0.f, x1 = 0.f;
      if (p.group > 0 && p.zp) {
        const int m0 = t * 8 + 2 * tig;
        if (m0 < p.M) x0 = p.xsum[int64_t(m0) * p.G + gi];
        if (m0 + 1 < p.M) x1 = p.xsum[int64_t(m0 + 1) * p.G + gi];
      }
      tot[t][0] += sa * (acc[t][0] - za * x0);
      tot[t][1] += sa * (acc[t][1] - za * x1);
      tot[t][2] += sb * (acc[t][2] - zb * x0);
      tot[t][3] += sb * (acc[t][3] - zb * x1);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
    }
  };

  for (int s0 = 0; s0 < total_steps; s0 += kBatch) {
    const int nb = min(kBatch, total_steps - s0);
    uint4 wq[kBatch], wq2[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i)
      if (i < nb) {
        wq[i] = __ldcs(reinterpret_cast<const uint4*>(wa + k + i * kStepK));
        if (BITS == 8) wq2[i] = __ldcs(reinterpret_cast<const uint4*>(wb + k + i * kStepK));
      }
#pragma unroll
    for (int i = 0; i < kBatch; ++i)
      if (i < nb) {
        // activations of token g (and g+8): 16 consecutive k starting at k + tig*16
        uint4 xv[NT][2];
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          if (tok_ok[t]) {
            const uint4* xp = reinterpret_cast<const uint4*>(act + int64_t(g + 8 * t) * p.lda + k + i * kStepK + tig * 16);
            xv[t][0] = __ldg(xp);
            xv[t][1] = __ldg(xp + 1);
          } else {
            xv[t][0] = xv[t][1] = make_uint4(0, 0, 0, 0);
          }
        }
        const uint32_t ww[4] = {wq[i].x, wq[i].y, wq[i].z, wq[i].w};
        const uint32_t ww2[4] = {wq2[i].x, wq2[i].y, wq2[i].z, wq2[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t a[4];
          if (BITS == 4) {
            dequant_int4<T>(ww[j], a);
          } else {
            dequant_int8<T>(ww[j], a[0], a[2]);
            dequant_int8<T>(ww2[j], a[1], a[3]);
          }
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const uint32_t xw[8] = {xv[t][0].x, xv[t][0].y, xv[t][0].z, xv[t][0].w,
                                    xv[t][1].x, xv[t][1].y, xv[t][1].z, xv[t][1].w};
            Mma<T>::run(acc[t], a, xw[2 * j], xw[2 * j + 1]);
          }
        }
        if (++step_in_unit == steps_per_unit) {
          step_in_unit = 0;
          if (p.group > 0) finish_group(grp);
          ++grp;
        }
      }
    k += nb * kStepK;
  }
  if (p.group == 0) {
    // per-channel: the whole K range is one group; scale and zero-point are applied after the reduction
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) tot[t][i] = acc[t][i];
  }

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
          if (p.group == 0) {
            const float s = load_as_f32(p.scale, p.scale_dtype, ch);
            if (p.zp) v -= load_as_f32(p.zp, p.scale_dtype, ch) * p.xsum[m];
            v *= s;
          }
          if (p.bias) v += load_as_f32(p.bias, p.bias_dtype, ch);
          out[int64_t(m) * p.ldo + ch] = from_f32<T>(v);
        }
      }
  }
}

// sum of x over each scale group: xsum[m, gi] = sum_{k in group gi} x[m, k]   (one warp per (m, gi))
template <typename T>
__global__ void group_sum_kernel(const T* __restrict__ act, int64_t lda, float* __restrict__ xsum, int M, int K, int G) {
  const int64_t w = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= int64_t(M) * G) return;
  const int m = int(w / G), gi = int(w % G);
  const int len = K / G;
  const T* x = act + int64_t(m) * lda + int64_t(gi) * len;
  float s = 0.f;
  for (int i = lane; i < len; i += 32) s += to_f32(x[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) xsum[w] = s;
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

bool gemv_path_ok(const WoParams& p, int bits) {
  if (p.M > 16) return false;
  if (p.K % kStepK != 0) return false;
  if (p.group > 0 && (p.group % kStepK != 0 || p.K % p.group != 0)) return false;
  if (reinterpret_cast<uintptr_t>(p.qw) % 16 != 0) return false;
  if (reinterpret_cast<uintptr_t>(p.act) % 16 != 0 || p.lda % 8 != 0) return false;
  if (bits == 4 && p.N % 2 != 0) return false;
  return true;
}

template <typename T, int BITS>
int launch_wo(WoParams p, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (!gemv_path_ok(p, BITS)) {
    const int64_t total = int64_t(p.M) * p.N;
    wo_generic_kernel<T, BITS><<<unsigned((total + 255) / 256), 256, 0, st>>>(p);
    return check_cuda(cudaGetLastError(), "weight-only generic launch");
  }
  if (p.zp) {
    const size_t need = size_t(p.M) * p.G * sizeof(float);
    if (!workspace || workspace_bytes < need)
      return fail(FNN_ERR_WORKSPACE, "gemm_weight_only: zero-points need %zu bytes of workspace, got %zu", need, workspace_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return fail(FNN_ERR_ALIGNMENT, "gemm_weight_only: workspace must be 256-byte aligned");
    float* xsum = static_cast<float*>(workspace);
    const int64_t warps = int64_t(p.M) * p.G;
    group_sum_kernel<T><<<unsigned((warps * 32 + 255) / 256), 256, 0, st>>>(reinterpret_cast<const T*>(p.act), p.lda, xsum, p.M, p.K, p.G);
    if (int e = check_cuda(cudaGetLastError(), "group_sum launch")) return e;
    p.xsum = xsum;
  }
  const unsigned grid = unsigned((p.N + 15) / 16);
  if (p.M <= 8) gemv_mma_kernel<T, BITS, 1><<<grid, kGemvThreads, 0, st>>>(p);
  else gemv_mma_kernel<T, BITS, 2><<<grid, kGemvThreads, 0, st>>>(p);
  return check_cuda(cudaGetLastError(), "weight-only gemv launch");
}

}  // namespace
}  // namespace fnn

extern "C" size_t fnn_gemm_weight_only_workspace_bytes(int64_t M, int64_t N, int64_t K, int weight_bits, int64_t group_size) {
  (void)N; (void)weight_bits;
  if (M <= 0 || K <= 0) return 0;
  const int64_t G = group_size > 0 ? (K + group_size - 1) / group_size : 1;
  return size_t(M) * size_t(G) * sizeof(float);  // activation sums per group (used with zero-points)
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
  p.xsum = nullptr; p.out = out; p.lda = lda; p.ldo = ldo; p.scale_dtype = scale_dtype; p.bias_dtype = bias_dtype;
  p.M = int(M); p.N = int(N); p.K = int(K); p.group = int(group_size); p.G = group_size > 0 ? int(K / group_size) : 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (act_dtype == FNN_F16)
    return weight_bits == 4 ? launch_wo<__half, 4>(p, workspace, workspace_bytes, st) : launch_wo<__half, 8>(p, workspace, workspace_bytes, st);
  return weight_bits == 4 ? launch_wo<__nv_bfloat16, 4>(p, workspace, workspace_bytes, st) : launch_wo<__nv_bfloat16, 8>(p, workspace, workspace_bytes, st);
}
