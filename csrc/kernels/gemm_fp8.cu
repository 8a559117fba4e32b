// fp8 (e4m3) GEMM with row-wise scales on the tcgen05 mainloop, and the row-wise quantiser that feeds it.
//
//   D[M, N] (bf16) = (A_q[M, K] * B_q[N, K]^T) * scale_a[m] * scale_b[n]
//
// A_q / B_q hold e4m3 codes, K-major; scale_a / scale_b are one fp32 scale per row of A and per row of B (per token and
// per output channel), so that x ~= code * scale.  The mainloop is the persistent warp-specialised kernel of the bf16
// GEMM instantiated for 8-bit operands: the same 128-byte-swizzled 128 x 128-byte and 256 x 128-byte stage tiles now
// hold 128 elements of K per k-block, each tcgen05.mma (kind::f8f6f4) consumes 32 of them, fp32 accumulators in TMEM.
// The scales are applied in the epilogue, so accumulation is exact in the codes.
//
// The reference has no fp8 path (it serves in bf16); this is the optional reduced-precision GEMM for rollout-side
// linears, at twice the tensor-core rate of bf16.
#include "../common/gemm2_sm100.cuh"
#include "../common/gemm_sm100.cuh"
#include "../common/tensormap.h"
#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace rlk {
namespace {

constexpr int kBN = 256;
constexpr int kStages = 4;
constexpr float kE4M3Max = 448.f;

struct EpiStoreRowScaled {
  struct Params {
    __nv_bfloat16* C;
    long long ldc;
    const float* scale_a;  // [M]
    const float* scale_b;  // [N]
  };
  struct State {
    float sa;
  };
  static constexpr int kCommWarps = 0;
  static constexpr int kStagingBytes = 0;

  __device__ static void start(const Params&, const GemmProblem&) {}
  __device__ static void begin_item(State& st, const Params& ep, const GemmProblem& p, const WorkItem&, int row) {
    st.sa = row < p.M ? ep.scale_a[row] : 0.f;
  }
  __device__ static void end_item(State&, const Params&, const GemmProblem&, const WorkItem&, int) {}
  __device__ static void finish(const Params&, const GemmProblem&, uint32_t) {}

  template <int BN>
  __device__ static void tile(State& st, const Params& ep, const GemmProblem& p, uint32_t acc, int row, int n0) {
    const bool row_ok = row < p.M;
    __nv_bfloat16* crow = ep.C + static_cast<long long>(row) * ep.ldc;
    const bool vec_ok = (ep.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(ep.C) & 15u) == 0);
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(acc + c, r);
      tmem_ld_wait();
      const int col0 = n0 + c;
      if (!row_ok || col0 >= p.N) continue;
      if (vec_ok && col0 + 32 <= p.N) {
        uint4* dst = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const float4 s0 = *reinterpret_cast<const float4*>(ep.scale_b + col0 + v * 8);
          const float4 s1 = *reinterpret_cast<const float4*>(ep.scale_b + col0 + v * 8 + 4);
          const float sb[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float lo = __uint_as_float(r[v * 8 + 2 * j]) * st.sa * sb[2 * j];
            const float hi = __uint_as_float(r[v * 8 + 2 * j + 1]) * st.sa * sb[2 * j + 1];
            __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
            w[j] = *reinterpret_cast<uint32_t*>(&b);
          }
          dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
        for (int j = 0; j < 32 && col0 + j < p.N; ++j)
          crow[col0 + j] = __float2bfloat16_rn(__uint_as_float(r[j]) * st.sa * ep.scale_b[col0 + j]);
      }
    }
  }
};

// One block per row: amax -> scale = amax / 448 (1 for an all-zero row), codes = round-to-nearest-even of x / scale,
// saturating.  `cols` is the logical width; codes beyond it up to `ldq` are written as zero so that the GEMM's
// k-tail reads zeros.
__global__ void quantize_rows_e4m3_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int cols, uint8_t* __restrict__ q,
                                          long long ldq, float* __restrict__ scale) {
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * ldx;
  // eight elements per access when the row starts on a 16-byte boundary (the second pass re-reads from L1 / L2)
  const bool vec = (ldx % 8 == 0) && (ldq % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) &&
                   ((reinterpret_cast<uintptr_t>(q) & 7u) == 0);
  const int nvec = vec ? cols / 8 : 0;
  float amax = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(xr)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  for (int c = nvec * 8 + threadIdx.x; c < cols; c += blockDim.x) amax = fmaxf(amax, fabsf(__bfloat162float(xr[c])));
  __shared__ float red[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  amax = red[0];
  const float s = amax > 0.f ? amax / kE4M3Max : 1.f;
  if (threadIdx.x == 0) scale[row] = s;
  const float inv = 1.f / s;
  uint8_t* qr = q + row * ldq;
  auto code = [inv](float v) { return static_cast<uint32_t>(__nv_cvt_float_to_fp8(v * inv, __NV_SATFINITE, __NV_E4M3)); };
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(xr)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      w[j >> 1] |= (code(f.x) | (code(f.y) << 8)) << (16 * (j & 1));
    }
    reinterpret_cast<uint2*>(qr)[i] = make_uint2(w[0], w[1]);
  }
  for (long long c = nvec * 8 + threadIdx.x; c < ldq; c += blockDim.x)
    qr[c] = c < cols ? static_cast<uint8_t>(code(__bfloat162float(xr[c]))) : uint8_t(0);
}

}  // namespace

void quantize_rows_e4m3(const void* x, long long ldx, long long rows, int cols, void* q, long long ldq, float* scale,
                        cudaStream_t stream) {
  if (rows <= 0) return;
  quantize_rows_e4m3_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, cols, static_cast<uint8_t*>(q), ldq, scale);
}

void gemm_fp8_rowscaled(const void* a_q, long long lda, const float* scale_a, const void* b_q, long long ldb,
                        const float* scale_b, void* d, long long ldd, int M, int N, int K, bool cta_pair, int sm_count,
                        uint32_t* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return;
  // one k-block = 128 bytes = 128 codes: the problem descriptor counts k-blocks of 64 two-byte elements
  const int k_units = (K + 1) / 2;
  EpiStoreRowScaled::Params ep{static_cast<__nv_bfloat16*>(d), ldd, scale_a, scale_b};
  const CUtensorMap ta = make_tmap_2d_u8(a_q, M, K, lda, kBM, 128);
  if (cta_pair) {
    // 256 x 256 tiles on SM pairs: every SM loads its 128 rows of A and half of the B tile, i.e. 32 KB instead of
    // 48 KB per k-block, which matters twice as much as for bf16 because a k-block is consumed in half the time
    constexpr int kPairStages = 6;
    GemmProblem p = make_gemm_problem(M, N, k_units, kBN, 1, 1);
    p.tiles_m = (M + kPairBM - 1) / kPairBM;
    p.num_items = p.tiles_m * p.items_per_m;
    p.group_m = raster_group_m(p.tiles_m, 2 * k_units, 4);
    const CUtensorMap tb = make_tmap_2d_u8(b_q, N, K, ldb, kBN / 2, 128);
    auto kernel = gemm_pair_sm100_kernel<kBN, false, false, kPairStages, EpiStoreRowScaled, 1>;
    using L = PairSmem<kBN, kPairStages, 0>;
    static PerDeviceOnce configured;
    if (configured.first()) {
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
    }
    int pairs = sm_count / 2;
    if (p.num_items < pairs) pairs = p.num_items;
    if (pairs < 1) return;
    kernel<<<2 * pairs, kGemmThreads, L::kDynamicBytes, stream>>>(ta, tb, p, ep, err, 112u);
    return;
  }
  const int group_m = raster_group_m((M + kBM - 1) / kBM, k_units, 8);
  GemmProblem p = make_gemm_problem(M, N, k_units, kBN, 1, group_m);
  const CUtensorMap tb = make_tmap_2d_u8(b_q, N, K, ldb, kBN, 128);
  auto kernel = gemm_sm100_kernel<kBN, false, false, kStages, EpiStoreRowScaled, 1>;
  using L = GemmSmem<kBN, kStages, 0>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  }
  const int grid = p.num_items < sm_count ? p.num_items : sm_count;
  kernel<<<grid, kGemmThreads, L::kDynamicBytes, stream>>>(ta, tb, p, ep, err, 111u);
}

}  // namespace rlk
