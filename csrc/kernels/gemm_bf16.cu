// Plain bf16 GEMM on the shared tcgen05 mainloop: every operand layout (NT / NN / TN / TT) and
// bf16 or fp32 output, optionally accumulating into the destination.  The reference has no GEMM of
// its own (it calls cuBLAS through torch.matmul, e.g. rl_engine/kernels/ops/pytorch/loss/
// linear_logp.py:17-38); this kernel exists so that no hot path needs a library GEMM.
#include <cstdlib>

#include "../common/gemm2_sm100.cuh"
#include "../common/gemm_sm100.cuh"
#include "../common/tensormap.h"
#include "kernels.h"

namespace rlk {

namespace {

constexpr int kBN = 256;
constexpr int kStages = 4;

// RLK_GEMM_GROUP_M=<n> fixes the number of M-tiles per rasterisation group on both tile engines (a tuning aid for
// shape sweeps; unset or 0 = the L2-budget rule of raster_group_m).
int group_m_override() {
  static const int v = [] {
    const char* env = std::getenv("RLK_GEMM_GROUP_M");
    return env != nullptr ? std::atoi(env) : 0;
  }();
  return v;
}

template <bool A_MN, bool B_MN, class Epi>
void launch(const GemmArgs& a, const typename Epi::Params& ep, cudaStream_t stream) {
  // Rasterise in groups of M-tiles so concurrently running CTAs share A and B tiles in L2 (at least 8; for
  // a plain GEMM as many as keep the group's A rows L2-resident, so that B streams from DRAM once per group).
  const int total_m = a.group_mode == 2 ? a.M * a.num_groups : a.M;
  int group_m = a.group_mode == 0 ? raster_group_m((total_m + kBM - 1) / kBM, a.K, 8) : 8;
  if (a.group_mode == 0 && group_m_override() > 0) group_m = group_m_override();
  GemmProblem p = make_gemm_problem(total_m, a.N, a.K, kBN, 1, group_m);
  const int g = a.group_mode ? a.num_groups : 1;
  p.group_mode = a.group_mode;
  p.tile_group = a.tile_group;
  p.group_offsets = a.group_offsets;
  p.tiles_m_per_group = a.group_mode == 2 ? a.M / kBM : 1;
  // B stacks the groups along its row axis: N rows per group when K-major, K rows per group when MN-major
  p.b_group_rows = a.group_mode == 1 ? (B_MN ? a.K : a.N) : 0;
  const int b_stack = a.group_mode == 1 ? g : 1;
  const CUtensorMap ta = A_MN ? make_tmap_2d_bf16(a.A, a.K, a.M, a.lda, kBK, 64)
                              : make_tmap_2d_bf16(a.A, a.M, a.K, a.lda, kBM, kBK);
  const CUtensorMap tb = B_MN ? make_tmap_2d_bf16(a.B, static_cast<uint64_t>(a.K) * b_stack, a.N, a.ldb, kBK, 64)
                              : make_tmap_2d_bf16(a.B, static_cast<uint64_t>(a.N) * b_stack, a.K, a.ldb, kBN, kBK);
  auto kernel = gemm_sm100_kernel<kBN, A_MN, B_MN, kStages, Epi>;
  using L = GemmSmem<kBN, kStages, Epi::kStagingBytes>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  }
  int grid = p.num_items < a.sm_count ? p.num_items : a.sm_count;
  if (grid < 1) return;
  kernel<<<grid, kGemmThreads, L::kDynamicBytes, stream>>>(ta, tb, p, ep, a.err, 100u);
}

// RLK_GEMM_TMA_STORE=0 keeps the pair kernel on the direct-store epilogue (for A/B comparisons).
bool pair_tma_store_disabled() {
  static const bool off = [] {
    const char* env = std::getenv("RLK_GEMM_TMA_STORE");
    return env != nullptr && env[0] == '0';
  }();
  return off;
}

// CTA-pair kernel: 256 x 256 tiles, one work item per pair of SMs.
constexpr int kPairStages = 6;
constexpr int kPairStagesTma = 5;  // one ring stage makes room for the 64 KB output staging tile

template <bool A_MN, bool B_MN, class Epi, int STAGES = kPairStages>
void launch_pair(const GemmArgs& a, const typename Epi::Params& ep, cudaStream_t stream) {
  GemmProblem p = make_gemm_problem(a.M, a.N, a.K, kBN, 1, 1);
  p.tiles_m = (a.M + kPairBM - 1) / kPairBM;
  p.num_items = p.tiles_m * p.items_per_m;
  // at least eight 256-row tiles per group: with fewer, B streams from DRAM too often on long-K problems (measured:
  // groups of 8 beat 4-6 by 2-4 % on K = 14336 / 28672, groups of 32 and more lose 5-10 % on every shape)
  p.group_m = raster_group_m(p.tiles_m, 2 * a.K, 8);
  if (group_m_override() > 0) p.group_m = group_m_override() < p.tiles_m ? group_m_override() : p.tiles_m;
  const CUtensorMap ta = A_MN ? make_tmap_2d_bf16(a.A, a.K, a.M, a.lda, kBK, 64)
                              : make_tmap_2d_bf16(a.A, a.M, a.K, a.lda, kBM, kBK);
  const CUtensorMap tb = B_MN ? make_tmap_2d_bf16(a.B, a.K, a.N, a.ldb, kBK, 64)
                              : make_tmap_2d_bf16(a.B, a.N, a.K, a.ldb, kBN / 2, kBK);
  auto kernel = gemm_pair_sm100_kernel<kBN, A_MN, B_MN, STAGES, Epi>;
  using L = PairSmem<kBN, STAGES, Epi::kStagingBytes>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  }
  int pairs = a.sm_count / 2;
  if (p.num_items < pairs) pairs = p.num_items;
  if (pairs < 1) return;
  kernel<<<2 * pairs, kGemmThreads, L::kDynamicBytes, stream>>>(ta, tb, p, ep, a.err, 110u);
}

// Skinny problems (one 128-row tile of A, e.g. the G tokens of a decoding step): the GEMM is a stream over the
// weight matrix, so parallelism has to come from N.  64-column tiles give four times as many CTAs as the 256-column
// engine (N = 4096: 64 instead of 16) and an 8-stage ring of 24 KB keeps enough loads in flight per SM.
constexpr int kSkinnyBN = 64;
constexpr int kSkinnyStages = 8;

void launch_skinny(const GemmArgs& a, cudaStream_t stream) {
  using Epi = EpiStore<__nv_bfloat16, false>;
  GemmProblem p = make_gemm_problem(a.M, a.N, a.K, kSkinnyBN, 1, 1);
  const CUtensorMap ta = make_tmap_2d_bf16(a.A, a.M, a.K, a.lda, kBM, kBK);
  const CUtensorMap tb = make_tmap_2d_bf16(a.B, a.N, a.K, a.ldb, kSkinnyBN, kBK);
  auto kernel = gemm_sm100_kernel<kSkinnyBN, false, false, kSkinnyStages, Epi>;
  using L = GemmSmem<kSkinnyBN, kSkinnyStages, 0>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  }
  const int grid = p.num_items < a.sm_count ? p.num_items : a.sm_count;
  if (grid < 1) return;
  kernel<<<grid, kGemmThreads, L::kDynamicBytes, stream>>>(
      ta, tb, p, typename Epi::Params{static_cast<__nv_bfloat16*>(a.D), a.ldd, a.alpha}, a.err, 101u);
}

template <bool A_MN, bool B_MN>
void dispatch_out(const GemmArgs& a, cudaStream_t stream) {
  if constexpr (!A_MN && !B_MN) {
    if (a.group_mode == 0 && a.M <= kBM && !a.out_fp32 && !a.accumulate && a.N >= 4 * kSkinnyBN) {
      launch_skinny(a, stream);
      return;
    }
  }
  if (!(a.cta_pair && a.group_mode == 0)) {
    // single-CTA engine, bf16 output that TMA can address: half-tile staging (32 KB next to the 4-stage ring)
    const bool tma_out = !a.out_fp32 && !a.accumulate && a.ldd % 8 == 0 && (reinterpret_cast<uintptr_t>(a.D) & 15u) == 0 &&
                         !pair_tma_store_disabled();
    if (tma_out) {
      EpiStoreTma<128>::Params ep;
      // grouped-K stacks one [M, N] block per group along the rows of D
      ep.tmap_c = make_tmap_2d_bf16(a.D, a.group_mode == 2 ? static_cast<uint64_t>(a.M) * a.num_groups : a.M, a.N, a.ldd, kBM, 64);
      ep.alpha = a.alpha;
      launch<A_MN, B_MN, EpiStoreTma<128>>(a, ep, stream);
      return;
    }
  }
  if (a.cta_pair && a.group_mode == 0) {
    // bf16 output that TMA can address: stage the tile in shared memory and store full lines
    const bool tma_out = !a.out_fp32 && !a.accumulate && a.ldd % 8 == 0 && (reinterpret_cast<uintptr_t>(a.D) & 15u) == 0 &&
                         !pair_tma_store_disabled();
    if (tma_out) {
      EpiStoreTma<256>::Params ep;
      ep.tmap_c = make_tmap_2d_bf16(a.D, a.M, a.N, a.ldd, kBM, 64);
      ep.alpha = a.alpha;
      launch_pair<A_MN, B_MN, EpiStoreTma<256>, kPairStagesTma>(a, ep, stream);
      return;
    }
    if (a.out_fp32) {
      if (a.accumulate) {
        using E = EpiStore<float, true>;
        launch_pair<A_MN, B_MN, E>(a, typename E::Params{static_cast<float*>(a.D), a.ldd, a.alpha}, stream);
      } else {
        using E = EpiStore<float, false>;
        launch_pair<A_MN, B_MN, E>(a, typename E::Params{static_cast<float*>(a.D), a.ldd, a.alpha}, stream);
      }
    } else {
      if (a.accumulate) {
        using E = EpiStore<__nv_bfloat16, true>;
        launch_pair<A_MN, B_MN, E>(a, typename E::Params{static_cast<__nv_bfloat16*>(a.D), a.ldd, a.alpha}, stream);
      } else {
        using E = EpiStore<__nv_bfloat16, false>;
        launch_pair<A_MN, B_MN, E>(a, typename E::Params{static_cast<__nv_bfloat16*>(a.D), a.ldd, a.alpha}, stream);
      }
    }
    return;
  }
  if (a.out_fp32) {
    if (a.accumulate) {
      using E = EpiStore<float, true>;
      launch<A_MN, B_MN, E>(a, typename E::Params{static_cast<float*>(a.D), a.ldd, a.alpha}, stream);
    } else {
      using E = EpiStore<float, false>;
      launch<A_MN, B_MN, E>(a, typename E::Params{static_cast<float*>(a.D), a.ldd, a.alpha}, stream);
    }
  } else {
    if (a.accumulate) {
      using E = EpiStore<__nv_bfloat16, true>;
      launch<A_MN, B_MN, E>(a, typename E::Params{static_cast<__nv_bfloat16*>(a.D), a.ldd, a.alpha}, stream);
    } else {
      using E = EpiStore<__nv_bfloat16, false>;
      launch<A_MN, B_MN, E>(a, typename E::Params{static_cast<__nv_bfloat16*>(a.D), a.ldd, a.alpha}, stream);
    }
  }
}

}  // namespace

void gemm_bf16(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return;
  if (a.a_mn_major) {
    if (a.b_mn_major) dispatch_out<true, true>(a, stream);
    else dispatch_out<true, false>(a, stream);
  } else {
    if (a.b_mn_major) dispatch_out<false, true>(a, stream);
    else dispatch_out<false, false>(a, stream);
  }
}

}  // namespace rlk
