// CTA-pair variant of the persistent bf16 GEMM mainloop: a cluster of two CTAs (one per SM of a pair)
// computes a 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
// Why: with one CTA per 128 x 256 tile every SM pulls (128 + 256) x 64 x 2 = 48 KB of operands through L2 for
// each 64-deep k-step; in a pair each SM loads its own 128 rows of A and only HALF of the B tile (the tensor
// cores of both SMs read both halves), i.e. 32 KB per SM for the same FLOPs: one third less L2 -> SM traffic,
// which is what bounds the single-CTA kernel.  The smaller stages also allow a deeper ring (6 stages).
//
//   both CTAs : warp 0 lane 0  TMA producer for this CTA's A rows and B half; bytes are counted on the EVEN
//                              CTA's full barrier (address mapped into the cluster window)
//   even CTA  : warp 1 lane 0  issues the pair MMAs; tcgen05.commit arrives on both CTAs' barriers
//   both CTAs : warps 2..5     epilogue on this CTA's 128 accumulator rows (TMEM lanes), same functor
//                              interface as the single-CTA kernel; one lane per warp releases the
//                              accumulator to the even CTA's MMA thread
//
// All waits are bounded (mbar_wait).  The pair synchronises on the cluster barrier after set-up and
// before TMEM is released, so neither CTA can leave while its partner may still touch its memory.
#pragma once

#include "gemm_sm100.cuh"

namespace rlk {

constexpr int kPairBM = 256;  // rows of the pair's tile (128 per CTA)

template <int BN, int STAGES, int STAGING = 0>
struct PairSmem {
  static constexpr int kABytes = kBM * kBK * 2;         // this CTA's A rows
  static constexpr int kBBytes = (BN / 2) * kBK * 2;    // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingOffset = STAGES * kStageBytes;  // output staging for TMA-store epilogues
  static constexpr int kBarrierOffset = kStagingOffset + STAGING;
  static constexpr int kBytes = kBarrierOffset + (2 * STAGES + 4) * 8 + 16;
  static constexpr int kDynamicBytes = kBytes + 1024;
};

// ELT: bytes per operand element (2 = bf16, 1 = e4m3 with K-major operands), as in the single-CTA kernel.
template <int BN, bool A_MN, bool B_MN, int STAGES, class Epi, int ELT = 2>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_pair_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const GemmProblem p, const __grid_constant__ typename Epi::Params ep, uint32_t* __restrict__ err,
                       const uint32_t kernel_id) {
  using L = PairSmem<BN, STAGES, Epi::kStagingBytes>;
  static_assert(BN == 256, "the pair kernel uses 256-wide N tiles (128 columns of B per CTA)");
  static_assert(Epi::kCommWarps == 0, "communication warps are not supported by the pair kernel");
  static_assert(ELT == 2 || (ELT == 1 && !A_MN && !B_MN), "8-bit operands must be K-major");
  constexpr int kBKElems = kBK * 2 / ELT;  // elements of one 128-byte k-block
  constexpr uint32_t kTmemCols = 512;
  constexpr int kHalfN = BN / 2;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarrierOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0: even CTA (issues the MMAs), 1: its partner
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);   // the even CTA's producer arrives once and announces both CTAs' bytes
      mbar_init(&empty_bar[s], 1);  // one commit arrival per use
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 8);  // one lane of each of the 4 epilogue warps of both CTAs
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_base_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // both CTAs' barriers are initialised before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int id = pair; id < p.num_items; id += num_pairs) {
        const WorkItem w = decode_item(p, id);
        const int m0 = w.m_tile * kPairBM + static_cast<int>(cta) * kBM;
        for (int nt = w.n_begin; nt < w.n_end; ++nt) {
          const int n0 = nt * BN + static_cast<int>(cta) * kHalfN;
          for (int kb = 0; kb < p.k_blocks; ++kb) {
            mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, err, kernel_id, 1);
            uint8_t* sa = smem + stage * L::kStageBytes;
            uint8_t* sb = sa + L::kABytes;
            if (cta == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
            const uint32_t bar = mapa_u32(smem_u32(&full_bar[stage]), 0);
            const int k0 = kb * kBKElems;
            if constexpr (!A_MN) {
              tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < kBM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tmap_a, bar, m0 + j * 64, k0);
            }
            if constexpr (!B_MN) {
              tma_load_2d_pair(sb, &tmap_b, bar, k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < kHalfN / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tmap_b, bar, n0 + j * 64, k0);
            }
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only) ------------------------------
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = ELT == 1 ? umma_idesc_e4m3(kPairBM, BN) : umma_idesc_bf16(kPairBM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      for (int id = pair; id < p.num_items; id += num_pairs) {
        const WorkItem w = decode_item(p, id);
        for (int nt = w.n_begin; nt < w.n_end; ++nt) {
          mbar_wait(&tmem_empty[buf], buf_phase ^ 1, abort_flag, err, kernel_id, 2);
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          for (int kb = 0; kb < p.k_blocks; ++kb) {
            mbar_wait(&full_bar[stage], phase, abort_flag, err, kernel_id, 3);
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
            const uint32_t sb = sa + L::kABytes;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k) {
              const uint64_t da = A_MN ? umma_smem_desc_sw128(sa + k * 2048, 8192, 1024)
                                       : umma_smem_desc_sw128(sa + k * 32, 16, 1024);
              const uint64_t db = B_MN ? umma_smem_desc_sw128(sb + k * 2048, 8192, 1024)
                                       : umma_smem_desc_sw128(sb + k * 32, 16, 1024);
              if constexpr (ELT == 1) umma_f8_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
              else umma_bf16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit_pair(&empty_bar[stage]);  // frees this stage in both CTAs
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          umma_commit_pair(&tmem_full[buf]);  // accumulator complete, in both CTAs
          if (++buf == 2) {
            buf = 0;
            buf_phase ^= 1;
          }
        }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs, own 128 rows) ------------------------------
    const int quad = warp & 3;
    EpiThread t;
    t.row_in_tile = quad * 32 + lane;
    t.lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    int buf = 0;
    uint32_t buf_phase = 0;
    typename Epi::State st;
    if constexpr (Epi::kStagingBytes > 0) st.staging = smem + L::kStagingOffset;
    Epi::start(ep, p);
    for (int id = pair; id < p.num_items; id += num_pairs) {
      const WorkItem w = decode_item(p, id);
      const int row = w.m_tile * kPairBM + static_cast<int>(cta) * kBM + t.row_in_tile;
      Epi::begin_item(st, ep, p, w, row);
      for (int nt = w.n_begin; nt < w.n_end; ++nt) {
        mbar_wait(&tmem_full[buf], buf_phase, abort_flag, err, kernel_id, 4);
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * BN + t.lane_addr;
        Epi::template tile<BN>(st, ep, p, acc, row, nt * BN);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[buf]), 0));
        if (++buf == 2) {
          buf = 0;
          buf_phase ^= 1;
        }
      }
      Epi::end_item(st, ep, p, w, row);
    }
    Epi::finish(ep, p, kernel_id);
  }

  // ------------------------------ teardown ------------------------------
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // the partner has finished reading this CTA's shared memory and signalling its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace rlk
