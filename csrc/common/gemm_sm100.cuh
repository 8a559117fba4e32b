// Persistent, warp-specialised bf16 GEMM mainloop for sm_100a, shared by every GEMM-shaped kernel of
// the library (plain GEMM, fused linear->logprob forward, its recompute backward, grouped expert
// GEMM).  D[M,N] = A[M,K] * B[N,K]^T with fp32 accumulation in tensor memory.
//
//   warp 0      : TMA producer  (cp.async.bulk.tensor 2-D, 128-byte swizzle, STAGES-deep ring)
//   warp 1      : TMEM allocator + single-thread tcgen05.mma issuer (128 x BN x 16 per instruction)
//   warps 2..5  : epilogue; warp w reads TMEM lanes 32*(w%4).. with tcgen05.ld, one accumulator
//                 row per thread, so row-wise reductions need no shuffles
//   warps 6..   : optional communication warps of a fused compute+collective functor (Epi::kCommWarps)
//
// Two accumulators (2 x BN columns) live in TMEM so the epilogue of tile i overlaps the MMAs of
// tile i+1.  Operands may be K-major (row-major [rows, K]) or MN-major (row-major [K, rows]); the
// latter lets the backward GEMMs (dX = dY*W, dW = dY^T*X) run without any transpose pass.
//
// A work item is `n_tiles_per_item` consecutive N-tiles of one M-tile; the epilogue functor keeps
// per-row state across the tiles of an item (used by the online-softmax epilogue).
//
// The kernel allocates all 512 TMEM columns when BN = 256, so at most one CTA may be resident per
// SM: the shared-memory footprint (> 114 KB) guarantees that.
#pragma once

#include "ptx.cuh"

namespace rlk {

constexpr int kBM = 128;
constexpr int kBK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int kGemmThreads = 192;
constexpr int kEpiThreads = 128;

struct GemmProblem {
  int M, N, K;
  int tiles_m, tiles_n;
  int n_tiles_per_item;  // >= 1
  int items_per_m;       // ceil(tiles_n / n_tiles_per_item)
  int num_items;         // tiles_m * items_per_m
  int group_m;           // M-tiles per rasterisation group
  int k_blocks;          // ceil(K / 64)
  // Grouped (mixture-of-experts) modes.  Rows of A are laid out expert by expert, each expert's block
  // padded to a multiple of 128 rows, so an M-tile never straddles two experts.
  //   0: plain GEMM.
  //   1: grouped-M.  D[rows, N] = A[rows, K] * B_g^T with g = tile_group[m_tile]; B holds all groups
  //      stacked along its row axis, b_group_rows rows per group.
  //   2: grouped-K.  D_g[Mg, N] = A[rows_g, Mg]^T * B[rows_g, N] (both operands MN-major), contraction
  //      over the rows of group g = [group_offsets[g], group_offsets[g+1]); D stacks the groups
  //      (tiles_m_per_group M-tiles each).
  int group_mode;
  const int* tile_group;
  const int* group_offsets;
  int b_group_rows;
  int tiles_m_per_group;
  // Tensor-parallel fusions.  m_rot rotates the M-tile order (each rank starts on a different slab).
  // When a_ready is set, the rows of M-tile t of A are produced by another agent (a peer GPU's copy
  // warps) and may be loaded only once a_ready[t] >= a_ready_target.
  int m_rot;
  const unsigned int* a_ready;
  unsigned int a_ready_target;
  unsigned long long a_wait_ns;
};

struct ItemGeometry {
  int a_m0;        // M coordinate of the A tile
  int b_row_off;   // added to B's row coordinate
  int k_row0;      // first contraction index
  int k_blocks;    // 64-wide contraction blocks
};

__host__ __device__ inline GemmProblem make_gemm_problem(int M, int N, int K, int BN, int n_tiles_per_item,
                                                         int group_m) {
  GemmProblem p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.tiles_m = (M + kBM - 1) / kBM;
  p.tiles_n = (N + BN - 1) / BN;
  p.n_tiles_per_item = n_tiles_per_item < 1 ? 1 : n_tiles_per_item;
  p.items_per_m = (p.tiles_n + p.n_tiles_per_item - 1) / p.n_tiles_per_item;
  p.num_items = p.tiles_m * p.items_per_m;
  p.group_m = group_m < 1 ? 1 : group_m;
  p.k_blocks = (K + kBK - 1) / kBK;
  p.group_mode = 0;
  p.tile_group = nullptr;
  p.group_offsets = nullptr;
  p.b_group_rows = 0;
  p.tiles_m_per_group = 1;
  p.m_rot = 0;
  p.a_ready = nullptr;
  p.a_ready_target = 0;
  p.a_wait_ns = 0;
  return p;
}

// M-tiles per rasterisation group.  The A rows of a group are re-read for every N-tile, B is streamed once
// per group: take as many M-tiles as keep the group's A rows within `budget_bytes` of L2 (never fewer than
// `min_group`), so that B comes from DRAM as few times as possible.
inline int raster_group_m(int tiles_m, int K, int min_group, long long budget_bytes = 48ll << 20) {
  const long long per_tile = static_cast<long long>(kBM) * K * 2;
  long long g = budget_bytes / (per_tile > 0 ? per_tile : 1);
  if (g < min_group) g = min_group;
  if (g > tiles_m) g = tiles_m;
  return g < 1 ? 1 : static_cast<int>(g);
}

struct WorkItem {
  int m_tile;
  int split;    // index of the item within its M-tile
  int n_begin;  // first N-tile
  int n_end;    // one past the last N-tile
};

__device__ __forceinline__ WorkItem decode_item(const GemmProblem& p, int id) {
  const int per_group = p.group_m * p.items_per_m;
  const int group = id / per_group;
  const int first_m = group * p.group_m;
  const int gm = min(p.group_m, p.tiles_m - first_m);
  const int within = id - group * per_group;
  WorkItem w;
  w.m_tile = first_m + within % gm;
  if (p.m_rot) w.m_tile = (w.m_tile + p.m_rot) % p.tiles_m;
  w.split = within / gm;
  w.n_begin = w.split * p.n_tiles_per_item;
  w.n_end = min(w.n_begin + p.n_tiles_per_item, p.tiles_n);
  return w;
}

__device__ __forceinline__ ItemGeometry item_geometry(const GemmProblem& p, int m_tile) {
  ItemGeometry g;
  g.a_m0 = m_tile * kBM;
  g.b_row_off = 0;
  g.k_row0 = 0;
  g.k_blocks = p.k_blocks;
  if (p.group_mode == 1) {
    g.b_row_off = p.tile_group[m_tile] * p.b_group_rows;
  } else if (p.group_mode == 2) {
    const int grp = m_tile / p.tiles_m_per_group;
    g.a_m0 = (m_tile - grp * p.tiles_m_per_group) * kBM;
    g.k_row0 = p.group_offsets[grp];
    g.k_blocks = (p.group_offsets[grp + 1] - g.k_row0 + kBK - 1) / kBK;
  }
  return g;
}

// Grouped-M mode: a 128-row tile whose group id is negative holds no rows (the unused tail of a
// statically sized slot buffer); the three warp roles skip it alike and its output stays unwritten.
__device__ __forceinline__ bool item_skipped(const GemmProblem& p, int m_tile) {
  return p.group_mode == 1 && p.tile_group[m_tile] < 0;
}

template <int BN, int STAGES, int STAGING = 0>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingOffset = STAGES * kStageBytes;  // output staging for TMA-store epilogues
  static constexpr int kBarrierOffset = kStagingOffset + STAGING;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem base (u32), abort flag (u32)
  static constexpr int kBytes = kBarrierOffset + (2 * STAGES + 4) * 8 + 16;
  static constexpr int kDynamicBytes = kBytes + 1024;  // slack for manual 1024-byte alignment
};

// Context handed to epilogue functors.
struct EpiThread {
  int row_in_tile;  // 0..127 : accumulator row owned by this thread
  uint32_t lane_addr;  // (32 * quadrant) << 16, to be OR-ed into TMEM addresses
};

// Bounded wait until the rows of M-tile `m_tile` of A have landed in this GPU's memory (written by a
// peer with generic stores + release); the fence orders the following TMA (async proxy) reads after it.
__device__ __forceinline__ void wait_a_ready(const GemmProblem& p, int m_tile, volatile uint32_t* abort_flag,
                                             uint32_t* err, uint32_t kernel_id) {
  const unsigned int* flag = p.a_ready + m_tile;
  unsigned int seen = 0;
  uint64_t deadline = 0;
  for (;;) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if (static_cast<int>(seen - p.a_ready_target) >= 0) break;
    if (*abort_flag) return;
    const uint64_t now = global_timer_ns();
    if (deadline == 0) {
      deadline = now + p.a_wait_ns;
    } else if (now > deadline) {
      *abort_flag = 1;
      report_error(err, kErrPeerTimeout, kernel_id, 20);
      return;
    }
    __nanosleep(100);
  }
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

// Number of threads of a kernel instance: the six mainloop warps plus the functor's communication warps.
template <class Epi>
constexpr int gemm_threads() {
  return kGemmThreads + 32 * Epi::kCommWarps;
}

// ELT: bytes per operand element.  2 = bf16 (kind::f16, 64 elements per 128-byte k-block); 1 = e4m3 (kind::f8f6f4,
// 128 elements per k-block, K-major operands only).  Tile bytes, swizzle and descriptors are the same for both.
template <int BN, bool A_MN, bool B_MN, int STAGES, class Epi, int ELT = 2>
__global__ void __launch_bounds__(gemm_threads<Epi>(), 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const GemmProblem p, const __grid_constant__ typename Epi::Params ep, uint32_t* __restrict__ err,
                  const uint32_t kernel_id) {
  using L = GemmSmem<BN, STAGES, Epi::kStagingBytes>;
  static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "BN must be 64, 128, 192 or 256");
  static_assert(ELT == 2 || (ELT == 1 && !A_MN && !B_MN), "8-bit operands must be K-major");
  constexpr int kBKElems = kBK * 2 / ELT;  // elements of one 128-byte k-block
  constexpr uint32_t kTmemCols = (2 * BN <= 128) ? 128 : (2 * BN <= 256 ? 256 : 512);
  static_assert(kTmemCols <= 256 || L::kDynamicBytes > 116 * 1024,
                "a kernel that takes all of TMEM must not share its SM with another CTA");

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

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], kEpiThreads);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      // Once a bounded wait has given up (abort flag), nothing more is issued: no further loads for the remaining
      // items, so the teardown only has to outlast the copies that were already in flight.
      for (int id = blockIdx.x; id < p.num_items && !*abort_flag; id += gridDim.x) {
        const WorkItem w = decode_item(p, id);
        if (item_skipped(p, w.m_tile)) continue;
        const ItemGeometry geo = item_geometry(p, w.m_tile);
        const int m0 = geo.a_m0;
        if (p.a_ready != nullptr) wait_a_ready(p, w.m_tile, abort_flag, err, kernel_id);
        for (int nt = w.n_begin; nt < w.n_end && !*abort_flag; ++nt) {
          const int n0 = nt * BN;
          for (int kb = 0; kb < geo.k_blocks; ++kb) {
            mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, err, kernel_id, 1);
            if (*abort_flag) break;
            uint8_t* sa = smem + stage * L::kStageBytes;
            uint8_t* sb = sa + L::kABytes;
            mbar_arrive_expect_tx(&full_bar[stage], L::kStageBytes);
            const int k0 = geo.k_row0 + kb * kBKElems;
            if constexpr (!A_MN) {
              tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < kBM / 64; ++j) tma_load_2d(sa + j * 8192, &tmap_a, &full_bar[stage], m0 + j * 64, k0);
            }
            if constexpr (!B_MN) {
              tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0 + geo.b_row_off);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[stage], n0 + j * 64, k0 + geo.b_row_off);
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
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = ELT == 1 ? umma_idesc_e4m3(kBM, BN) : umma_idesc_bf16(kBM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      for (int id = blockIdx.x; id < p.num_items && !*abort_flag; id += gridDim.x) {
        const WorkItem w = decode_item(p, id);
        if (item_skipped(p, w.m_tile)) continue;
        const int item_k_blocks = item_geometry(p, w.m_tile).k_blocks;
        for (int nt = w.n_begin; nt < w.n_end && !*abort_flag; ++nt) {
          mbar_wait(&tmem_empty[buf], buf_phase ^ 1, abort_flag, err, kernel_id, 2);
          if (*abort_flag) break;  // no MMAs on operands that may never have arrived
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          for (int kb = 0; kb < item_k_blocks; ++kb) {
            mbar_wait(&full_bar[stage], phase, abort_flag, err, kernel_id, 3);
            if (*abort_flag) break;
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
            const uint32_t sb = sa + L::kABytes;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k) {
              const uint64_t da = A_MN ? umma_smem_desc_sw128(sa + k * 2048, 8192, 1024)
                                       : umma_smem_desc_sw128(sa + k * 32, 16, 1024);
              const uint64_t db = B_MN ? umma_smem_desc_sw128(sb + k * 2048, 8192, 1024)
                                       : umma_smem_desc_sw128(sb + k * 32, 16, 1024);
              if constexpr (ELT == 1) umma_f8(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
              else umma_bf16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          umma_commit(&tmem_full[buf]);  // accumulator complete
          if (++buf == 2) {
            buf = 0;
            buf_phase ^= 1;
          }
        }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------ communication warps (optional) ------------------------------
    if constexpr (Epi::kCommWarps > 0) Epi::comm(ep, p, err, kernel_id);
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    EpiThread t;
    t.row_in_tile = quad * 32 + lane;
    t.lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    int buf = 0;
    uint32_t buf_phase = 0;
    typename Epi::State st;
    if constexpr (Epi::kStagingBytes > 0) st.staging = smem + L::kStagingOffset;
    Epi::start(ep, p);
    for (int id = blockIdx.x; id < p.num_items; id += gridDim.x) {
      const WorkItem w = decode_item(p, id);
      if (item_skipped(p, w.m_tile)) continue;
      const int row = w.m_tile * kBM + t.row_in_tile;
      Epi::begin_item(st, ep, p, w, row);
      for (int nt = w.n_begin; nt < w.n_end; ++nt) {
        mbar_wait(&tmem_full[buf], buf_phase, abort_flag, err, kernel_id, 4);
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * BN + t.lane_addr;
        Epi::template tile<BN>(st, ep, p, acc, row, nt * BN);
        tc_fence_before();
        mbar_arrive(&tmem_empty[buf]);
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
    // Give copies that may still be in flight time to land before the CTA's smem is released.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Epilogue: store (or accumulate into) a row-major C[M, ldc].
// ---------------------------------------------------------------------------------------------
template <typename OutT, bool ACCUMULATE>
struct EpiStore {
  struct Params {
    OutT* C;
    long long ldc;
    float alpha;
  };
  struct State {};
  static constexpr int kCommWarps = 0;
  static constexpr int kStagingBytes = 0;

  __device__ static void begin_item(State&, const Params&, const GemmProblem&, const WorkItem&, int) {}
  __device__ static void end_item(State&, const Params&, const GemmProblem&, const WorkItem&, int) {}
  __device__ static void finish(const Params&, const GemmProblem&, uint32_t) {}
  __device__ static void start(const Params&, const GemmProblem&) {}

  template <int BN>
  __device__ static void tile(State&, const Params& ep, const GemmProblem& p, uint32_t acc, int row, int n0) {
    const bool row_ok = row < p.M;
    OutT* crow = ep.C + static_cast<long long>(row) * ep.ldc;
    const bool vec_ok = (ep.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(ep.C) & 15u) == 0);
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(acc + c, r);
      tmem_ld_wait();
      const int col0 = n0 + c;
      if (!row_ok || col0 >= p.N) continue;
      if constexpr (sizeof(OutT) == 2) {
        if (vec_ok && col0 + 32 <= p.N) {
          uint4* dst = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float lo = __uint_as_float(r[v * 8 + 2 * j]) * ep.alpha;
              float hi = __uint_as_float(r[v * 8 + 2 * j + 1]) * ep.alpha;
              if constexpr (ACCUMULATE) {
                lo += __bfloat162float(crow[col0 + v * 8 + 2 * j]);
                hi += __bfloat162float(crow[col0 + v * 8 + 2 * j + 1]);
              }
              __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
              w[j] = *reinterpret_cast<uint32_t*>(&b);
            }
            dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        } else {
          for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
            float x = __uint_as_float(r[j]) * ep.alpha;
            if constexpr (ACCUMULATE) x += __bfloat162float(crow[col0 + j]);
            crow[col0 + j] = __float2bfloat16_rn(x);
          }
        }
      } else {
        if (((ep.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(ep.C) & 15u) == 0) && col0 + 32 <= p.N) {
          float4* dst = reinterpret_cast<float4*>(crow + col0);
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            float4 o;
            o.x = __uint_as_float(r[v * 4 + 0]) * ep.alpha;
            o.y = __uint_as_float(r[v * 4 + 1]) * ep.alpha;
            o.z = __uint_as_float(r[v * 4 + 2]) * ep.alpha;
            o.w = __uint_as_float(r[v * 4 + 3]) * ep.alpha;
            if constexpr (ACCUMULATE) {
              const float4 old = dst[v];
              o.x += old.x;
              o.y += old.y;
              o.z += old.z;
              o.w += old.w;
            }
            dst[v] = o;
          }
        } else {
          for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
            float x = __uint_as_float(r[j]) * ep.alpha;
            if constexpr (ACCUMULATE) x += crow[col0 + j];
            crow[col0 + j] = x;
          }
        }
      }
    }
  }
};

// ---------------------------------------------------------------------------------------------
// Epilogue with coalesced output: the accumulator tile is converted to bf16 into a 128B-swizzled staging
// tile in shared memory, COLS columns at a time, and written by TMA bulk-tensor stores (64 columns x 128 rows
// each) instead of thousands of scattered 16-byte stores.  Full 128-byte lines reach L2, and the M / N tails
// are clipped by the tensor map.  Needs a 16-byte aligned C with a 16-byte row pitch; the launchers fall back to
// EpiStore otherwise.  COLS = 256 stages a whole tile (64 KB), COLS = 128 half a tile (32 KB).
// ---------------------------------------------------------------------------------------------
template <int COLS>
struct EpiStoreTma {
  struct Params {
    CUtensorMap tmap_c;  // bf16 [M, N], box 64 x 128, 128B swizzle
    float alpha;
  };
  struct State {
    uint8_t* staging;
  };
  static constexpr int kCommWarps = 0;
  static constexpr int kStagingBytes = kBM * COLS * 2;

  __device__ static void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

  __device__ static void begin_item(State&, const Params&, const GemmProblem&, const WorkItem&, int) {}
  __device__ static void end_item(State&, const Params&, const GemmProblem&, const WorkItem&, int) {}
  __device__ static void start(const Params&, const GemmProblem&) {}
  __device__ static void finish(const Params&, const GemmProblem&, uint32_t) {
    if (threadIdx.x == 64) tma_store_wait<0>();  // the stores must have drained before the CTA's smem goes away
  }

  template <int BN>
  __device__ static void tile(State& st, const Params& ep, const GemmProblem& p, uint32_t acc, int row, int n0) {
    static_assert(BN % COLS == 0 && COLS % 64 == 0, "staging width must divide the tile width");
    const int r = ((threadIdx.x >> 5) & 3) * 32 + (threadIdx.x & 31);  // row inside the tile = TMEM lane of this thread
    const int m0 = row - r;                                             // first row of this CTA's tile
#pragma unroll 1
    for (int seg = 0; seg < BN; seg += COLS) {
      // the previous stores have finished READING the staging tile
      if (threadIdx.x == 64) tma_store_wait_read<0>();
      epi_bar();
#pragma unroll 1
      for (int c = 0; c < COLS; c += 32) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(acc + seg + c, t);
        tmem_ld_wait();
        uint8_t* box = st.staging + (c >> 6) * (kBM * 128) + r * 128;  // 64-column box, 128 bytes per row
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(t[v * 8 + 2 * j]) * ep.alpha,
                                                     __uint_as_float(t[v * 8 + 2 * j + 1]) * ep.alpha);
            w[j] = *reinterpret_cast<uint32_t*>(&b);
          }
          const int chunk = ((c & 63) >> 3) + v;  // 16-byte chunk inside the 128-byte row
          *reinterpret_cast<uint4*>(box + ((chunk ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      fence_proxy_async_smem();
      epi_bar();
      if (threadIdx.x == 64) {
#pragma unroll
        for (int b = 0; b < COLS / 64; ++b) {
          if (n0 + seg + b * 64 < p.N) tma_store_2d(&ep.tmap_c, st.staging + b * (kBM * 128), n0 + seg + b * 64, m0);
        }
        tma_store_commit();
      }
    }
  }
};

}  // namespace rlk
