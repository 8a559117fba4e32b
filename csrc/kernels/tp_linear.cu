// Tensor-parallel linears fused with their collectives, on the shared tcgen05 mainloop.
//
//   tp_ag_gemm : C[M, N] = allgather_rows(X_local)[M, K] * B^T.   Two extra warps per CTA copy this rank's
//                rows of X into every rank's gathered buffer with plain peer stores (128-row tile by tile,
//                own rank first) and publish a per-tile arrival count; the TMA producer of each CTA waits for
//                the count of the M-tile it is about to load, so the math on the tiles that have landed
//                overlaps the transfer of the rest.  The gathered rows cross NVLink once and are then
//                read by TMA from this GPU's own memory.
//   tp_gemm_rs : out[M / W, N] = reduce_scatter_rows(A[M, K_local] * B^T).   The epilogue stores each
//                partial tile as bf16 straight into the slab of the rank that owns its rows and bumps
//                that rank's arrival counter; after its GEMM items every CTA turns to the tiles owned
//                here and, once all W partials of a tile have arrived, sums them in rank order in fp32.
//
// Every cross-GPU wait is bounded and reports through the error word.  Buffers and counters are
// double-buffered by call parity: a peer can be at most one call ahead, because finishing call n needs
// data that this rank only sends from inside its own call n.  Counters are monotonic (never reset).
//
// The reference has no tensor-parallel linear; its only TP-aware op is the vocab-parallel log-prob
// (rl_engine/kernels/ops/pytorch/loss/linear_logp.py:176-377), which goes through NCCL all-reduces.
#include "../common/gemm_sm100.cuh"
#include "../common/tensormap.h"
#include "kernels.h"

namespace rlk {

namespace {

constexpr int kBN = 256;
constexpr int kStages = 4;
constexpr int kCommThreads = 64;

struct PeerPtrs {
  void* p[8];
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void comm_bar_sync() { asm volatile("bar.sync 2, 64;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// all-gather -> GEMM
// ---------------------------------------------------------------------------------------------
struct AgParams {
  EpiStoreTma<128>::Params store;  // output tensor map (bf16 [M, N]) + alpha, used by the staged TMA-store epilogue
  const __nv_bfloat16* x_local;    // [rows_local, K]
  long long ldx;
  int rows_local;
  int k;        // elements per row (multiple of 8 * chunks)
  int chunks;   // column chunks per 128-row tile = arrivals per tile and call
  int rank, world;
  PeerPtrs gathered;  // bf16 [M, K] on every rank
  PeerPtrs ready;     // unsigned int [tiles_m] on every rank
};

struct EpiAgStore {
  using Params = AgParams;
  using Store = EpiStoreTma<128>;  // half-tile staging + TMA bulk stores: full lines to L2
  using State = Store::State;
  static constexpr int kCommWarps = kCommThreads / 32;
  static constexpr int kStagingBytes = Store::kStagingBytes;

  __device__ static void begin_item(State&, const Params&, const GemmProblem&, const WorkItem&, int) {}
  __device__ static void end_item(State&, const Params&, const GemmProblem&, const WorkItem&, int) {}
  __device__ static void finish(const Params& ep, const GemmProblem& p, uint32_t id) { Store::finish(ep.store, p, id); }
  __device__ static void start(const Params&, const GemmProblem&) {}

  template <int BN>
  __device__ static void tile(State& st, const Params& ep, const GemmProblem& p, uint32_t acc, int row, int n0) {
    Store::template tile<BN>(st, ep.store, p, acc, row, n0);
  }

  // Copy units (tile, chunk) are striped over the CTAs; each unit goes to every rank, own rank first.
  __device__ static void comm(const Params& ep, const GemmProblem&, uint32_t*, uint32_t) {
    const int tid = threadIdx.x - kGemmThreads;
    const int tiles_local = ep.rows_local / kBM;
    const int vec_row = ep.k / 8;                 // 16-byte vectors per row
    const int vec_chunk = vec_row / ep.chunks;    // vectors per row of one unit
    const long long ldx_vec = ep.ldx / 8;
    const int units = tiles_local * ep.chunks;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const int t = u / ep.chunks;
      const int c0 = (u - t * ep.chunks) * vec_chunk;
      const uint4* src = reinterpret_cast<const uint4*>(ep.x_local) + static_cast<long long>(t) * kBM * ldx_vec + c0;
      for (int step = 0; step < ep.world; ++step) {
        const int peer = (ep.rank + step) % ep.world;
        uint4* dst = static_cast<uint4*>(ep.gathered.p[peer]) +
                     (static_cast<long long>(ep.rank) * ep.rows_local + static_cast<long long>(t) * kBM) * vec_row + c0;
        for (int r = 0; r < kBM; ++r) {
          const uint4* s = src + r * ldx_vec;
          uint4* d = dst + static_cast<long long>(r) * vec_row;
#pragma unroll 4
          for (int c = tid; c < vec_chunk; c += kCommThreads) d[c] = s[c];
        }
        __threadfence_system();
        comm_bar_sync();
        if (tid == 0) {
          unsigned int* flag = static_cast<unsigned int*>(ep.ready.p[peer]) + ep.rank * tiles_local + t;
          asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(flag), "r"(1u) : "memory");
        }
      }
    }
  }
};

// ---------------------------------------------------------------------------------------------
// GEMM -> reduce-scatter
// ---------------------------------------------------------------------------------------------
struct RsParams {
  PeerPtrs partial;   // bf16 [world, rows_local, N] on every rank
  PeerPtrs counters;  // unsigned int [tiles_local * tiles_n] on every rank
  __nv_bfloat16* out; // [rows_local, N]
  long long ldo;
  int rows_local;
  int rank, world;
  unsigned int target;  // arrivals per tile counter once every rank has delivered this call's partial
  unsigned long long wait_ns;
  uint32_t* err;
};

struct EpiRsStore {
  using Params = RsParams;
  struct State {
    uint8_t* staging;
  };
  static constexpr int kCommWarps = 0;
  static constexpr int kSegCols = 128;                      // columns staged at a time
  static constexpr int kStagingBytes = kBM * kSegCols * 2;  // 32 KB next to the 4-stage ring

  __device__ static void begin_item(State&, const Params&, const GemmProblem&, const WorkItem&, int) {}
  __device__ static void end_item(State&, const Params&, const GemmProblem&, const WorkItem&, int) {}
  __device__ static void start(const Params&, const GemmProblem&) {}

  // The partial tile goes to the rank that owns its rows.  Accumulator rows live one per thread, so writing them
  // out directly would send 16-byte pieces of 128 different rows over NVLink per instruction; instead the tile is
  // converted to bf16 into a swizzled shared-memory buffer, 128 columns at a time, and every warp then stores whole
  // 256-byte row segments (two rows per instruction), which reach the link as full lines.
  template <int BN>
  __device__ static void tile(State& st, const Params& ep, const GemmProblem& p, uint32_t acc, int row, int n0) {
    const int warp = (threadIdx.x >> 5) - 2, lane = threadIdx.x & 31;
    const int r = ((threadIdx.x >> 5) & 3) * 32 + lane;  // accumulator row of this thread
    const int m0 = row - r;
    const int owner = m0 / ep.rows_local;
    __nv_bfloat16* dbase = static_cast<__nv_bfloat16*>(ep.partial.p[owner]) +
                           (static_cast<long long>(ep.rank) * ep.rows_local + (m0 - owner * ep.rows_local)) * p.N;
#pragma unroll 1
    for (int seg = 0; seg < BN; seg += kSegCols) {
      epi_bar_sync();  // the previous segment has been copied out of the staging buffer
#pragma unroll 1
      for (int c = 0; c < kSegCols; c += 32) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(acc + seg + c, t);
        tmem_ld_wait();
        uint8_t* srow = st.staging + r * (kSegCols * 2);  // 256 bytes per row, 16 chunks of 16 bytes
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(t[v * 8 + 2 * j]), __uint_as_float(t[v * 8 + 2 * j + 1]));
            w[j] = *reinterpret_cast<uint32_t*>(&b);
          }
          const int chunk = (c >> 3) + v;
          *reinterpret_cast<uint4*>(srow + ((chunk ^ (r & 15)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      epi_bar_sync();
      // warp w copies rows w*32 .. w*32+31, two rows per instruction (16 lanes x 16 bytes each)
      const int sub = lane >> 4, chunk = lane & 15;
      const int col = n0 + seg + chunk * 8;
#pragma unroll 4
      for (int i = 0; i < 32; i += 2) {
        const int rr = warp * 32 + i + sub;
        const uint4 q = *reinterpret_cast<const uint4*>(st.staging + rr * (kSegCols * 2) + ((chunk ^ (rr & 15)) << 4));
        __nv_bfloat16* dst = dbase + static_cast<long long>(rr) * p.N + col;
        if (col + 8 <= p.N) {
          *reinterpret_cast<uint4*>(dst) = q;
        } else {
          const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&q);
          for (int e = 0; e < 8 && col + e < p.N; ++e) dst[e] = h[e];
        }
      }
    }
    __threadfence_system();
    epi_bar_sync();
    if (threadIdx.x == 64) {
      const int tiles_local = ep.rows_local / kBM;
      const int lt = m0 / kBM - owner * tiles_local;
      unsigned int* ctr = static_cast<unsigned int*>(ep.counters.p[owner]) + lt * p.tiles_n + n0 / BN;
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(ctr), "r"(1u) : "memory");
    }
  }

  // Reduce phase: tiles owned by this rank, striped over the CTAs; warp w sums rows w, w+4, ...
  __device__ static void finish(const Params& ep, const GemmProblem& p, uint32_t kernel_id) {
    const int tid = threadIdx.x - 64;
    const int warp = tid >> 5, lane = tid & 31;
    const int tiles_local = ep.rows_local / kBM;
    const int units = tiles_local * p.tiles_n;
    const unsigned int* counters = static_cast<const unsigned int*>(ep.counters.p[ep.rank]);
    const __nv_bfloat16* mine = static_cast<const __nv_bfloat16*>(ep.partial.p[ep.rank]);
    const long long slab = static_cast<long long>(ep.rows_local) * p.N;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      unsigned int seen = 0;
      uint64_t deadline = 0;
      bool ok = true;
      for (;;) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(counters + u) : "memory");
        if (static_cast<int>(seen - ep.target) >= 0) break;
        const uint64_t now = global_timer_ns();
        if (deadline == 0) deadline = now + ep.wait_ns;
        if (now > deadline) {
          ok = false;
          break;
        }
        __nanosleep(200);
      }
      if (!ok) {
        report_error(ep.err, kErrPeerTimeout, kernel_id, 21);
        continue;
      }
      const int lt = u / p.tiles_n;
      const int n0 = (u - lt * p.tiles_n) * kBN;
      for (int cc = 0; cc < kBN; cc += 256) {
        const int col = n0 + cc + lane * 8;
        if (col >= p.N) continue;
        for (int r = warp; r < kBM; r += 4) {
          const long long off = static_cast<long long>(lt * kBM + r) * p.N + col;
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
          if (col + 8 <= p.N) {
            for (int s = 0; s < ep.world; ++s) {
              const uint4 q = *reinterpret_cast<const uint4*>(mine + s * slab + off);
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                acc[2 * j] += f.x;
                acc[2 * j + 1] += f.y;
              }
            }
            uint4 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
            *reinterpret_cast<uint4*>(ep.out + static_cast<long long>(lt * kBM + r) * ep.ldo + col) = o;
          } else {
            for (int j = 0; j < 8 && col + j < p.N; ++j) {
              float a = 0.f;
              for (int s = 0; s < ep.world; ++s) a += __bfloat162float(mine[s * slab + off + j]);
              ep.out[static_cast<long long>(lt * kBM + r) * ep.ldo + col + j] = __float2bfloat16_rn(a);
            }
          }
        }
      }
    }
  }
};

PeerPtrs to_peers(void* const* p, int world) {
  PeerPtrs out;
  for (int r = 0; r < 8; ++r) out.p[r] = r < world ? p[r] : nullptr;
  return out;
}

template <bool B_MN, class Epi>
void launch(const void* a_base, int M, int K, long long lda, const void* b_base, int N, long long ldb, GemmProblem p,
            const typename Epi::Params& ep, int sm_count, uint32_t* err, uint32_t kernel_id, cudaStream_t stream) {
  const CUtensorMap ta = make_tmap_2d_bf16(a_base, M, K, lda, kBM, kBK);
  const CUtensorMap tb = B_MN ? make_tmap_2d_bf16(b_base, K, N, ldb, kBK, 64) : make_tmap_2d_bf16(b_base, N, K, ldb, kBN, kBK);
  auto kernel = gemm_sm100_kernel<kBN, false, B_MN, kStages, Epi>;
  using L = GemmSmem<kBN, kStages, Epi::kStagingBytes>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes);
  }
  const int grid = p.num_items < sm_count ? p.num_items : sm_count;
  if (grid < 1) return;
  kernel<<<grid, gemm_threads<Epi>(), L::kDynamicBytes, stream>>>(ta, tb, p, ep, err, kernel_id);
}

}  // namespace

void tp_ag_gemm(const TpAgGemmArgs& a, cudaStream_t stream) {
  const int M = a.rows_local * a.world;
  const int tiles_local = a.rows_local / kBM;
  GemmProblem p = make_gemm_problem(M, a.N, a.K, kBN, 1, tiles_local < 8 ? tiles_local : 8);
  p.m_rot = a.rank * tiles_local;
  p.a_ready = static_cast<const unsigned int*>(a.ready[a.rank]);
  p.a_ready_target = a.epoch * static_cast<unsigned int>(a.chunks);
  p.a_wait_ns = a.wait_ns;
  AgParams ep;
  ep.store.tmap_c = make_tmap_2d_bf16(a.C, M, a.N, a.ldc, kBM, 64);
  ep.store.alpha = 1.f;
  ep.x_local = a.x_local;
  ep.ldx = a.ldx;
  ep.rows_local = a.rows_local;
  ep.k = a.K;
  ep.chunks = a.chunks;
  ep.rank = a.rank;
  ep.world = a.world;
  ep.gathered = to_peers(a.gathered, a.world);
  ep.ready = to_peers(a.ready, a.world);
  if (a.b_mn) {
    launch<true, EpiAgStore>(a.gathered[a.rank], M, a.K, a.K, a.B, a.N, a.ldb, p, ep, a.sm_count, a.err, 400u, stream);
  } else {
    launch<false, EpiAgStore>(a.gathered[a.rank], M, a.K, a.K, a.B, a.N, a.ldb, p, ep, a.sm_count, a.err, 400u, stream);
  }
}

void tp_gemm_rs(const TpGemmRsArgs& a, cudaStream_t stream) {
  const int M = a.rows_local * a.world;
  const int tiles_local = a.rows_local / kBM;
  GemmProblem p = make_gemm_problem(M, a.N, a.K, kBN, 1, tiles_local < 8 ? tiles_local : 8);
  p.m_rot = ((a.rank + 1) % a.world) * tiles_local;  // produce for the next rank first, own rows last
  RsParams ep;
  ep.partial = to_peers(a.partial, a.world);
  ep.counters = to_peers(a.counters, a.world);
  ep.out = a.out;
  ep.ldo = a.ldo;
  ep.rows_local = a.rows_local;
  ep.rank = a.rank;
  ep.world = a.world;
  ep.target = a.target;
  ep.wait_ns = a.wait_ns;
  ep.err = a.err;
  if (a.b_mn) {
    launch<true, EpiRsStore>(a.A, M, a.K, a.lda, a.B, a.N, a.ldb, p, ep, a.sm_count, a.err, 410u, stream);
  } else {
    launch<false, EpiRsStore>(a.A, M, a.K, a.lda, a.B, a.N, a.ldb, p, ep, a.sm_count, a.err, 410u, stream);
  }
}

}  // namespace rlk
