// Fused linear -> selected-token log-prob (+ entropy) for sm_100a.
//
// Forward: one persistent kernel computes z = hidden * W_local^T tile by tile with tcgen05 (the
// [N, V] logits only ever exist as 128 x 256 fp32 tiles in tensor memory), folds every tile into a
// per-row online (max, sum-exp, sum-exp*z, target-logit) record, pushes the record of each finished
// (row-tile, vocab-split) item into EVERY tensor-parallel peer's partial buffer with plain peer
// stores over NVLink, and, once a row tile has all world x splits records, merges them in fixed
// (rank, split) order.  No NCCL call, no separate combine kernel, bitwise identical on all ranks.
//
// Backward (recompute): per token chunk, a second persistent kernel recomputes the logits tile and
// writes dz = g * (onehot - exp(z - lse)) as bf16 into a chunk workspace; the two products
// dz * W and dz^T * X then run on the shared GEMM mainloop with MN-major operands.
//
// What the reference does instead: csrc/cuda/fused_linear_logp_sm90.cu:55-280 (mma.sync tiles
// spilled to shared memory, row-serial softmax, separate combine kernel) and, for tensor
// parallelism, three NCCL all-reduces (rl_engine/kernels/ops/cuda/loss/linear_logp.py:151-161).
#include "../common/gemm_sm100.cuh"
#include "../common/tensormap.h"
#include "kernels.h"

namespace rlk {

constexpr int kLogpBN = 256;
constexpr int kLogpStages = 4;
constexpr int kMaxWorld = 8;

struct LogpFwdParams {
  const long long* target;  // [N] global vocab ids
  const float* bias;        // [V_local] or null
  long long vocab_start;    // global id of local column 0
  long long global_vocab;   // > 0: a target id outside [0, global_vocab) is reported in the error word
  int rank, world;
  int slot_base;            // first record slot of this rank (sum of the lower ranks' items_per_m)
  int total_records;        // records per row over all ranks
  int n_pad;                // row pitch of the partial buffers (>= tiles_m * 128)
  float4* peer_partials[kMaxWorld];   // each: [world * items_per_m, n_pad] records (m2, s, t, zt)
  unsigned int* peer_counters[kMaxWorld];  // each: [tiles_m] arrival counters of the current set
  unsigned int* next_counters;        // local counters of the other set, zeroed by this launch
  int counter_capacity;
  float* logp;     // [N]
  float* lse;      // [N] or null
  float* entropy;  // [N] or null
  uint32_t* err;
  unsigned long long wait_limit_ns;
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct EpiLogpStats {
  using Params = LogpFwdParams;
  static constexpr int kCommWarps = 0;
  static constexpr int kStagingBytes = 0;
  struct State {
    float m2, s, t, zt;
    int tgt;  // local target column or -1
  };

  __device__ static void begin_item(State& st, const Params& ep, const GemmProblem& p, const WorkItem&, int row) {
    st.m2 = -INFINITY;
    st.s = 0.f;
    st.t = 0.f;
    st.zt = 0.f;
    st.tgt = -1;
    if (row < p.M) {
      const long long local = ep.target[row] - ep.vocab_start;
      if (local >= 0 && local < p.N) st.tgt = static_cast<int>(local);
    }
  }

  template <int BN>
  __device__ static void tile(State& st, const Params& ep, const GemmProblem& p, uint32_t acc, int /*row*/, int n0) {
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(acc + c, r);
      tmem_ld_wait();
      const int col0 = n0 + c;
      if (col0 >= p.N) continue;
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      if (ep.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) v[j] += __ldg(ep.bias + col0 + j);
      }
      if (col0 + 32 > p.N) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j >= p.N) v[j] = -INFINITY;
      }
      float cmax = v[0];
#pragma unroll
      for (int j = 1; j < 32; ++j) cmax = fmaxf(cmax, v[j]);
      const float new_m2 = fmaxf(st.m2, cmax * kLog2e);
      const float rescale = fast_exp2(st.m2 - new_m2);  // 0 on the first chunk (m2 = -inf)
      float sum = 0.f, tsum = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float e = fast_exp2(fmaf(v[j], kLog2e, -new_m2));
        sum += e;
        tsum = fmaf(e, (col0 + j < p.N) ? v[j] : 0.f, tsum);
      }
      st.s = fmaf(st.s, rescale, sum);
      st.t = fmaf(st.t, rescale, tsum);
      st.m2 = new_m2;
      const int tl = st.tgt - col0;
      if (tl >= 0 && tl < 32) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j == tl) st.zt = v[j];
      }
    }
  }

  __device__ static void end_item(State& st, const Params& ep, const GemmProblem& p, const WorkItem& w, int row) {
    const float4 rec = make_float4(st.m2, st.s, st.t, st.zt);
    const size_t slot = static_cast<size_t>(ep.slot_base + w.split) * ep.n_pad + row;
    for (int r = 0; r < ep.world; ++r) ep.peer_partials[r][slot] = rec;
    __threadfence_system();
    epi_bar_sync();
    if (threadIdx.x == 64) {  // one epilogue thread publishes the arrival
      for (int r = 0; r < ep.world; ++r) {
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(ep.peer_counters[r] + w.m_tile), "r"(1u)
                     : "memory");
      }
    }
  }
};

// The merge phase is attached to the shared mainloop through the epilogue functor's `finish` hook.
// Merge phase, run by the 128 epilogue threads of each CTA after its GEMM items.
__device__ void logp_merge_phase(const LogpFwdParams& ep, const GemmProblem& p, uint32_t kernel_id) {
  const int tid = threadIdx.x - 64;  // 0..127
  const unsigned int expect = static_cast<unsigned int>(ep.total_records);
  const unsigned int* counters = ep.peer_counters[ep.rank];
  const float4* parts = ep.peer_partials[ep.rank];
  for (int t = blockIdx.x; t < p.tiles_m; t += gridDim.x) {
    // bounded wait for all records of row tile t
    unsigned int seen = 0;
    uint64_t deadline = 0;
    bool ok = true;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(counters + t) : "memory");
      if (seen >= expect) break;
      const uint64_t now = global_timer_ns();
      if (deadline == 0) deadline = now + ep.wait_limit_ns;
      if (now > deadline) {
        ok = false;
        break;
      }
      __nanosleep(200);
    }
    if (!ok) {
      report_error(ep.err, kErrPeerTimeout, kernel_id, 10);
      continue;
    }
    const int row = t * kBM + tid;
    if (row >= p.M) continue;
    const int records = ep.total_records;
    float M2 = -INFINITY;
    for (int i = 0; i < records; ++i) M2 = fmaxf(M2, parts[static_cast<size_t>(i) * ep.n_pad + row].x);
    float S = 0.f, T = 0.f, ZT = 0.f;
    for (int i = 0; i < records; ++i) {
      const float4 rec = parts[static_cast<size_t>(i) * ep.n_pad + row];
      const float w = fast_exp2(rec.x - M2);
      S = fmaf(rec.y, w, S);
      T = fmaf(rec.z, w, T);
      ZT += rec.w;
    }
    const float lse = (M2 + log2f(S)) * kLn2;
    if (ep.global_vocab > 0) {
      // The range check of the target ids happens here, on the device, instead of a host read-back per call: the
      // row's log-prob becomes NaN and the error word tells the host at its next check.
      const long long id = ep.target[row];
      if (id < 0 || id >= ep.global_vocab) {
        report_error(ep.err, kErrBadArgument, kernel_id, 11);
        ZT = __int_as_float(0x7fc00000);
      }
    }
    ep.logp[row] = ZT - lse;
    if (ep.lse != nullptr) ep.lse[row] = lse;
    if (ep.entropy != nullptr) ep.entropy[row] = lse - T / S;
  }
}

struct EpiLogpStatsWithMerge : EpiLogpStats {
  // Zero the counter set of the NEXT launch before this CTA publishes its first arrival.  A peer can
  // only begin its next launch after it has seen every arrival of this one, so the zeroing is ordered
  // before any arrival that will ever be counted in that set (every CTA of the grid owns >= 1 item).
  __device__ static void start(const Params& ep, const GemmProblem&) {
    const int tid = threadIdx.x - 64;
    for (int t = blockIdx.x * 128 + tid; t < ep.counter_capacity; t += gridDim.x * 128) ep.next_counters[t] = 0u;
    __threadfence();
    epi_bar_sync();
  }
  __device__ static void finish(const Params& ep, const GemmProblem& p, uint32_t kernel_id) {
    logp_merge_phase(ep, p, kernel_id);
  }
};

// ---------------------------------------------------------------------------------------------
// Backward epilogue: dz = g * (onehot - exp(z - lse)) written as bf16.
// ---------------------------------------------------------------------------------------------
struct LogpDzParams {
  const long long* target;
  const float* bias;
  const float* lse;    // [N] global log-sum-exp
  const float* grad;   // [N] dL/dlogp
  long long vocab_start;
  __nv_bfloat16* dz;   // [M, ld]
  long long ld;
};

struct EpiLogpDz {
  static constexpr int kCommWarps = 0;
  static constexpr int kStagingBytes = 0;
  using Params = LogpDzParams;
  struct State {
    float g, lse2;
    int tgt;
  };
  __device__ static void begin_item(State& st, const Params& ep, const GemmProblem& p, const WorkItem&, int row) {
    st.g = 0.f;
    st.lse2 = 0.f;
    st.tgt = -1;
    if (row < p.M) {
      st.g = ep.grad[row];
      st.lse2 = ep.lse[row] * kLog2e;
      const long long local = ep.target[row] - ep.vocab_start;
      if (local >= 0 && local < p.N) st.tgt = static_cast<int>(local);
    }
  }
  template <int BN>
  __device__ static void tile(State& st, const Params& ep, const GemmProblem& p, uint32_t acc, int row, int n0) {
    __nv_bfloat16* out = ep.dz + static_cast<long long>(row) * ep.ld;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(acc + c, r);
      tmem_ld_wait();
      const int col0 = n0 + c;
      if (row >= p.M || col0 >= p.N) continue;
      float d[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float z = __uint_as_float(r[j]);
        if (ep.bias != nullptr && col0 + j < p.N) z += __ldg(ep.bias + col0 + j);
        const float prob = fast_exp2(fmaf(z, kLog2e, -st.lse2));
        d[j] = -st.g * prob;
      }
      const int tl = st.tgt - col0;
      if (tl >= 0 && tl < 32) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j == tl) d[j] += st.g;
      }
      if (col0 + 32 <= p.N) {
        uint4* dst = reinterpret_cast<uint4*>(out + col0);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 b = __floats2bfloat162_rn(d[v * 8 + 2 * j], d[v * 8 + 2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t*>(&b);
          }
          dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
        for (int j = 0; j < 32 && col0 + j < p.N; ++j) out[col0 + j] = __float2bfloat16_rn(d[j]);
      }
    }
  }
  __device__ static void end_item(State&, const Params&, const GemmProblem&, const WorkItem&, int) {}
  __device__ static void finish(const Params&, const GemmProblem&, uint32_t) {}
  __device__ static void start(const Params&, const GemmProblem&) {}
};

// ---------------------------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------------------------
template <class Kernel>
static void set_smem(Kernel k, int bytes) {
  static PerDeviceOnce done;  // one static per instantiation
  if (done.first()) {
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  }
}

int linear_logp_vocab_tiles_per_split() { return 32; }  // 32 * 256 = 8192 vocab columns per split

void linear_logp_workspace_shape(int n_tokens, int v_local, int world, int* items_per_m, int* n_pad, int* tiles_m) {
  const GemmProblem p = make_gemm_problem(n_tokens, v_local, 64, kLogpBN, linear_logp_vocab_tiles_per_split(), 1);
  *items_per_m = p.items_per_m;
  *tiles_m = p.tiles_m;
  *n_pad = p.tiles_m * kBM;
  (void)world;
}

void linear_logp_forward(const LinearLogpFwdArgs& a, cudaStream_t stream) {
  const int splits_tiles = linear_logp_vocab_tiles_per_split();
  int items_per_m_probe = (((a.v_local + kLogpBN - 1) / kLogpBN) + splits_tiles - 1) / splits_tiles;
  int group_m = a.sm_count / (items_per_m_probe > 0 ? items_per_m_probe : 1);
  if (group_m < 1) group_m = 1;
  // keep as many token tiles per group as stay L2-resident, so the weight streams from DRAM once per group
  group_m = raster_group_m((a.n_tokens + kBM - 1) / kBM, a.hidden_dim, group_m, 64ll << 20);
  const GemmProblem p = make_gemm_problem(a.n_tokens, a.v_local, a.hidden_dim, kLogpBN, splits_tiles, group_m);
  const CUtensorMap ta = make_tmap_2d_bf16(a.hidden, a.n_tokens, a.hidden_dim, a.ld_hidden, kBM, kBK);
  const CUtensorMap tb = make_tmap_2d_bf16(a.weight, a.v_local, a.hidden_dim, a.ld_weight, kLogpBN, kBK);
  LogpFwdParams ep;
  ep.target = a.target;
  ep.bias = a.bias;
  ep.vocab_start = a.vocab_start;
  ep.global_vocab = a.global_vocab;
  ep.rank = a.rank;
  ep.world = a.world;
  ep.slot_base = a.slot_base;
  ep.total_records = a.total_records > 0 ? a.total_records : p.items_per_m * a.world;
  ep.n_pad = p.tiles_m * kBM;
  for (int r = 0; r < kMaxWorld; ++r) {
    ep.peer_partials[r] = r < a.world ? reinterpret_cast<float4*>(a.peer_partials[r]) : nullptr;
    ep.peer_counters[r] = r < a.world ? a.peer_counters[r] : nullptr;
  }
  ep.next_counters = a.next_counters;
  ep.counter_capacity = a.counter_capacity;
  ep.logp = a.logp;
  ep.lse = a.lse;
  ep.entropy = a.entropy;
  ep.err = a.err;
  ep.wait_limit_ns = a.wait_limit_ns ? a.wait_limit_ns : kWaitLimitNs;
  auto kernel = gemm_sm100_kernel<kLogpBN, false, false, kLogpStages, EpiLogpStatsWithMerge>;
  using L = GemmSmem<kLogpBN, kLogpStages>;
  set_smem(kernel, L::kDynamicBytes);
  int grid = p.num_items < a.sm_count ? p.num_items : a.sm_count;
  if (grid < 1) grid = 1;
  kernel<<<grid, kGemmThreads, L::kDynamicBytes, stream>>>(ta, tb, p, ep, a.err, 101u);
}

void linear_logp_dz(const LinearLogpDzArgs& a, cudaStream_t stream) {
  const int tiles_n = (a.v_local + kLogpBN - 1) / kLogpBN;
  (void)tiles_n;
  const GemmProblem p = make_gemm_problem(a.n_tokens, a.v_local, a.hidden_dim, kLogpBN, 1,
                                          raster_group_m((a.n_tokens + kBM - 1) / kBM, a.hidden_dim, 16, 64ll << 20));
  const CUtensorMap ta = make_tmap_2d_bf16(a.hidden, a.n_tokens, a.hidden_dim, a.ld_hidden, kBM, kBK);
  const CUtensorMap tb = make_tmap_2d_bf16(a.weight, a.v_local, a.hidden_dim, a.ld_weight, kLogpBN, kBK);
  LogpDzParams ep;
  ep.target = a.target;
  ep.bias = a.bias;
  ep.lse = a.lse;
  ep.grad = a.grad;
  ep.vocab_start = a.vocab_start;
  ep.dz = a.dz;
  ep.ld = a.ld_dz;
  auto kernel = gemm_sm100_kernel<kLogpBN, false, false, kLogpStages, EpiLogpDz>;
  using L = GemmSmem<kLogpBN, kLogpStages>;
  set_smem(kernel, L::kDynamicBytes);
  int grid = p.num_items < a.sm_count ? p.num_items : a.sm_count;
  if (grid < 1) grid = 1;
  kernel<<<grid, kGemmThreads, L::kDynamicBytes, stream>>>(ta, tb, p, ep, a.err, 102u);
}

}  // namespace rlk
