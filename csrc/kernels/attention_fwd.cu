// Flash attention forward for sm_100a with a shared-prefix + causal-suffix key range per sequence.
//
// Tokens are packed (no padding): q [Tq, Hq*128], k/v [Tkv, Hkv*128] bf16.  Each sequence s attends
//   (a) a "prefix" key range [pk_start, pk_start + pk_len) without a mask  (e.g. the prompt K/V that
//       all G completions of a GRPO group share -- stored once, read by every completion), and
//   (b) its "self" key range [sk_start, sk_start + sk_len), causally (key i visible to query i..)
//       or fully when causal == 0.
// Plain causal / non-causal attention and the reference's non-causal prefix-shared form
// (csrc/cuda/attention/prefix_shared_attention.cu:85-311: mma.sync m16n8k16 tiles, no causal part, no
// LSE, no tails, D == 128 only) are special cases.  The log-sum-exp of every row is returned so a
// backward pass or a cross-rank merge can follow.
//
// One CTA = one 128-query tile of one head.  Warp 0 loads Q once and K/V tiles through a 2-stage TMA
// ring; warp 1 issues S = Q K^T and O_j = P_j V_j on tcgen05 with S, O_j double-buffered in TMEM
// (4 x 128 columns).  Two groups of four warps own one query row per thread each:
//   softmax warps 2..5   : pull the whole S row into registers with four tcgen05.ld in flight (one wait), free
//                          the S buffer at once, online softmax, P as bf16 into a 128B-swizzled smem tile (the
//                          A operand of the second MMA), the row's rescale factor alpha into shared memory;
//   output warps 6..9    : O = O * alpha + O_j in registers, final normalisation, output and log-sum-exp.
// Splitting the two jobs keeps each thread under the register limit with all its TMEM loads in flight and
// puts two warps on every scheduler, so TMEM-load latency of one group hides behind the other's arithmetic.
#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "kernels.h"

namespace rlk {

namespace {

constexpr int kD = 128;        // head dim
constexpr int kTileQ = 128;
constexpr int kTileK = 128;
constexpr int kThreads = 320;
constexpr int kTileBytes = kTileQ * kD * 2;  // 32 KB: two 128B-swizzle atoms of [128 x 64]
constexpr int kAtomBytes = 128 * 64 * 2;     // 16 KB

struct Smem {
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;       // 2 stages
  static constexpr int kV = kK + 2 * kTileBytes;   // 2 stages
  static constexpr int kP = kV + 2 * kTileBytes;   // 2 buffers
  static constexpr int kAlpha = kP + 2 * kTileBytes;  // float [2][128] rescale factors
  static constexpr int kBars = kAlpha + 2 * 128 * 4;
  // q_full, kv_full[2], kv_empty[2], s_full[2], s_empty[2], p_full[2], o_full[2], o_empty[2], a_full[2], a_empty[2], fin
  static constexpr int kNumBars = 20;
  static constexpr int kBytes = kBars + kNumBars * 8 + 16;
  static constexpr int kDynamic = kBytes + 1024;
};
static_assert(Smem::kDynamic <= 232448, "attention forward exceeds the 227 KB shared-memory limit");

struct SeqDesc {  // one per sequence, int32 x 8
  int q_start, q_len, pk_start, pk_len, sk_start, sk_len, pad0, pad1;
};

__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const SeqDesc* __restrict__ seqs,
                const int2* __restrict__ tiles,  // (sequence, first query row within the sequence)
                int num_heads_q, int q_per_kv, int causal, float scale_log2e, __nv_bfloat16* __restrict__ out,
                long long ld_out, float* __restrict__ lse, long long lse_head_stride, uint32_t* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 3;
  uint64_t* s_full = bars + 5;
  uint64_t* s_empty = bars + 7;
  uint64_t* p_full = bars + 9;
  uint64_t* o_full = bars + 11;
  uint64_t* o_empty = bars + 13;
  uint64_t* a_full = bars + 15;
  uint64_t* a_empty = bars + 17;
  uint64_t* fin = bars + 19;
  float* alpha_s = reinterpret_cast<float*>(smem + Smem::kAlpha);
  // final (m2, l) per row: overlays the Q tile, which is dead once the last S = Q K^T has completed
  float2* final_s = reinterpret_cast<float2*>(smem + Smem::kQ);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Smem::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_id = blockIdx.x / num_heads_q;
  const int head = blockIdx.x - tile_id * num_heads_q;
  const int kv_head = head / q_per_kv;
  const int2 tile = tiles[tile_id];
  const SeqDesc sd = seqs[tile.x];
  const int q0 = tile.y;

  const int n_prefix = (sd.pk_len + kTileK - 1) / kTileK;
  int self_keys = sd.sk_len;
  if (causal) self_keys = min(self_keys, q0 + kTileQ);
  const int n_self = (self_keys + kTileK - 1) / kTileK;
  const int n_tiles = n_prefix + n_self;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&kv_full[b], 1);
      mbar_init(&kv_empty[b], 1);
      mbar_init(&s_full[b], 1);
      mbar_init(&s_empty[b], 128);
      mbar_init(&p_full[b], 128);
      mbar_init(&o_full[b], 1);
      mbar_init(&o_empty[b], 128);
      mbar_init(&a_full[b], 128);
      mbar_init(&a_empty[b], 128);
    }
    mbar_init(fin, 128);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, kTileBytes);
      tma_load_2d(smem + Smem::kQ, &tmap_q, q_full, head * kD, sd.q_start + q0);
      tma_load_2d(smem + Smem::kQ + kAtomBytes, &tmap_q, q_full, head * kD + 64, sd.q_start + q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        mbar_wait(&kv_empty[b], ph ^ 1, abort_flag, err, 200, 1);
        const int row = j < n_prefix ? sd.pk_start + j * kTileK : sd.sk_start + (j - n_prefix) * kTileK;
        mbar_arrive_expect_tx(&kv_full[b], 2 * kTileBytes);
        uint8_t* sk = smem + Smem::kK + b * kTileBytes;
        uint8_t* sv = smem + Smem::kV + b * kTileBytes;
        tma_load_2d(sk, &tmap_k, &kv_full[b], kv_head * kD, row);
        tma_load_2d(sk + kAtomBytes, &tmap_k, &kv_full[b], kv_head * kD + 64, row);
        tma_load_2d(sv, &tmap_v, &kv_full[b], kv_head * kD, row);
        tma_load_2d(sv + kAtomBytes, &tmap_v, &kv_full[b], kv_head * kD + 64, row);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, false, false);  // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, 128, false, true);   // P (K-major) x V (MN-major)
      const uint32_t sq = smem_u32(smem + Smem::kQ);
      mbar_wait(q_full, 0, abort_flag, err, 200, 2);
      auto issue_pv = [&](int j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        mbar_wait(&p_full[b], ph, abort_flag, err, 200, 3);
        mbar_wait(&o_empty[b], ph ^ 1, abort_flag, err, 200, 4);
        tc_fence_after();
        const uint32_t sp = smem_u32(smem + Smem::kP + b * kTileBytes);
        const uint32_t sv = smem_u32(smem + Smem::kV + b * kTileBytes);
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k) {
          // A = P: K-major, K = keys; 4 k-steps per 64-key atom.  B = V: MN-major, 16 key rows = 2048 bytes.
          const uint64_t da = umma_smem_desc_sw128(sp + (k >> 2) * kAtomBytes + (k & 3) * 32, 16, 1024);
          const uint64_t db = umma_smem_desc_sw128(sv + k * 2048, kAtomBytes, 1024);
          umma_bf16(tmem + 256 + b * 128, da, db, idesc_o, k != 0 ? 1u : 0u);
        }
        umma_commit(&o_full[b]);
        umma_commit(&kv_empty[b]);
      };
      for (int j = 0; j < n_tiles; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        mbar_wait(&kv_full[b], ph, abort_flag, err, 200, 5);
        mbar_wait(&s_empty[b], ph ^ 1, abort_flag, err, 200, 6);
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + Smem::kK + b * kTileBytes);
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const uint32_t off = (k >> 2) * kAtomBytes + (k & 3) * 32;
          umma_bf16(tmem + b * 128, umma_smem_desc_sw128(sq + off, 16, 1024), umma_smem_desc_sw128(sk + off, 16, 1024),
                    idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[b]);
        if (j >= 1) issue_pv(j - 1);
      }
      if (n_tiles >= 1) issue_pv(n_tiles - 1);
    }
  } else if (warp < 6) {
    // ------------------------------ softmax warps ------------------------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // query row within the tile
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int qi = q0 + r;           // query index within the sequence
    float m2 = -INFINITY, l = 0.f;
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const bool is_self = j >= n_prefix;
      const int key0 = is_self ? (j - n_prefix) * kTileK : j * kTileK;
      const int range_len = is_self ? sd.sk_len : sd.pk_len;
      int limit = range_len - key0;  // keys [0, limit) of this tile are in range
      if (is_self && causal) limit = min(limit, qi - key0 + 1);
      mbar_wait(&s_full[b], ph, abort_flag, err, 200, 8);
      tc_fence_after();
      // the whole S row: four loads in flight, one wait, then the TMEM buffer is free for S(j + 2)
      uint32_t t[kTileK];
      tmem_ld_32x32b_x32(tmem + b * 128 + 0 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&t[0]));
      tmem_ld_32x32b_x32(tmem + b * 128 + 32 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&t[32]));
      tmem_ld_32x32b_x32(tmem + b * 128 + 64 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&t[64]));
      tmem_ld_32x32b_x32(tmem + b * 128 + 96 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&t[96]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&s_empty[b]);
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < kTileK; ++i)
        if (i < limit) mx = fmaxf(mx, __uint_as_float(t[i]));
      const float new_m2 = fmaxf(m2, mx * scale_log2e);
      const float m_safe = new_m2 == -INFINITY ? 0.f : new_m2;
      const float alpha = fast_exp2(m2 - m_safe);  // m2 = -inf -> 0
      mbar_wait(&a_empty[b], ph ^ 1, abort_flag, err, 200, 9);
      alpha_s[b * 128 + r] = alpha;
      mbar_arrive(&a_full[b]);
      float sum = 0.f;
      uint8_t* prow = smem + Smem::kP + b * kTileBytes + r * 128;
      // p = 2^(s * scale - m), packed to bf16 into the swizzled P tile
#pragma unroll
      for (int c8 = 0; c8 < kTileK / 8; ++c8) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = c8 * 8 + 2 * i;
          const float p0 = col < limit ? fast_exp2(fmaf(__uint_as_float(t[col]), scale_log2e, -m_safe)) : 0.f;
          const float p1 = col + 1 < limit ? fast_exp2(fmaf(__uint_as_float(t[col + 1]), scale_log2e, -m_safe)) : 0.f;
          sum += p0 + p1;
          __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          w[i] = *reinterpret_cast<uint32_t*>(&pk);
        }
        // 128B swizzle: 16-byte chunk index XOR (row mod 8); one atom = 64 keys
        const int atom = c8 >> 3, chunk = c8 & 7;
        *reinterpret_cast<uint4*>(prow + atom * kAtomBytes + ((chunk ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l = fmaf(l, alpha, sum);
      m2 = new_m2;
      fence_proxy_async_smem();
      mbar_arrive(&p_full[b]);
    }
    if (n_tiles == 0) mbar_wait(q_full, 0, abort_flag, err, 200, 12);  // Q's TMA write must have landed before the overlay
    final_s[r] = make_float2(m2, l);
    mbar_arrive(fin);
  } else {
    // ------------------------------ output warps ------------------------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int qi = q0 + r;
    float o[kD];
#pragma unroll
    for (int i = 0; i < kD; ++i) o[i] = 0.f;
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      mbar_wait(&a_full[b], ph, abort_flag, err, 200, 10);
      const float alpha = alpha_s[b * 128 + r];
      mbar_arrive(&a_empty[b]);
      mbar_wait(&o_full[b], ph, abort_flag, err, 200, 7);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < kD; c += 64) {
        uint32_t t0[32], t1[32];
        tmem_ld_32x32b_x32(tmem + 256 + b * 128 + c + lane_addr, t0);
        tmem_ld_32x32b_x32(tmem + 256 + b * 128 + c + 32 + lane_addr, t1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] = fmaf(o[c + i], alpha, __uint_as_float(t0[i]));
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + 32 + i] = fmaf(o[c + 32 + i], alpha, __uint_as_float(t1[i]));
      }
      tc_fence_before();
      mbar_arrive(&o_empty[b]);
    }
    mbar_wait(fin, 0, abort_flag, err, 200, 11);
    const float2 ml = final_s[r];
    const float m2 = ml.x, l = ml.y;
    if (qi < sd.q_len) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = out + static_cast<long long>(sd.q_start + qi) * ld_out + head * kD;
#pragma unroll
      for (int c8 = 0; c8 < kD / 8; ++c8) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 pk = __floats2bfloat162_rn(o[c8 * 8 + 2 * i] * inv, o[c8 * 8 + 2 * i + 1] * inv);
          w[i] = *reinterpret_cast<uint32_t*>(&pk);
        }
        reinterpret_cast<uint4*>(dst)[c8] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (lse != nullptr) {
        lse[static_cast<long long>(head) * lse_head_stride + sd.q_start + qi] =
            l > 0.f ? (m2 + log2f(l)) * kLn2 : -INFINITY;
      }
    }
  }

  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace

void attention_forward(const AttnFwdArgs& a, cudaStream_t stream) {
  if (a.num_tiles <= 0) return;
  const CUtensorMap tq = make_tmap_2d_bf16(a.q, a.total_q, static_cast<uint64_t>(a.heads_q) * kD, a.ld_q, kTileQ, 64);
  const CUtensorMap tk = make_tmap_2d_bf16(a.k, a.total_kv, static_cast<uint64_t>(a.heads_kv) * kD, a.ld_k, kTileK, 64);
  const CUtensorMap tv = make_tmap_2d_bf16(a.v, a.total_kv, static_cast<uint64_t>(a.heads_kv) * kD, a.ld_v, kTileK, 64);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kDynamic);
    configured = true;
  }
  const long long grid = static_cast<long long>(a.num_tiles) * a.heads_q;
  attn_fwd_kernel<<<static_cast<unsigned int>(grid), kThreads, Smem::kDynamic, stream>>>(
      tq, tk, tv, reinterpret_cast<const SeqDesc*>(a.seqs), reinterpret_cast<const int2*>(a.tiles), a.heads_q,
      a.heads_q / a.heads_kv, a.causal ? 1 : 0, a.softmax_scale * kLog2e, a.out, a.ld_out, a.lse, a.lse_head_stride,
      a.err);
}

}  // namespace rlk
