// Flash attention backward for sm_100a (packed tokens, shared prefix + causal self range, GQA).
// Deterministic by construction: no atomics; every output element is produced by one CTA (or by a
// fixed-order reduction of per-split partials).
//
//   attn_delta      : delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]
//   attn_bwd_dq     : one CTA per (128-query tile, q head); loops over 64-key tiles:
//                       S = Q K^T, dP = dO V^T  (tcgen05, TMEM)   ->  P = exp2(S c - lse), dS = P (dP - delta)
//                       dQ += dS K            (K tile re-read from the same smem bytes as an MN-major operand)
//   attn_bwd_dkv    : one CTA per (128-key tile, kv head, split of its query-block list); for every
//                     q head of the GQA group and every 64-query block that can see the tile:
//                       S^T = K Q^T, dP^T = V dO^T  ->  P^T, dS^T (thread per key row)
//                       dV += P^T dO ,  dK += dS^T Q  (accumulated in TMEM across the whole loop)
//                     partial results of split items are summed in split order by attn_bwd_reduce.
//
// The reference has no attention backward of its own: its Triton tutorial kernel
// (rl_engine/kernels/ops/triton/triton_attn.py:185-330) accumulates dQ with tl.atomic_add
// (non-deterministic) and is not wired into its registry.
#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "kernels.h"

namespace rlk {

#ifdef RLK_ATTN_PROFILE
// Phase timing of one compute thread of the dQ kernel (debug builds only), cycles per phase summed over its tiles.
__device__ unsigned long long g_attn_bwd_prof[16];
#define BPROF_DECL unsigned long long prof_t = clock64(); const bool prof_on = (blockIdx.x == gridDim.x / 2) && threadIdx.x == 64
#define BPROF(slot)                                     \
  if (prof_on) {                                        \
    const unsigned long long now = clock64();           \
    atomicAdd(&g_attn_bwd_prof[slot], now - prof_t);    \
    prof_t = now;                                       \
  }
// The same for the MMA-issuing thread of the profiled CTA (slots 8..15): waits and issue sections.
#define MPROF_DECL unsigned long long mprof_t = clock64(); const bool mprof_on = (blockIdx.x == gridDim.x / 2)
#define MPROF(slot)                                          \
  if (mprof_on) {                                            \
    const unsigned long long now = clock64();                \
    atomicAdd(&g_attn_bwd_prof[8 + slot], now - mprof_t);    \
    mprof_t = now;                                           \
  }
void attention_bwd_profile_read(unsigned long long* out) {
  cudaMemcpyFromSymbol(out, g_attn_bwd_prof, sizeof(unsigned long long) * 16);
  unsigned long long z[16] = {0};
  cudaMemcpyToSymbol(g_attn_bwd_prof, z, sizeof(z));
}
#else
#define BPROF_DECL
#define BPROF(slot)
#define MPROF_DECL
#define MPROF(slot)
#endif

namespace {

constexpr int kD = 128;
constexpr int kThreads = 320;  // TMA warp, MMA warp, two compute groups of four warps (ping-pong over tiles)
constexpr int kAtom128 = 128 * 128;  // bytes of a [128 rows x 64 cols] bf16 swizzle atom
constexpr int kAtom64 = 64 * 128;    // bytes of a [64 rows x 64 cols] atom

struct SeqDesc {
  int q_start, q_len, pk_start, pk_len, sk_start, sk_len, pad0, pad1;
};

// ------------------------------------------------------------------------------------- delta
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                  long long ld, int heads, long long tokens, float* __restrict__ delta) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= tokens * heads) return;
  const long long t = warp / heads;
  const int h = static_cast<int>(warp - t * heads);
  const uint2 a = *reinterpret_cast<const uint2*>(out + t * ld + h * kD + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + t * ld + h * kD + lane * 4);
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
    s = fmaf(x.x, y.x, s);
    s = fmaf(x.y, y.y, s);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[static_cast<long long>(h) * tokens + t] = s;
}

// One query row against a 64-key tile: dS = P * (dP - delta) with P = 2^(S * scale - lse), packed to bf16 into the
// row's 128-byte swizzle line.  MASKED = false: the whole tile is visible to the row.
template <bool MASKED>
__device__ __forceinline__ void dq_row(const uint32_t (&ts)[64], const uint32_t (&tp)[64], int limit, float scale_log2e,
                                       float lse2, float dlt, uint8_t* dsrow, int r) {
#pragma unroll
  for (int c8 = 0; c8 < 8; ++c8) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int col = c8 * 8 + 2 * i;
      const float x0 = fmaf(__uint_as_float(ts[col]), scale_log2e, -lse2);
      const float x1 = fmaf(__uint_as_float(ts[col + 1]), scale_log2e, -lse2);
      float p0 = fast_exp2(x0);
      float p1 = (i & 1) ? poly_exp2(x1) : fast_exp2(x1);
      if (MASKED) {
        p0 = col < limit ? p0 : 0.f;
        p1 = col + 1 < limit ? p1 : 0.f;
      }
      __nv_bfloat162 pk = __floats2bfloat162_rn(p0 * (__uint_as_float(tp[col]) - dlt), p1 * (__uint_as_float(tp[col + 1]) - dlt));
      w[i] = *reinterpret_cast<uint32_t*>(&pk);
    }
    *reinterpret_cast<uint4*>(dsrow + ((c8 ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ---------------------------------------------------------------------------------------- dQ
struct DqSmem {
  static constexpr int kQ = 0;                       // [128 x 128] 32 KB
  static constexpr int kDO = 32768;                  // 32 KB
  static constexpr int kStages = 4;                    // barrier slots: K ring (3) + the V buffer (1)
  static constexpr int kKRing = 3;                     // K pair stages; a stage is held until the dQ products of its pair
  static constexpr int kPairBytes = 2 * kAtom128;      // [128 keys x 128 d] = two [128 x 64] atoms = 32 KB
  static constexpr int kKV = 65536;                    // K ring
  static constexpr int kV = kKV + kKRing * kPairBytes; // one V pair buffer
  static constexpr int kDS = kV + kPairBytes;          // 2 buffers of [128 x 64] bf16 = 16 KB each
  static constexpr int kBars = kDS + 2 * kAtom128;
  // qdo_full, kv_full[4], kv_empty[4], s_full[2], s_empty[2], ds_full[2], ds_empty[2], dq_done
  static constexpr int kNumBars = 18;
  static constexpr int kDynamic = kBars + kNumBars * 8 + 16 + 1024;
};
static_assert(DqSmem::kDynamic <= 232448 && DqSmem::kDynamic > 116 * 1024, "dQ kernel shared memory out of range");

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                   const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                   const SeqDesc* __restrict__ seqs, const int2* __restrict__ tiles, int num_heads_q, int q_per_kv,
                   int causal, float scale, const float* __restrict__ lse, const float* __restrict__ delta,
                   long long head_stride, __nv_bfloat16* __restrict__ dq, long long ld_dq, uint32_t* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DqSmem::kBars);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + DqSmem::kStages;
  uint64_t* k_full = kv_full;        // [kKRing]
  uint64_t* k_empty = kv_empty;      // [kKRing]
  uint64_t* v_full = kv_full + DqSmem::kKRing;
  uint64_t* v_empty = kv_empty + DqSmem::kKRing;
  uint64_t* s_full = kv_empty + DqSmem::kStages;
  uint64_t* s_empty = s_full + 2;
  uint64_t* ds_full = s_empty + 2;
  uint64_t* ds_empty = ds_full + 2;
  uint64_t* dq_done = ds_empty + 2;  // all dQ MMAs of this CTA have completed
  static_assert(1 + 2 * DqSmem::kStages + 9 == DqSmem::kNumBars, "dQ barrier layout");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + DqSmem::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_id = blockIdx.x / num_heads_q;
  const int head = blockIdx.x - tile_id * num_heads_q;
  const int kv_head = head / q_per_kv;
  const int2 tile = tiles[tile_id];
  const SeqDesc sd = seqs[tile.x];
  const int q0 = tile.y;
  constexpr int TK = 64;
  const int n_prefix = (sd.pk_len + TK - 1) / TK;
  int self_keys = sd.sk_len;
  if (causal) self_keys = min(self_keys, q0 + 128);
  const int n_self = (self_keys + TK - 1) / TK;
  const int n_tiles = n_prefix + n_self;
  const int n_pairs = (n_tiles + 1) / 2;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < DqSmem::kStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&s_empty[b], 4);  // one arrival per warp of the group that owns buffer b
      mbar_init(&ds_full[b], 4);
      mbar_init(&ds_empty[b], 1);
    }
    mbar_init(dq_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: S[b] at b*64 (b = 0,1), dP[b] at 128 + b*64, dQ at 256..383
  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(qdo_full, 65536);
      for (int c = 0; c < 2; ++c) {
        tma_load_2d(smem + DqSmem::kQ + c * kAtom128, &tmap_q, qdo_full, head * kD + c * 64, sd.q_start + q0);
        tma_load_2d(smem + DqSmem::kDO + c * kAtom128, &tmap_do, qdo_full, head * kD + c * 64, sd.q_start + q0);
      }
      // Key tiles travel in PAIRS (128 keys): S and dP of a pair are one N = 128 product each, at the tensor cores' full
      // rate and with half the instructions of two N = 64 products.  K has a ring of three pair stages (a stage is held
      // until the dQ products of its pair), V one pair buffer (free again as soon as dP of the pair has completed).
      // Inside a [128 keys x 64 d] swizzle atom the first tile of the pair is rows 0..63, the second rows 64..127; each
      // tile is loaded by its own TMA copies, so a pair may straddle the prefix / self boundary.
      auto key_row = [&](int j) { return j < n_prefix ? sd.pk_start + j * TK : sd.sk_start + (j - n_prefix) * TK; };
      int ks = 0;
      uint32_t kphase = 0;
      for (int p = 0; p < n_pairs; ++p) {
        const int halves = min(2, n_tiles - 2 * p);
        uint8_t* sk = smem + DqSmem::kKV + ks * DqSmem::kPairBytes;
        uint8_t* sv = smem + DqSmem::kV;
        mbar_wait(&k_empty[ks], kphase ^ 1, abort_flag, err, 210, 1);
        mbar_arrive_expect_tx(&k_full[ks], halves * 2 * kAtom64);
        for (int h = 0; h < halves; ++h)
          for (int c = 0; c < 2; ++c)
            tma_load_2d(sk + c * kAtom128 + h * kAtom64, &tmap_k, &k_full[ks], kv_head * kD + c * 64, key_row(2 * p + h));
        mbar_wait(v_empty, (p & 1) ^ 1, abort_flag, err, 210, 9);
        mbar_arrive_expect_tx(v_full, halves * 2 * kAtom64);
        for (int h = 0; h < halves; ++h)
          for (int c = 0; c < 2; ++c)
            tma_load_2d(sv + c * kAtom128 + h * kAtom64, &tmap_v, v_full, kv_head * kD + c * 64, key_row(2 * p + h));
        if (++ks == DqSmem::kKRing) {
          ks = 0;
          kphase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, false, false);  // [128 q] x [128 keys of a pair], K = d
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, 128, false, true);  // dS (K-major) x K tile (MN-major)
      const uint32_t sq = smem_u32(smem + DqSmem::kQ);
      const uint32_t sdo = smem_u32(smem + DqSmem::kDO);
      mbar_wait(qdo_full, 0, abort_flag, err, 210, 2);
      // This thread's instruction stream is the kernel's critical path, so every descriptor is built once: Q / dO / V
      // operands are fixed, K and dS operands are stage 0 / buffer 0 plus one add per use.
      const uint32_t sk0 = smem_u32(smem + DqSmem::kKV), sv0 = smem_u32(smem + DqSmem::kV);
      uint64_t desc_q[kD / 16], desc_do[kD / 16], desc_k0[kD / 16], desc_v[kD / 16];
#pragma unroll
      for (int k = 0; k < kD / 16; ++k) {
        const uint32_t off = (k >> 2) * kAtom128 + (k & 3) * 32;  // all four are [128 rows x 64 cols] atoms
        desc_q[k] = umma_smem_desc_sw128(sq + off, 16, 1024);
        desc_do[k] = umma_smem_desc_sw128(sdo + off, 16, 1024);
        desc_k0[k] = umma_smem_desc_sw128(sk0 + off, 16, 1024);
        desc_v[k] = umma_smem_desc_sw128(sv0 + off, 16, 1024);
      }
      // dQ operands: dS buffer 0 (K-major) and the first tile of K stage 0 read MN-major (its two d atoms are kAtom128 apart)
      uint64_t desc_ds0[TK / 16], desc_kt0[TK / 16];
#pragma unroll
      for (int k = 0; k < TK / 16; ++k) {
        desc_ds0[k] = umma_smem_desc_sw128(smem_u32(smem + DqSmem::kDS) + k * 32, 16, 1024);
        desc_kt0[k] = umma_smem_desc_sw128(sk0 + k * 2048, kAtom128, 1024);
      }
      MPROF_DECL;
      auto issue_dq_pair = [&](int p) {
        const int ks = p % DqSmem::kKRing;
        for (int h = 0; h < 2 && 2 * p + h < n_tiles; ++h) {
          const int j = 2 * p + h;
          MPROF(0);
          mbar_wait(&ds_full[h], p & 1, abort_flag, err, 210, 3);
          MPROF(3);
          tc_fence_after();
          const uint32_t ds_off = h * kAtom128, k_off = ks * DqSmem::kPairBytes + h * kAtom64;
#pragma unroll
          for (int k = 0; k < TK / 16; ++k) {
            umma_bf16(tmem + 256, umma_desc_advance(desc_ds0[k], ds_off), umma_desc_advance(desc_kt0[k], k_off), idesc_dq,
                      (j | k) != 0 ? 1u : 0u);
          }
          umma_commit(&ds_empty[h]);
          MPROF(4);
        }
        umma_commit(&k_empty[ks]);
      };
      for (int p = 0; p < n_pairs; ++p) {
        const int ks = p % DqSmem::kKRing;
        MPROF(0);
        mbar_wait(&k_full[ks], (p / DqSmem::kKRing) & 1, abort_flag, err, 210, 4);
        MPROF(5);
        // both halves of the S / dP columns are rewritten, so both groups must have taken the previous pair's values
        mbar_wait(&s_empty[0], (p & 1) ^ 1, abort_flag, err, 210, 5);
        mbar_wait(&s_empty[1], (p & 1) ^ 1, abort_flag, err, 210, 5);
        MPROF(1);
        tc_fence_after();
        const uint32_t k_off = ks * DqSmem::kPairBytes;
#pragma unroll
        for (int k = 0; k < kD / 16; ++k)
          umma_bf16(tmem, desc_q[k], umma_desc_advance(desc_k0[k], k_off), idesc_s, k != 0 ? 1u : 0u);
        mbar_wait(v_full, p & 1, abort_flag, err, 210, 10);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) umma_bf16(tmem + 128, desc_do[k], desc_v[k], idesc_s, k != 0 ? 1u : 0u);
        umma_commit(&s_full[0]);
        if (2 * p + 1 < n_tiles) umma_commit(&s_full[1]);
        umma_commit(v_empty);
        MPROF(2);
        // dQ trails S / dP by one PAIR: a compute group releases its S / dP columns as soon as the values are in
        // registers, so S, dP of the next pair are issued before this thread blocks on the dS of the previous one.
        if (p >= 1) issue_dq_pair(p - 1);
      }
      if (n_pairs >= 1) issue_dq_pair(n_pairs - 1);
      // A barrier of its own for "dQ complete": the groups must not take this from ds_empty of the last tile, because
      // a group that does not own that buffer has not followed its phases and could see an older phase of the same
      // parity as complete.
      umma_commit(dq_done);
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int qi = q0 + r;
    const bool row_ok = qi < sd.q_len;
    const long long stat_idx = static_cast<long long>(head) * head_stride + sd.q_start + qi;
    const float lse2 = row_ok ? lse[stat_idx] * kLog2e : 0.f;
    const float dlt = row_ok ? delta[stat_idx] : 0.f;
    const float scale_log2e = scale * kLog2e;
    // Two groups of four warps: group g handles the tiles j = g, g + 2, ... (TMEM / smem buffer g), so that the
    // exponentials of one tile overlap the TMEM loads and the MMAs of the next.
    const int group = (warp - 2) >> 2;
    BPROF_DECL;
    for (int j = group; j < n_tiles; j += 2) {
      const int b = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const bool is_self = j >= n_prefix;
      const int key0 = is_self ? (j - n_prefix) * TK : j * TK;
      int limit = (is_self ? sd.sk_len : sd.pk_len) - key0;
      if (is_self && causal) limit = min(limit, qi - key0 + 1);
      if (!row_ok) limit = 0;
      BPROF(0);
      mbar_wait(&s_full[b], ph, abort_flag, err, 210, 6);
      BPROF(1);
      tc_fence_after();
      uint8_t* dsrow = smem + DqSmem::kDS + b * kAtom128 + r * 128;
      uint32_t ts[64], tp[64];
      tmem_ld_32x32b_x32(tmem + b * 64 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&ts[0]));
      tmem_ld_32x32b_x32(tmem + b * 64 + 32 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&ts[32]));
      tmem_ld_32x32b_x32(tmem + 128 + b * 64 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&tp[0]));
      tmem_ld_32x32b_x32(tmem + 128 + b * 64 + 32 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&tp[32]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(&s_empty[b]);  // S / dP are in registers: the TMEM buffers are free for tile j + 2
      BPROF(2);
      mbar_wait(&ds_empty[b], ph ^ 1, abort_flag, err, 210, 7);  // dS buffer b free (dQ MMA of tile j-2 done)
      BPROF(3);
      if (__any_sync(0xffffffffu, limit < TK)) {
        dq_row<true>(ts, tp, limit, scale_log2e, lse2, dlt, dsrow, r);
      } else {
        dq_row<false>(ts, tp, limit, scale_log2e, lse2, dlt, dsrow, r);
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(&ds_full[b]);
      BPROF(4);
    }
    // wait for the last dQ MMA, then write dQ * scale
    if (n_tiles >= 1) {
      mbar_wait(dq_done, 0, abort_flag, err, 210, 8);
      tc_fence_after();
    }
    __nv_bfloat16* dst = dq + static_cast<long long>(sd.q_start + qi) * ld_dq + head * kD;
    // each group writes its half of the dQ columns
#pragma unroll
    for (int c = group * 64; c < group * 64 + 64; c += 32) {
      uint32_t t[32];
      if (n_tiles >= 1) {
        tmem_ld_32x32b_x32(tmem + 256 + c + lane_addr, t);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) t[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(t[v * 8 + 2 * i]) * scale,
                                                      __uint_as_float(t[v * 8 + 2 * i + 1]) * scale);
            w[i] = *reinterpret_cast<uint32_t*>(&pk);
          }
          reinterpret_cast<uint4*>(dst + c)[v] = make_uint4(w[0], w[1], w[2], w[3]);
        }
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

// ------------------------------------------------------------------------------------- dK, dV
struct KvItem {  // one work item: a 128-key tile of one key range and a slice of its query-block list
  int k_row;     // first key row in the packed K/V arrays
  int k_len;     // valid keys (<= 128)
  int k_pos;     // index of the first key inside its range (for the causal test)
  int qb_begin;  // [qb_begin, qb_end) into the query-block list
  int qb_end;
  int out_slot;  // >= 0: partial slot in the fp32 workspace; -1: write bf16 dK/dV directly
  int pad0, pad1;
};
struct QBlock {  // up to 64 consecutive queries of one sequence
  int q_row;     // first query row in the packed arrays
  int n_rows;
  int q_pos;     // index of the first query inside its sequence
  int causal;    // 1: key visible iff k_pos + r <= q_pos + c
};

struct DkvSmem {
  static constexpr int kK = 0;        // [128 keys x 128 d] 32 KB
  static constexpr int kV = 32768;    // 32 KB
  static constexpr int kStages = 3;  // a stage is held until the dV / dK MMAs of its block: depth hides the TMA latency
  static constexpr int kStageBytes = 2 * 2 * kAtom64;  // Q block + dO block, each [64 q x 128 d] = 16 KB
  static constexpr int kQdO = 65536;
  static constexpr int kPT = kQdO + kStages * kStageBytes;  // P^T: 2 buffers of [128 keys x 64 q] = 16 KB
  static constexpr int kDST = kPT + 2 * kAtom128;           // dS^T: 2 buffers
  static constexpr int kStat = kDST + 2 * kAtom128;         // float [2 groups][64 lse * log2e | 64 delta]
  static constexpr int kBars = kStat + 2 * 128 * 4;
  // kv_full, q_full[3], q_empty[3], s_full[2], s_empty[2], p_full[2], p_empty[2], acc_full
  static constexpr int kNumBars = 16;
  static constexpr int kDynamic = kBars + kNumBars * 8 + 16 + 1024;
};
static_assert(DkvSmem::kDynamic <= 232448 && DkvSmem::kDynamic > 116 * 1024, "dK/dV kernel shared memory out of range");

// One key row against a 64-query block: P^T = 2^(S^T * scale - lse) and dS^T = P^T * (dP^T - delta), both packed to
// bf16 into the row's 128-byte swizzle lines.  `stat` holds lse * log2(e) for the 64 queries followed by their delta.
// MASKED = false: every query of the block is visible to the row.  One exponential in four runs on the FMA pipe.
template <bool MASKED>
__device__ __forceinline__ void dkv_row(const uint32_t (&ts)[64], const uint32_t (&tp)[64], const float* stat, int c_lo,
                                        int c_hi, float scale_log2e, uint8_t* prow, uint8_t* dsrow, int r) {
#pragma unroll
  for (int c8 = 0; c8 < 8; ++c8) {
    uint32_t wp[4], wd[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int col = c8 * 8 + 2 * i;
      const float2 l2 = *reinterpret_cast<const float2*>(stat + col);
      const float2 dl = *reinterpret_cast<const float2*>(stat + 64 + col);
      const float x0 = fmaf(__uint_as_float(ts[col]), scale_log2e, -l2.x);
      const float x1 = fmaf(__uint_as_float(ts[col + 1]), scale_log2e, -l2.y);
      float p0 = fast_exp2(x0);
      float p1 = (i & 1) ? poly_exp2(x1) : fast_exp2(x1);
      if (MASKED) {
        p0 = (col >= c_lo && col < c_hi) ? p0 : 0.f;
        p1 = (col + 1 >= c_lo && col + 1 < c_hi) ? p1 : 0.f;
      }
      const float d0 = p0 * (__uint_as_float(tp[col]) - dl.x);
      const float d1 = p1 * (__uint_as_float(tp[col + 1]) - dl.y);
      __nv_bfloat162 a = __floats2bfloat162_rn(p0, p1);
      __nv_bfloat162 d = __floats2bfloat162_rn(d0, d1);
      wp[i] = *reinterpret_cast<uint32_t*>(&a);
      wd[i] = *reinterpret_cast<uint32_t*>(&d);
    }
    const int sw = (c8 ^ (r & 7)) << 4;
    *reinterpret_cast<uint4*>(prow + sw) = make_uint4(wp[0], wp[1], wp[2], wp[3]);
    *reinterpret_cast<uint4*>(dsrow + sw) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
  }
}

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                    const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                    const KvItem* __restrict__ items, const QBlock* __restrict__ qblocks, int num_heads_kv,
                    int q_per_kv, float scale, const float* __restrict__ lse, const float* __restrict__ delta,
                    long long head_stride, __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                    long long ld_dkv, float* __restrict__ partials, uint32_t* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DkvSmem::kBars);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;
  uint64_t* q_empty = q_full + DkvSmem::kStages;
  uint64_t* s_full = q_empty + DkvSmem::kStages;
  uint64_t* s_empty = s_full + 2;
  uint64_t* p_full = s_empty + 2;
  uint64_t* p_empty = p_full + 2;
  uint64_t* acc_full = p_empty + 2;
  static_assert(1 + 2 * DkvSmem::kStages + 8 + 1 == DkvSmem::kNumBars, "dK/dV barrier layout");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + DkvSmem::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item_id = blockIdx.x / num_heads_kv;
  const int kv_head = blockIdx.x - item_id * num_heads_kv;
  const KvItem it = items[item_id];
  const int n_qb = it.qb_end - it.qb_begin;
  const int n_iter = n_qb * q_per_kv;  // iteration t -> (q head = t / n_qb, block = t % n_qb)

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(acc_full, 1);
    for (int s = 0; s < DkvSmem::kStages; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&s_empty[b], 4);  // one arrival per warp of the group that owns buffer b
      mbar_init(&p_full[b], 4);
      mbar_init(&p_empty[b], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: S^T[b] at b*64, dP^T[b] at 128 + b*64, dV at 256, dK at 384

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 65536);
      for (int c = 0; c < 2; ++c) {
        tma_load_2d(smem + DkvSmem::kK + c * kAtom128, &tmap_k, kv_full, kv_head * kD + c * 64, it.k_row);
        tma_load_2d(smem + DkvSmem::kV + c * kAtom128, &tmap_v, kv_full, kv_head * kD + c * 64, it.k_row);
      }
      for (int t = 0; t < n_iter; ++t) {
        const int st = t % DkvSmem::kStages;
        const uint32_t ph = (t / DkvSmem::kStages) & 1;
        const int hq = kv_head * q_per_kv + t / n_qb;
        const QBlock qb = qblocks[it.qb_begin + t % n_qb];
        mbar_wait(&q_empty[st], ph ^ 1, abort_flag, err, 220, 1);
        uint8_t* sq = smem + DkvSmem::kQdO + st * DkvSmem::kStageBytes;
        uint8_t* sdo = sq + 2 * kAtom64;
        mbar_arrive_expect_tx(&q_full[st], DkvSmem::kStageBytes);
        for (int c = 0; c < 2; ++c) {
          tma_load_2d(sq + c * kAtom64, &tmap_q, &q_full[st], hq * kD + c * 64, qb.q_row);
          tma_load_2d(sdo + c * kAtom64, &tmap_do, &q_full[st], hq * kD + c * 64, qb.q_row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false, false);    // [128 keys] x [64 q], K = d
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, 128, false, true);  // P^T (K-major) x dO (MN-major)
      const uint32_t sk = smem_u32(smem + DkvSmem::kK);
      const uint32_t sv = smem_u32(smem + DkvSmem::kV);
      mbar_wait(kv_full, 0, abort_flag, err, 220, 2);
      auto issue_acc = [&](int t) {
        const int b = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        mbar_wait(&p_full[b], ph, abort_flag, err, 220, 3);
        tc_fence_after();
        const uint32_t spt = smem_u32(smem + DkvSmem::kPT + b * kAtom128);
        const uint32_t sdst = smem_u32(smem + DkvSmem::kDST + b * kAtom128);
        const int st = t % DkvSmem::kStages;
        const uint32_t sq = smem_u32(smem + DkvSmem::kQdO + st * DkvSmem::kStageBytes);
        const uint32_t sdo = sq + 2 * kAtom64;
#pragma unroll
        for (int k = 0; k < 64 / 16; ++k) {
          umma_bf16(tmem + 256, umma_smem_desc_sw128(spt + k * 32, 16, 1024),
                    umma_smem_desc_sw128(sdo + k * 2048, kAtom64, 1024), idesc_acc, (t | k) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 64 / 16; ++k) {
          umma_bf16(tmem + 384, umma_smem_desc_sw128(sdst + k * 32, 16, 1024),
                    umma_smem_desc_sw128(sq + k * 2048, kAtom64, 1024), idesc_acc, (t | k) != 0 ? 1u : 0u);
        }
        umma_commit(&p_empty[b]);
        umma_commit(&q_empty[st]);
      };
      for (int t = 0; t < n_iter; ++t) {
        const int b = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        const int st = t % DkvSmem::kStages;
        mbar_wait(&q_full[st], (t / DkvSmem::kStages) & 1, abort_flag, err, 220, 4);
        mbar_wait(&s_empty[b], ph ^ 1, abort_flag, err, 220, 5);
        tc_fence_after();
        const uint32_t sq = smem_u32(smem + DkvSmem::kQdO + st * DkvSmem::kStageBytes);
        const uint32_t sdo = sq + 2 * kAtom64;
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const uint32_t offa = (k >> 2) * kAtom128 + (k & 3) * 32;
          const uint32_t offb = (k >> 2) * kAtom64 + (k & 3) * 32;
          umma_bf16(tmem + b * 64, umma_smem_desc_sw128(sk + offa, 16, 1024), umma_smem_desc_sw128(sq + offb, 16, 1024),
                    idesc_s, k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const uint32_t offa = (k >> 2) * kAtom128 + (k & 3) * 32;
          const uint32_t offb = (k >> 2) * kAtom64 + (k & 3) * 32;
          umma_bf16(tmem + 128 + b * 64, umma_smem_desc_sw128(sv + offa, 16, 1024),
                    umma_smem_desc_sw128(sdo + offb, 16, 1024), idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[b]);
        if (t >= 1) issue_acc(t - 1);
      }
      if (n_iter >= 1) issue_acc(n_iter - 1);
      umma_commit(acc_full);
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // key row within the tile
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const bool key_ok = r < it.k_len;
    const float scale_log2e = scale * kLog2e;
    const int group = (warp - 2) >> 2;  // group g handles the iterations t = g, g + 2, ... (buffer g)
    for (int t = group; t < n_iter; t += 2) {
      const int b = t & 1;
      const uint32_t ph = (t >> 1) & 1;
      const int hq = kv_head * q_per_kv + t / n_qb;
      const QBlock qb = qblocks[it.qb_begin + t % n_qb];
      // columns c (queries) visible to this key row: c < n_rows and (not causal or k_pos + r <= q_pos + c)
      int c_lo = 0;
      if (qb.causal) c_lo = max(0, it.k_pos + r - qb.q_pos);
      const int c_hi = key_ok ? qb.n_rows : 0;
      // stage the block's 64 (lse * log2e, delta) pairs in shared memory: every key row needs all of them
      float* stat = reinterpret_cast<float*>(smem + DkvSmem::kStat) + group * 128;
      const int gt = threadIdx.x - 64 - group * 128;  // 0..127 inside the group
      asm volatile("bar.sync %0, 128;" ::"r"(3 + group) : "memory");  // the previous block's readers are done
      {
        const int c = gt & 63;
        const long long idx = static_cast<long long>(hq) * head_stride + qb.q_row + c;
        float val = 0.f;
        if (c < qb.n_rows) val = gt < 64 ? lse[idx] * kLog2e : delta[idx];
        stat[gt] = val;
      }
      asm volatile("bar.sync %0, 128;" ::"r"(3 + group) : "memory");
      mbar_wait(&s_full[b], ph, abort_flag, err, 220, 6);
      tc_fence_after();
      mbar_wait(&p_empty[b], ph ^ 1, abort_flag, err, 220, 7);
      uint8_t* prow = smem + DkvSmem::kPT + b * kAtom128 + r * 128;
      uint8_t* dsrow = smem + DkvSmem::kDST + b * kAtom128 + r * 128;
      uint32_t ts[64], tp[64];
      tmem_ld_32x32b_x32(tmem + b * 64 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&ts[0]));
      tmem_ld_32x32b_x32(tmem + b * 64 + 32 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&ts[32]));
      tmem_ld_32x32b_x32(tmem + 128 + b * 64 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&tp[0]));
      tmem_ld_32x32b_x32(tmem + 128 + b * 64 + 32 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&tp[32]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(&s_empty[b]);  // S^T / dP^T are in registers: the TMEM buffers are free for block t + 2
      if (__any_sync(0xffffffffu, c_lo > 0 || c_hi < 64)) {
        dkv_row<true>(ts, tp, stat, c_lo, c_hi, scale_log2e, prow, dsrow, r);
      } else {
        dkv_row<false>(ts, tp, stat, c_lo, c_hi, scale_log2e, prow, dsrow, r);
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(&p_full[b]);
    }
    // epilogue: dV (TMEM 256..383) and dK * scale (384..511)
    mbar_wait(acc_full, 0, abort_flag, err, 220, 8);
    tc_fence_after();
    const long long krow = static_cast<long long>(it.k_row) + r;
    // group 0 writes dV, group 1 writes dK
    {
      const int which = group;
      const float mul = which == 0 ? 1.f : scale;
#pragma unroll
      for (int c = 0; c < kD; c += 32) {
        uint32_t t[32];
        if (n_iter >= 1) {
          tmem_ld_32x32b_x32(tmem + 256 + which * 128 + c + lane_addr, t);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = 0u;
        }
        if (!key_ok) continue;
        if (it.out_slot >= 0) {
          float* dst = partials + ((static_cast<long long>(it.out_slot) * num_heads_kv + kv_head) * 2 + which) * (128 * kD) +
                       r * kD + c;
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            reinterpret_cast<float4*>(dst)[v] =
                make_float4(__uint_as_float(t[v * 4]) * mul, __uint_as_float(t[v * 4 + 1]) * mul,
                            __uint_as_float(t[v * 4 + 2]) * mul, __uint_as_float(t[v * 4 + 3]) * mul);
          }
        } else {
          __nv_bfloat16* dst = (which == 0 ? dv : dk) + krow * ld_dkv + kv_head * kD + c;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(t[v * 8 + 2 * i]) * mul,
                                                        __uint_as_float(t[v * 8 + 2 * i + 1]) * mul);
              w[i] = *reinterpret_cast<uint32_t*>(&pk);
            }
            reinterpret_cast<uint4*>(dst)[v] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
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

// Sum the partial slots of a split key tile in slot order and write bf16 dK / dV.
struct ReduceJob {
  int k_row, k_len, slot_begin, slot_end;
};
__global__ void attn_bwd_reduce_kernel(const ReduceJob* __restrict__ jobs, const float* __restrict__ partials,
                                       int num_heads_kv, __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                                       long long ld_dkv) {
  const ReduceJob job = jobs[blockIdx.x];
  const int kv_head = blockIdx.y;
  for (int e = threadIdx.x; e < job.k_len * kD; e += blockDim.x) {
    const int r = e / kD, c = e - r * kD;
    float acc_v = 0.f, acc_k = 0.f;
    for (int s = job.slot_begin; s < job.slot_end; ++s) {
      const float* base = partials + (static_cast<long long>(s) * num_heads_kv + kv_head) * 2 * (128 * kD);
      acc_v += base[r * kD + c];
      acc_k += base[128 * kD + r * kD + c];
    }
    const long long o = (static_cast<long long>(job.k_row) + r) * ld_dkv + kv_head * kD + c;
    dv[o] = __float2bfloat16_rn(acc_v);
    dk[o] = __float2bfloat16_rn(acc_k);
  }
}

template <class K>
void set_max_smem(K kernel, int bytes) {
  static PerDeviceOnce done;
  if (done.first()) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  }
}

}  // namespace

void attention_delta(const __nv_bfloat16* out, const __nv_bfloat16* dout, long long ld, int heads, long long tokens,
                     float* delta, cudaStream_t stream) {
  const long long warps = tokens * heads;
  if (warps <= 0) return;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  attn_delta_kernel<<<static_cast<unsigned int>(blocks), threads, 0, stream>>>(out, dout, ld, heads, tokens, delta);
}

void attention_backward_dq(const AttnBwdArgs& a, cudaStream_t stream) {
  if (a.num_q_tiles <= 0) return;
  const uint64_t wq = static_cast<uint64_t>(a.heads_q) * kD, wk = static_cast<uint64_t>(a.heads_kv) * kD;
  const CUtensorMap tq = make_tmap_2d_bf16(a.q, a.total_q, wq, a.ld_q, 128, 64);
  const CUtensorMap tdo = make_tmap_2d_bf16(a.dout, a.total_q, wq, a.ld_do, 128, 64);
  const CUtensorMap tk = make_tmap_2d_bf16(a.k, a.total_kv, wk, a.ld_k, 64, 64);
  const CUtensorMap tv = make_tmap_2d_bf16(a.v, a.total_kv, wk, a.ld_v, 64, 64);
  set_max_smem(attn_bwd_dq_kernel, DqSmem::kDynamic);
  const long long grid = static_cast<long long>(a.num_q_tiles) * a.heads_q;
  attn_bwd_dq_kernel<<<static_cast<unsigned int>(grid), kThreads, DqSmem::kDynamic, stream>>>(
      tq, tdo, tk, tv, reinterpret_cast<const SeqDesc*>(a.seqs), reinterpret_cast<const int2*>(a.q_tiles), a.heads_q,
      a.heads_q / a.heads_kv, a.causal ? 1 : 0, a.softmax_scale, a.lse, a.delta, a.total_q, a.dq, a.ld_dq, a.err);
}

void attention_backward_dkv(const AttnBwdArgs& a, cudaStream_t stream) {
  if (a.num_kv_items <= 0) return;
  const uint64_t wq = static_cast<uint64_t>(a.heads_q) * kD, wk = static_cast<uint64_t>(a.heads_kv) * kD;
  const CUtensorMap tq = make_tmap_2d_bf16(a.q, a.total_q, wq, a.ld_q, 64, 64);
  const CUtensorMap tdo = make_tmap_2d_bf16(a.dout, a.total_q, wq, a.ld_do, 64, 64);
  const CUtensorMap tk = make_tmap_2d_bf16(a.k, a.total_kv, wk, a.ld_k, 128, 64);
  const CUtensorMap tv = make_tmap_2d_bf16(a.v, a.total_kv, wk, a.ld_v, 128, 64);
  set_max_smem(attn_bwd_dkv_kernel, DkvSmem::kDynamic);
  const long long grid = static_cast<long long>(a.num_kv_items) * a.heads_kv;
  attn_bwd_dkv_kernel<<<static_cast<unsigned int>(grid), kThreads, DkvSmem::kDynamic, stream>>>(
      tq, tdo, tk, tv, reinterpret_cast<const KvItem*>(a.kv_items), reinterpret_cast<const QBlock*>(a.q_blocks),
      a.heads_kv, a.heads_q / a.heads_kv, a.softmax_scale, a.lse, a.delta, a.total_q, a.dk, a.dv, a.ld_dkv, a.partials,
      a.err);
  if (a.num_reduce_jobs > 0) {
    attn_bwd_reduce_kernel<<<dim3(a.num_reduce_jobs, a.heads_kv), 256, 0, stream>>>(
        reinterpret_cast<const ReduceJob*>(a.reduce_jobs), a.partials, a.heads_kv, a.dk, a.dv, a.ld_dkv);
  }
}

}  // namespace rlk
