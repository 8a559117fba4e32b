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
// Persistent CTAs (one per SM) walk the list of work items, one item = one 128-query tile of one head.  Warp 0 loads
// Q once per item and K/V tiles through 2-stage TMA rings; warp 1 issues S = Q K^T and O += P V on tcgen05 with S
// double-buffered in TMEM.  Rings, buffers and barriers run on across items, so the next item's Q, K and first S tile
// are in flight while the softmax warps still normalise and store the current item's output.
// Eight softmax warps share the 128 query rows TWO threads per row: warps 2..5 own keys 0..63 of every tile and output
// columns 0..63, warps 6..9 own keys 64..127 and output columns 64..127 (four threads per row, and two independent
// groups alternating over the key tiles, were both measured slower: 0.61 and 0.63 ms against 0.55 ms on the GRPO
// layout).  Each thread pulls its half of the S row with two tcgen05.ld in flight, the two halves exchange their row
// maximum through shared memory (one named barrier per tile), then each runs its half of the online softmax and
// writes its 64-key atom of P as bf16 into the 128B-swizzled smem tile (the A operand of the second MMA).
// O stays in TMEM: every P V product accumulates into the same 128 columns, and the softmax threads rescale them
// (tcgen05.ld, multiply, tcgen05.st) only on tiles where some row's maximum grew by more than 2^8 over the value the
// exponentials are taken against; until then that value lags the true maximum, which changes no result (numerator
// and denominator carry the same factor, at most 2^8, far inside bf16 / fp32 range).  After the first tiles of a row
// that is rare, so the per-tile accumulator traffic (128 fp32 per row in and out of registers) is gone.
#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "kernels.h"

namespace rlk {

#ifdef RLK_ATTN_PROFILE
// Phase timing of one softmax thread (debug builds only): cycles accumulated per phase over the tiles of one CTA.
__device__ unsigned long long g_attn_prof[16];
#define PROF_DECL unsigned long long prof_t = clock64(); const bool prof_on = (blockIdx.x == gridDim.x / 2) && threadIdx.x == 64
#define PROF(slot)                                   \
  if (prof_on) {                                     \
    const unsigned long long now = clock64();        \
    atomicAdd(&g_attn_prof[slot], now - prof_t);     \
    prof_t = now;                                    \
  }
void attention_profile_read(unsigned long long* out) { cudaMemcpyFromSymbol(out, g_attn_prof, sizeof(unsigned long long) * 16); }
void attention_profile_reset() { unsigned long long z[16] = {0}; cudaMemcpyToSymbol(g_attn_prof, z, sizeof(z)); }
#else
#define PROF_DECL
#define PROF(slot)
#endif

namespace {

constexpr int kD = 128;        // head dim
constexpr int kTileQ = 128;
constexpr int kTileK = 128;
constexpr int kThreads = 320;
constexpr int kSoftmaxThreads = 256;
constexpr int kTileBytes = kTileQ * kD * 2;  // 32 KB: two 128B-swizzle atoms of [128 x 64]
constexpr int kAtomBytes = 128 * 64 * 2;     // 16 KB

struct Smem {
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;       // 2 stages
  static constexpr int kV = kK + 2 * kTileBytes;   // 2 stages
  static constexpr int kP = kV + 2 * kTileBytes;   // 2 buffers
  static constexpr int kXmax = kP + 2 * kTileBytes;  // float [2 halves][128 rows]: row-maximum exchange
  static constexpr int kBars = kXmax + 2 * 128 * 4;
  // q_full, k_full[2], k_empty[2], s_full[2], s_empty[2], p_full[2], o_full[2], o_done, o_free, v_full[2], v_empty[2], q_empty
  static constexpr int kNumBars = 20;
  static constexpr int kBytes = kBars + kNumBars * 8 + 16;
  static constexpr int kDynamic = kBytes + 1024;
};
static_assert(Smem::kDynamic <= 232448, "attention forward exceeds the 227 KB shared-memory limit");

struct SeqDesc {  // one per sequence, int32 x 8
  int q_start, q_len, pk_start, pk_len, sk_start, sk_len, pad0, pad1;
};

// Half a score row (64 keys) of one query: p = 2^(s * scale - m) packed to bf16 into the row's 128-byte swizzle
// line; returns the fp32 sum.  One exponential in four runs on the FMA pipe (poly_exp2), the rest on MUFU.
// MASKED = false is the common case of a tile that is entirely visible to the row.
template <bool MASKED>
__device__ __forceinline__ float softmax_half_row(const uint32_t (&t)[64], int limit, float scale_log2e, float m_safe,
                                                  uint8_t* prow, int r) {
  float sum = 0.f;
#pragma unroll
  for (int c8 = 0; c8 < 8; ++c8) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int col = c8 * 8 + 2 * i;
      const float x0 = fmaf(__uint_as_float(t[col]), scale_log2e, -m_safe);
      const float x1 = fmaf(__uint_as_float(t[col + 1]), scale_log2e, -m_safe);
      float p0 = fast_exp2(x0);
      float p1 = (i & 1) ? poly_exp2(x1) : fast_exp2(x1);
      if (MASKED) {
        p0 = col < limit ? p0 : 0.f;
        p1 = col + 1 < limit ? p1 : 0.f;
      }
      sum += p0 + p1;
      __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
      w[i] = *reinterpret_cast<uint32_t*>(&pk);
    }
    // 128B swizzle: 16-byte chunk index XOR (row mod 8)
    *reinterpret_cast<uint4*>(prow + ((c8 ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  return sum;
}

template <bool MASKED>
__device__ __forceinline__ float max_half_row(const uint32_t (&t)[64], int limit) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 64; i += 4) {
    if (!MASKED || i < limit) m0 = fmaxf(m0, __uint_as_float(t[i]));
    if (!MASKED || i + 1 < limit) m1 = fmaxf(m1, __uint_as_float(t[i + 1]));
    if (!MASKED || i + 2 < limit) m2 = fmaxf(m2, __uint_as_float(t[i + 2]));
    if (!MASKED || i + 3 < limit) m3 = fmaxf(m3, __uint_as_float(t[i + 3]));
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// One work item = one 128-query tile of one head; what every role needs to know about it.
struct Item {
  SeqDesc sd;
  int q0, head, kv_head, n_prefix, n_tiles;
  bool ok;
};

__device__ __forceinline__ Item decode_item(int w, const SeqDesc* __restrict__ seqs, const int2* __restrict__ tiles,
                                            int num_heads_q, int q_per_kv, int causal, int num_seqs, int total_q,
                                            int total_kv, uint32_t* err) {
  Item it;
  const int tile_id = w / num_heads_q;
  it.head = w - tile_id * num_heads_q;
  it.kv_head = it.head / q_per_kv;
  const int2 tile = tiles[tile_id];
  it.q0 = tile.y;
  it.n_prefix = it.n_tiles = 0;
  // The layout tables come from the caller.  Debug-bounds builds check them against the tensors before anything is
  // read or written through them; every role of the CTA decodes the same item and takes the same decision.
  it.ok = RLK_INDEX_OK(tile.x, num_seqs, err, 200u, 1);
  if (!it.ok) return it;
  it.sd = seqs[tile.x];
  it.ok = RLK_INDEX_OK(it.q0, it.sd.q_len > 0 ? it.sd.q_len : 1, err, 200u, 2) &&
          RLK_INDEX_OK(it.sd.q_start, total_q - it.sd.q_len + 1, err, 200u, 3) &&
          RLK_INDEX_OK(it.sd.pk_start, total_kv - it.sd.pk_len + 1, err, 200u, 4) &&
          RLK_INDEX_OK(it.sd.sk_start, total_kv - it.sd.sk_len + 1, err, 200u, 5);
  if (!it.ok) return it;
  it.n_prefix = (it.sd.pk_len + kTileK - 1) / kTileK;
  int self_keys = it.sd.sk_len;
  if (causal) self_keys = min(self_keys, it.q0 + kTileQ);
  it.n_tiles = it.n_prefix + (self_keys + kTileK - 1) / kTileK;
  return it;
}

// Persistent: CTA c handles work items total - 1 - c, total - 1 - c - gridDim.x, ... (the caller's tile list usually
// ends with the sequences that see the most keys, so the heavy items go first and the light ones fill the tail).
// The K / V rings, the S and P buffers and their barriers run on across items (`g`, the number of key tiles this CTA
// has handled so far, selects buffer and phase), so the loader and the MMA warp start on the next item's Q, K and S
// while the softmax warps still normalise and store the current item's output: the per-item set-up, the first loads
// from DRAM and the output stores are hidden, which was about half of a CTA's lifetime when one CTA handled one item.
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const SeqDesc* __restrict__ seqs,
                const int2* __restrict__ tiles,  // (sequence, first query row within the sequence)
                int total_items, int num_heads_q, int q_per_kv, int causal, float scale_log2e,
                __nv_bfloat16* __restrict__ out, long long ld_out, float* __restrict__ lse, long long lse_head_stride,
                uint32_t* __restrict__ err, int num_seqs, int total_q, int total_kv) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
  uint64_t* q_full = bars;
  // K and V have separate rings: a K stage is free as soon as S = Q K^T of its tile has completed, long before
  // the P V product releases the V stage, so the K tile two steps ahead is in flight while the softmax runs.
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 3;
  uint64_t* v_full = bars + 15;
  uint64_t* v_empty = bars + 17;
  uint64_t* s_full = bars + 5;
  uint64_t* s_empty = bars + 7;
  uint64_t* p_full = bars + 9;
  uint64_t* o_full = bars + 11;   // P V of a tile has completed (commit per product; waited where O or P[b] is touched)
  uint64_t* o_done = bars + 13;   // per item: every product of the item has completed
  uint64_t* o_free = bars + 14;   // per item: the softmax warps have pulled the item's O out of TMEM
  uint64_t* q_empty = bars + 19;  // per item: every S product of the item has completed, Q may be overwritten
  float* xmax_s = reinterpret_cast<float*>(smem + Smem::kXmax);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Smem::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(o_done, 1);
    mbar_init(o_free, kSoftmaxThreads / 32);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&k_full[b], 1);
      mbar_init(&k_empty[b], 1);
      mbar_init(&v_full[b], 1);
      mbar_init(&v_empty[b], 1);
      mbar_init(&s_full[b], 1);
      mbar_init(&s_empty[b], kSoftmaxThreads / 32);  // one arrival per softmax warp
      mbar_init(&p_full[b], kSoftmaxThreads / 32);
      mbar_init(&o_full[b], 1);
    }
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
  const int first = total_items - 1 - static_cast<int>(blockIdx.x), step = static_cast<int>(gridDim.x);
#define RLK_ATTN_ITEM(w) decode_item(w, seqs, tiles, num_heads_q, q_per_kv, causal, num_seqs, total_q, total_kv, err)

  if (warp == 0) {
    if (lane == 0) {
      int g0 = 0, n_item = 0;  // key tiles and items (with at least one key tile) handled so far
      // The next item's descriptor is fetched while the current one is worked on: its two dependent global loads
      // (tile entry, then sequence entry) would otherwise sit on the critical path between two items.
      Item next = RLK_ATTN_ITEM(first);
      for (int w = first; w >= 0 && !*abort_flag; w -= step) {
        const Item it = next;
        if (w - step >= 0) next = RLK_ATTN_ITEM(w - step);
        if (!it.ok || it.n_tiles == 0) continue;
        mbar_wait(q_empty, (n_item & 1) ^ 1, abort_flag, err, 200, 15);  // the previous item's S products are done with Q
        mbar_arrive_expect_tx(q_full, kTileBytes);
        tma_load_2d(smem + Smem::kQ, &tmap_q, q_full, it.head * kD, it.sd.q_start + it.q0);
        tma_load_2d(smem + Smem::kQ + kAtomBytes, &tmap_q, q_full, it.head * kD + 64, it.sd.q_start + it.q0);
        auto key_row = [&](int j) {
          return j < it.n_prefix ? it.sd.pk_start + j * kTileK : it.sd.sk_start + (j - it.n_prefix) * kTileK;
        };
        auto load_k = [&](int j) {
          const int g = g0 + j, b = g & 1;
          mbar_wait(&k_empty[b], ((g >> 1) & 1) ^ 1, abort_flag, err, 200, 1);
          mbar_arrive_expect_tx(&k_full[b], kTileBytes);
          uint8_t* sk = smem + Smem::kK + b * kTileBytes;
          tma_load_2d(sk, &tmap_k, &k_full[b], it.kv_head * kD, key_row(j));
          tma_load_2d(sk + kAtomBytes, &tmap_k, &k_full[b], it.kv_head * kD + 64, key_row(j));
        };
        auto load_v = [&](int j) {
          const int g = g0 + j, b = g & 1;
          mbar_wait(&v_empty[b], ((g >> 1) & 1) ^ 1, abort_flag, err, 200, 13);
          mbar_arrive_expect_tx(&v_full[b], kTileBytes);
          uint8_t* sv = smem + Smem::kV + b * kTileBytes;
          tma_load_2d(sv, &tmap_v, &v_full[b], it.kv_head * kD, key_row(j));
          tma_load_2d(sv + kAtomBytes, &tmap_v, &v_full[b], it.kv_head * kD + 64, key_row(j));
        };
        // K runs one tile ahead of V in issue order: K(j + 1) only waits for S(j - 1), V(j) for P V of tile j - 2
        load_k(0);
        for (int j = 0; j < it.n_tiles; ++j) {
          if (j + 1 < it.n_tiles) load_k(j + 1);
          load_v(j);
        }
        g0 += it.n_tiles;
        ++n_item;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, false, false);  // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, 128, false, true);   // P (K-major) x V (MN-major)
      const uint32_t sq = smem_u32(smem + Smem::kQ);
      int g0 = 0, n_item = 0;
      // P V of a tile is issued one S product later than the tile's own S product, across item boundaries too: the
      // first S tile of the next item is computed while the softmax warps finish the last tile of this one.
      struct Pending {
        int g, item;       // global key-tile index and item index of the product that is still to be issued
        bool first, last;  // first / last key tile of its item
      } pend{0, 0, false, false};
      bool have_pend = false;
      auto issue_pv = [&](const Pending& pv) {
        const int b = pv.g & 1;
        const uint32_t ph = (pv.g >> 1) & 1;
        mbar_wait(&p_full[b], ph, abort_flag, err, 200, 3);  // also orders any rescale of O before this product
        mbar_wait(&v_full[b], ph, abort_flag, err, 200, 14);
        // the first product of an item overwrites O: the softmax warps must have read the previous item's
        if (pv.first) mbar_wait(o_free, (pv.item & 1) ^ 1, abort_flag, err, 200, 16);
        tc_fence_after();
        const uint32_t sp = smem_u32(smem + Smem::kP + b * kTileBytes);
        const uint32_t sv = smem_u32(smem + Smem::kV + b * kTileBytes);
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k) {
          // A = P: K-major, K = keys; 4 k-steps per 64-key atom.  B = V: MN-major, 16 key rows = 2048 bytes.
          const uint64_t da = umma_smem_desc_sw128(sp + (k >> 2) * kAtomBytes + (k & 3) * 32, 16, 1024);
          const uint64_t db = umma_smem_desc_sw128(sv + k * 2048, kAtomBytes, 1024);
          umma_bf16(tmem + 256, da, db, idesc_o, (!pv.first || k != 0) ? 1u : 0u);
        }
        umma_commit(&o_full[b]);
        umma_commit(&v_empty[b]);
        if (pv.last) umma_commit(o_done);
      };
      Item next = RLK_ATTN_ITEM(first);
      for (int w = first; w >= 0 && !*abort_flag; w -= step) {
        const Item it = next;
        if (w - step >= 0) next = RLK_ATTN_ITEM(w - step);
        if (!it.ok || it.n_tiles == 0) continue;
        mbar_wait(q_full, n_item & 1, abort_flag, err, 200, 2);
        for (int j = 0; j < it.n_tiles; ++j) {
          const int g = g0 + j, b = g & 1;
          const uint32_t ph = (g >> 1) & 1;
          mbar_wait(&k_full[b], ph, abort_flag, err, 200, 5);
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
          umma_commit(&k_empty[b]);
          if (j + 1 == it.n_tiles) umma_commit(q_empty);  // every S product of the item has been issued
          if (have_pend) issue_pv(pend);
          pend = Pending{g, n_item, j == 0, j + 1 == it.n_tiles};
          have_pend = true;
        }
        g0 += it.n_tiles;
        ++n_item;
      }
      if (have_pend) issue_pv(pend);
    }
  } else {
    // ------------------------------ softmax / output warps ------------------------------
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;  // 0: keys / output columns 0..63, 1: 64..127
    const int r = quad * 32 + lane;    // query row within the tile
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    constexpr int kHalf = 64;
    constexpr float kLazy = 8.f;  // the exponent base follows the row maximum only in steps of more than 2^8
    const uint32_t o_addr = tmem + 256 + half * kHalf + lane_addr;
    int g0 = 0, n_item = 0;
    PROF_DECL;

    Item next = RLK_ATTN_ITEM(first);
    for (int w = first; w >= 0 && !*abort_flag; w -= step) {
      const Item it = next;
      if (w - step >= 0) next = RLK_ATTN_ITEM(w - step);
      if (!it.ok) continue;
      const SeqDesc& sd = it.sd;
      const int qi = it.q0 + r;  // query index within the sequence
      float m_used = -INFINITY, l = 0.f;  // m_used: what the exponentials are taken against (log2 domain, scaled)

      for (int j = 0; j < it.n_tiles; ++j) {
        const int g = g0 + j, b = g & 1;
        const uint32_t ph = (g >> 1) & 1;
        const bool is_self = j >= it.n_prefix;
        const int key0 = is_self ? (j - it.n_prefix) * kTileK : j * kTileK;
        const int range_len = is_self ? sd.sk_len : sd.pk_len;
        int limit = range_len - key0;  // keys [0, limit) of this tile are in range
        if (is_self && causal) limit = min(limit, qi - key0 + 1);
        limit -= half * kHalf;         // in this thread's 64 columns
        PROF(0);
        mbar_wait(&s_full[b], ph, abort_flag, err, 200, 8);
        PROF(1);
        tc_fence_after();
        // this thread's half of the S row: both loads in flight, one wait, then the TMEM buffer is released
        uint32_t t[kHalf];
        tmem_ld_32x32b_x32(tmem + b * 128 + half * kHalf + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&t[0]));
        tmem_ld_32x32b_x32(tmem + b * 128 + half * kHalf + 32 + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&t[32]));
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive_warp(&s_empty[b]);
        PROF(2);
        // a tile is mask-free for the whole warp in all but the diagonal and the last tile of a range
        const bool masked = __any_sync(0xffffffffu, limit < kHalf);
        float mx = masked ? max_half_row<true>(t, limit) : max_half_row<false>(t, limit);
        // exchange the half-row maxima through shared memory; the second barrier keeps the next tile's writes
        // behind this tile's reads
        xmax_s[half * 128 + r] = mx;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");  // only the two warps that share these 32 rows
        mx = fmaxf(mx, xmax_s[(half ^ 1) * 128 + r]);
        asm volatile("bar.sync %0, 64;" ::"r"(5 + quad) : "memory");
        PROF(3);
        // Both threads of a row hold the same mx, so both take the same branch and keep the same m_used.
        const float cand = fmaxf(m_used, mx * scale_log2e);
        if (j == 0) {
          m_used = cand;  // nothing accumulated yet
        } else if (__any_sync(0xffffffffu, cand - m_used > kLazy)) {  // (-inf) - (-inf) = NaN compares false
          const float alpha = cand == -INFINITY ? 1.f : fast_exp2(m_used - cand);  // m_used = -inf -> 0
          // O holds the products up to tile j - 1 once P V of that tile has completed; P V of tile j is issued only
          // after every softmax warp has arrived on p_full below, i.e. after this rescale.
          mbar_wait(&o_full[b ^ 1], ((g - 1) >> 1) & 1, abort_flag, err, 200, 7);
          tc_fence_after();
          uint32_t o0[32], o1[32];
          tmem_ld_32x32b_x32(o_addr, o0);
          tmem_ld_32x32b_x32(o_addr + 32, o1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            o0[i] = __float_as_uint(__uint_as_float(o0[i]) * alpha);
            o1[i] = __float_as_uint(__uint_as_float(o1[i]) * alpha);
          }
          tmem_st_32x32b_x32(o_addr, o0);
          tmem_st_32x32b_x32(o_addr + 32, o1);
          tmem_st_wait();
          tc_fence_before();
          l *= alpha;
          m_used = cand;
        }
        const float m_safe = m_used == -INFINITY ? 0.f : m_used;
        // P[b] was the A operand of P V two tiles ago: that product must have finished reading it.  (For the first
        // two tiles of an item that product belongs to the previous item, whose o_done this thread has waited for.)
        if (j >= 2) mbar_wait(&o_full[b], ((g - 2) >> 1) & 1, abort_flag, err, 200, 4);
        // 64 keys of a row = one 128-byte swizzle row of atom `half`
        uint8_t* prow = smem + Smem::kP + b * kTileBytes + half * kAtomBytes + r * 128;
        const float sum = masked ? softmax_half_row<true>(t, limit, scale_log2e, m_safe, prow, r)
                                 : softmax_half_row<false>(t, limit, scale_log2e, m_safe, prow, r);
        l += sum;  // this thread's share of the row sum; both halves use the same m_used
        fence_proxy_async_smem();
        mbar_arrive_warp(&p_full[b]);
        PROF(4);
      }

      // this thread's 64 columns of O, once the item's last product has completed; then TMEM is handed back so that
      // the next item's first product may overwrite it while this item is normalised and stored
      uint32_t o[kHalf];  // fp32 bits
      if (it.n_tiles >= 1) {
        mbar_wait(o_done, n_item & 1, abort_flag, err, 200, 9);
        tc_fence_after();
        tmem_ld_32x32b_x32(o_addr, *reinterpret_cast<uint32_t(*)[32]>(&o[0]));
        tmem_ld_32x32b_x32(o_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&o[32]));
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive_warp(o_free);
        g0 += it.n_tiles;
        ++n_item;
      } else {
#pragma unroll
        for (int i = 0; i < kHalf; ++i) o[i] = 0u;
      }
      const float m2 = m_used;

      // total row sum = the two halves' shares (the exchange buffer is free: every reader passed barrier 5 + quad;
      // the barrier after the read keeps the next item's first write behind it)
      xmax_s[half * 128 + r] = l;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
      l += xmax_s[(half ^ 1) * 128 + r];
      asm volatile("bar.sync %0, 64;" ::"r"(5 + quad) : "memory");

      if (qi < sd.q_len) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = out + static_cast<long long>(sd.q_start + qi) * ld_out + it.head * kD + half * kHalf;
#pragma unroll
        for (int c8 = 0; c8 < kHalf / 8; ++c8) {
          uint32_t wd[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(o[c8 * 8 + 2 * i]) * inv,
                                                      __uint_as_float(o[c8 * 8 + 2 * i + 1]) * inv);
            wd[i] = *reinterpret_cast<uint32_t*>(&pk);
          }
          reinterpret_cast<uint4*>(dst)[c8] = make_uint4(wd[0], wd[1], wd[2], wd[3]);
        }
        if (lse != nullptr && half == 0) {
          lse[static_cast<long long>(it.head) * lse_head_stride + sd.q_start + qi] =
              l > 0.f ? (m2 + log2f(l)) * kLn2 : -INFINITY;
        }
      }
    }
  }
#undef RLK_ATTN_ITEM

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
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kDynamic);
  }
  const long long items = static_cast<long long>(a.num_tiles) * a.heads_q;
  const long long grid = items < a.sm_count ? items : a.sm_count;  // one persistent CTA per SM (227 KB of shared memory each)
  attn_fwd_kernel<<<static_cast<unsigned int>(grid), kThreads, Smem::kDynamic, stream>>>(
      tq, tk, tv, reinterpret_cast<const SeqDesc*>(a.seqs), reinterpret_cast<const int2*>(a.tiles),
      static_cast<int>(items), a.heads_q, a.heads_q / a.heads_kv, a.causal ? 1 : 0, a.softmax_scale * kLog2e, a.out, a.ld_out, a.lse, a.lse_head_stride,
      a.err, a.num_seqs, static_cast<int>(a.total_q), static_cast<int>(a.total_kv));
}

}  // namespace rlk
