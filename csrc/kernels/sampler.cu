// Temperature / top-k / top-p sampling, one CTA per row of logits.
//
//   1. a candidate threshold from ONE vectorised pass over the row without atomics: every thread keeps the maximum of
//      its elements, and the k-th largest of the 1024 thread maxima (found by rank counting in shared memory) is a
//      lower bound of the row's k-th largest value, so {x >= threshold} contains the top k and, for ordinary logits,
//      only a few more.  If that set does not fit the candidate buffer (masses of ties), the exact radix select on
//      order-preserving 32-bit keys (integer histograms in shared memory, 12-bit first digit) takes over;
//   2. those candidates are gathered into shared memory and bitonic-sorted by (logit descending, index
//      ascending) -- a total order, so the gather order does not matter -- and cut to the first k plus ties;
//   3. softmax with temperature over the candidates, inclusive scan in a fixed tree, top-p cut
//      "keep token i iff the mass strictly before it is <= p" (first token always kept);
//   4. inverse-CDF draw with a Philox4x32-10 uniform keyed by (seed, row, offset).
//
// The draw is a pure function of (logits row, k, p, T, seed, offset, row index).  The reference
// delegates this to FlashInfer (rl_engine/kernels/sampling.py:41-78: softmax -> top_k_renorm_probs
// -> top_p_sampling_from_probs) and has no kernel of its own.
#include "../common/ptx.cuh"
#include "kernels.h"

#include <cuda_fp16.h>

namespace rlk {

namespace {

constexpr int kThreads = 1024;
constexpr int kCap = 2048;  // candidate capacity (k <= 1024 plus ties)

template <typename T> __device__ __forceinline__ float ldv(const T* p, int i);
template <> __device__ __forceinline__ float ldv<float>(const float* p, int i) { return p[i]; }
template <> __device__ __forceinline__ float ldv<__nv_bfloat16>(const __nv_bfloat16* p, int i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float ldv<__half>(const __half* p, int i) { return __half2float(p[i]); }

__device__ __forceinline__ uint32_t f2key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float -> larger key
}
__device__ __forceinline__ float key2f(uint32_t k) {
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, c.x), lo0 = M0 * c.x;
    const uint32_t hi1 = __umulhi(M1, c.z), lo1 = M1 * c.z;
    c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
    k.x += W0;
    k.y += W1;
  }
  return c;
}

// Calls f(value, index) for every element of the row, thread t taking 16-byte vectors t, t + 1024, ... when the row
// is 16-byte aligned (scalar otherwise).  The visiting order per thread is fixed, the union over threads is the row.
template <typename T, typename F>
__device__ __forceinline__ void for_each_in_row(const T* __restrict__ z, int V, F&& f) {
  constexpr int kVec = 16 / sizeof(T);
  if ((reinterpret_cast<uintptr_t>(z) & 15u) == 0) {
    const int body = V / kVec;
    const uint4* p = reinterpret_cast<const uint4*>(z);
    for (int v = threadIdx.x; v < body; v += kThreads) {
      const uint4 q = p[v];
      const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
      for (int j = 0; j < kVec; ++j) f(ldv(e, j), v * kVec + j);
    }
    for (int i = body * kVec + threadIdx.x; i < V; i += kThreads) f(ldv(z, i), i);
  } else {
    for (int i = threadIdx.x; i < V; i += kThreads) f(ldv(z, i), i);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
sample_topk_topp_kernel(const T* __restrict__ logits, long long ld, int V, int top_k, float top_p, float inv_temp,
                        unsigned long long seed, unsigned long long offset, long long* __restrict__ out_ids,
                        float* __restrict__ out_logprob) {
  __shared__ unsigned int hist[4096];
  __shared__ unsigned long long cand[kCap];
  __shared__ float prob[kCap];
  __shared__ float warp_tot[kThreads / 32];
  __shared__ unsigned int warp_cnt[kThreads / 32];
  __shared__ unsigned int s_prefix, s_remaining, s_above, s_pop, s_count, s_nkeep;
  __shared__ float s_mass;

  const int row = blockIdx.x;
  const T* z = logits + static_cast<long long>(row) * ld;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int k = top_k < 1 ? 1 : (top_k > V ? V : top_k);

  // ---- 1. radix select on order-preserving keys, digits of 12, 8, 8 and 4 bits from the top.  After each digit
  //         the threshold bin is located by a parallel suffix scan; as soon as the elements above the bin plus the
  //         bin itself fit into the candidate buffer the search stops and they are all gathered (the sort below
  //         finds the exact k-th among them).  With k <= 1024 that is the case after the first digit for any
  //         reasonable logit distribution, so a row is read twice (histogram, gather) instead of five times.
  if (tid == 0) {
    s_prefix = 0;
    s_remaining = static_cast<unsigned int>(k);
    s_above = 0;
    s_pop = static_cast<unsigned int>(V);
    s_count = 0;
  }
  // ---- 1a. threshold from the thread maxima (one pass, no atomics).  hist[] doubles as the key array.
  {
    uint32_t best = 0u;  // smaller than the key of any float
    for_each_in_row(z, V, [&](float x, int) {
      const uint32_t key = f2key(x);
      best = key > best ? key : best;
    });
    hist[tid] = best;
    __syncthreads();
    // k-th largest of the 1024 thread maxima by a radix select over their keys (four 8-bit digits from the top;
    // bins in hist[1024 .. 1279], scanned by warp 0): a few microseconds, against tens for comparing all pairs.
    {
      unsigned int* bins = hist + kThreads;
      uint32_t prefix = 0u, mask = 0u;
      unsigned int remaining = static_cast<unsigned int>(k <= kThreads ? k : kThreads);
#pragma unroll 1
      for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) bins[tid] = 0u;
        __syncthreads();
        {
          // warp-aggregated counting: the maxima share their leading bits, so most lanes of a warp hit the same bin
          const bool active = (best & mask) == prefix;
          const uint32_t digit = (best >> shift) & 0xffu;
          const unsigned int peers = __match_any_sync(0xffffffffu, active ? digit : 0xffffffffu);
          if (active && lane == __ffs(peers) - 1) atomicAdd(&bins[digit], static_cast<unsigned int>(__popc(peers)));
        }
        __syncthreads();
        if (warp == 0) {
          // lane l owns bins 255 - 8 l ... 248 - 8 l (highest first); inclusive scan of the lanes' sums
          unsigned int mine = 0u;
#pragma unroll
          for (int j = 0; j < 8; ++j) mine += bins[255 - (lane * 8 + j)];
          unsigned int incl = mine;
#pragma unroll
          for (int off = 1; off < 32; off <<= 1) {
            const unsigned int o = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += o;
          }
          const unsigned int before = incl - mine;
          if (before < remaining && remaining <= incl) {  // exactly one lane: the digit is one of its bins
            unsigned int acc = before;
            int bin = 255 - lane * 8;
            for (int j = 0; j < 8; ++j) {
              bin = 255 - (lane * 8 + j);
              if (acc + bins[bin] >= remaining) break;
              acc += bins[bin];
            }
            s_prefix = prefix | (static_cast<uint32_t>(bin) << shift);
            s_remaining = remaining - acc;
          }
        }
        __syncthreads();
        prefix = s_prefix;
        remaining = s_remaining;
        mask |= 0xffu << shift;
        __syncthreads();
      }
      // s_prefix now is the k-th largest thread maximum: a lower bound of the row's k-th largest key
      if (tid == 0) s_remaining = static_cast<unsigned int>(k);
    }
    __syncthreads();
    const uint32_t from = s_prefix;
    if (k <= kThreads) {
      for_each_in_row(z, V, [&](float x, int i) {
        const uint32_t key = f2key(x);
        if (key >= from) {
          const unsigned int slot = atomicAdd(&s_count, 1u);
          if (slot < kCap) cand[slot] = (static_cast<unsigned long long>(key) << 32) | (0xffffffffu - static_cast<uint32_t>(i));
        }
      });
    }
    __syncthreads();
  }
  const bool gathered = k <= kThreads && s_count <= static_cast<unsigned int>(kCap);  // uniform over the block
  __syncthreads();
  if (!gathered && tid == 0) s_prefix = 0;
  __syncthreads();
  int shift = 32;
#pragma unroll 1
  for (int pass = 0; pass < 4 && !gathered; ++pass) {
    const int bits = pass == 0 ? 12 : (pass == 3 ? 4 : 8);
    if (s_above + s_pop <= static_cast<unsigned int>(kCap)) break;  // uniform: shared values behind a barrier
    const uint32_t himask = pass == 0 ? 0u : (0xffffffffu << shift);
    shift -= bits;
    const int nb = 1 << bits;
    for (int i = tid; i < nb; i += kThreads) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    for (int i = tid; i < V; i += kThreads) {
      const uint32_t key = f2key(ldv(z, i));
      if ((key & himask) == prefix) atomicAdd(&hist[(key >> shift) & static_cast<uint32_t>(nb - 1)], 1u);
    }
    __syncthreads();
    // thread t owns `per` consecutive bins, highest bins first; block-wide exclusive scan of the per-thread sums
    const int per = (nb + kThreads - 1) / kThreads;
    const int top = nb - 1 - tid * per;  // highest bin of this thread
    unsigned int mine = 0;
    for (int j = 0; j < per; ++j)
      if (top - j >= 0) mine += hist[top - j];
    unsigned int incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned int o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += o;
    }
    if (lane == 31) warp_cnt[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      unsigned int w = warp_cnt[lane];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const unsigned int o = __shfl_up_sync(0xffffffffu, w, off);
        if (lane >= off) w += o;
      }
      warp_cnt[lane] = w;
    }
    __syncthreads();
    const unsigned int before = (warp == 0 ? 0u : warp_cnt[warp - 1]) + (incl - mine);  // count in higher bins
    const unsigned int need = s_remaining;
    __syncthreads();
    if (before < need && need <= before + mine) {  // exactly one thread: the threshold bin is one of its bins
      unsigned int acc = before;
      int bsel = top;
      for (int j = 0; j < per; ++j) {
        bsel = top - j;
        if (acc + hist[bsel] >= need) break;
        acc += hist[bsel];
      }
      s_prefix = prefix | (static_cast<uint32_t>(bsel) << shift);
      s_remaining = need - acc;
      s_above += acc;
      s_pop = hist[bsel];
    }
    __syncthreads();
  }
  // keys >= gather_from are candidates: everything above the threshold bin plus the bin itself
  const uint32_t gather_from = s_prefix;

  // ---- 2. gather the candidates (unless 1a already did), then sort (key desc, index asc)
  if (!gathered) {
    if (tid == 0) s_count = 0;
    __syncthreads();
    for (int i = tid; i < V; i += kThreads) {
      const uint32_t key = f2key(ldv(z, i));
      if (key >= gather_from) {
        const unsigned int slot = atomicAdd(&s_count, 1u);
        if (slot < kCap) cand[slot] = (static_cast<unsigned long long>(key) << 32) | (0xffffffffu - static_cast<uint32_t>(i));
      }
    }
    __syncthreads();
  }
  int n = static_cast<int>(s_count < static_cast<unsigned int>(kCap) ? s_count : kCap);
  // sort only as many slots as the candidates need (a power of two >= n, at least 64): the usual few dozen
  // candidates take 21 compare-exchange rounds instead of the 66 of the full buffer
  int sort_n = 64;
  while (sort_n < n) sort_n <<= 1;
  for (int i = n + tid; i < sort_n; i += kThreads) cand[i] = 0ull;
  __syncthreads();
  // bitonic sort, descending, sort_n elements
  for (int size = 2; size <= sort_n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = tid; t < sort_n / 2; t += kThreads) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool desc = ((lo & size) == 0);
        const unsigned long long a = cand[lo], b = cand[hi];
        if ((a < b) == desc) {
          cand[lo] = b;
          cand[hi] = a;
        }
      }
      __syncthreads();
    }
  }

  // the gathered set may extend below the k-th largest value: keep the first k and everything tied with the k-th
  {
    const uint32_t kth_key = static_cast<uint32_t>(cand[(k < n ? k : n) - 1] >> 32);
    if (tid == 0) s_count = 0;
    __syncthreads();
    unsigned int local = 0;
    for (int i = tid; i < n; i += kThreads)
      if (static_cast<uint32_t>(cand[i] >> 32) >= kth_key) ++local;
    if (local) atomicAdd(&s_count, local);
    __syncthreads();
    n = static_cast<int>(s_count);
  }

  // ---- 3. softmax over candidates + inclusive scan (fixed tree) + top-p cut
  const float zmax = key2f(static_cast<uint32_t>(cand[0] >> 32));
  float e0 = 0.f, e1 = 0.f;
  {
    const int i0 = 2 * tid, i1 = 2 * tid + 1;
    if (i0 < n) e0 = expf((key2f(static_cast<uint32_t>(cand[i0] >> 32)) - zmax) * inv_temp);
    if (i1 < n) e1 = expf((key2f(static_cast<uint32_t>(cand[i1] >> 32)) - zmax) * inv_temp);
  }
  float incl = e0 + e1;  // thread total, then warp inclusive scan
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float o = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += o;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    float w = warp_tot[lane];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float o = __shfl_up_sync(0xffffffffu, w, off);
      if (lane >= off) w += o;
    }
    warp_tot[lane] = w;  // inclusive over warps
  }
  __syncthreads();
  const float base = (warp == 0 ? 0.f : warp_tot[warp - 1]) + (incl - (e0 + e1));  // mass before element 2*tid
  if (2 * tid < kCap) {
    prob[2 * tid] = base + e0;
    prob[2 * tid + 1] = base + e0 + e1;
  }
  __syncthreads();
  const float total = warp_tot[kThreads / 32 - 1];
  if (tid == 0) s_nkeep = 0;
  __syncthreads();
  // keep i iff mass strictly before i <= p * total ; kept set is a prefix, so count it
  {
    const float lim = top_p * total;
    unsigned int local = 0;
    const int i0 = 2 * tid, i1 = 2 * tid + 1;
    if (i0 < n && (i0 == 0 || prob[i0 - 1] <= lim)) ++local;
    if (i1 < n && prob[i1 - 1] <= lim) ++local;
    if (local) atomicAdd(&s_nkeep, local);
  }
  __syncthreads();
  const int nkeep = s_nkeep < 1u ? 1 : static_cast<int>(s_nkeep);
  if (tid == 0) s_mass = prob[nkeep - 1];
  __syncthreads();

  // ---- 4. inverse-CDF draw
  if (tid == 0) {
    const uint4 rnd = philox4x32_10(
        make_uint4(static_cast<uint32_t>(offset), static_cast<uint32_t>(offset >> 32), static_cast<uint32_t>(row), 0u),
        make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)));
    const float u = (static_cast<float>(rnd.x >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float target = u * s_mass;
    int lo = 0, hi = nkeep - 1;  // first i with prob[i] > target
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (prob[mid] > target) hi = mid;
      else lo = mid + 1;
    }
    const unsigned long long c = cand[lo];
    out_ids[row] = static_cast<long long>(0xffffffffu - static_cast<uint32_t>(c & 0xffffffffu));
    if (out_logprob) {
      const float e = prob[lo] - (lo ? prob[lo - 1] : 0.f);
      out_logprob[row] = logf(e / s_mass);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Full-vocabulary nucleus sampling (no top-k): temperature softmax over the whole row, keep the
// smallest set of highest-probability tokens whose mass reaches top_p (all tokens tied with the
// cut value are kept), draw by inverse CDF in INDEX order inside the kept set.
//
// The cut is found by a 4-pass radix search over the order-preserving keys, with the bins holding
// probability MASS instead of counts.  Masses are 40-bit fixed point in 64-bit integers, so the
// shared-memory atomics that build the histograms are order-independent and the result is
// deterministic: a pure function of (row, top_p, T, seed, offset, row index).
// ---------------------------------------------------------------------------------------------
constexpr int kNucleusThreads = 1024;

__device__ __forceinline__ unsigned long long fixed_mass(float x, float row_max, float inv_temp) {
  // exp((x - max) / T) in [0, 1], scaled by 2^40 and rounded down; every token gets at least 0
  const float e = __expf((x - row_max) * inv_temp);
  return static_cast<unsigned long long>(e * 1099511627776.0f);
}

template <typename T>
__global__ void __launch_bounds__(kNucleusThreads)
sample_nucleus_kernel(const T* __restrict__ logits, long long ld, int V, float top_p, float inv_temp,
                      unsigned long long seed, unsigned long long offset, long long* __restrict__ out_ids,
                      float* __restrict__ out_logprob) {
  __shared__ unsigned long long hist[256];
  __shared__ unsigned long long warp_part[kNucleusThreads / 32];
  __shared__ float warp_max[kNucleusThreads / 32];
  __shared__ unsigned long long s_total, s_above, s_target, s_base;
  __shared__ uint32_t s_prefix;
  __shared__ int s_pick;
  __shared__ float s_max;
  const int row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* z = logits + static_cast<long long>(row) * ld;

  // ---- row maximum
  float m = -INFINITY;
  for (int i = tid; i < V; i += kNucleusThreads) m = fmaxf(m, ldv(z, i));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) warp_max[warp] = m;
  __syncthreads();
  if (tid == 0) {
    float r = warp_max[0];
    for (int w = 1; w < kNucleusThreads / 32; ++w) r = fmaxf(r, warp_max[w]);
    s_max = r;
    s_prefix = 0u;
    s_above = 0ull;
  }
  __syncthreads();
  const float row_max = s_max;

  // ---- radix search for the cut key: after pass r the top 8*(r+1) bits of the cut are known
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int b = tid; b < 256; b += kNucleusThreads) hist[b] = 0ull;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < V; i += kNucleusThreads) {
      const float x = ldv(z, i);
      const uint32_t key = f2key(x);
      if ((key & mask) == (prefix & mask)) atomicAdd(&hist[(key >> shift) & 0xffu], fixed_mass(x, row_max, inv_temp));
    }
    __syncthreads();
    if (tid == 0) {
      if (pass == 0) {
        unsigned long long total = 0ull;
        for (int b = 0; b < 256; ++b) total += hist[b];
        s_total = total;
        // mass that the kept set must reach (at least one unit so that the best token is always kept)
        const double want = static_cast<double>(top_p) * static_cast<double>(total);
        s_target = want < 1.0 ? 1ull : static_cast<unsigned long long>(want);
      }
      unsigned long long above = s_above;
      int b = 255;
      for (; b > 0; --b) {
        if (above + hist[b] >= s_target) break;
        above += hist[b];
      }
      s_above = above;  // mass of the tokens strictly above the chosen bin
      s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
    }
    __syncthreads();
  }
  const uint32_t cut = s_prefix;  // keep every token with key >= cut

  // ---- mass of the kept set, then the draw
  unsigned long long part = 0ull;
  for (int i = tid; i < V; i += kNucleusThreads) {
    const float x = ldv(z, i);
    if (f2key(x) >= cut) part += fixed_mass(x, row_max, inv_temp);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (lane == 0) warp_part[warp] = part;
  __syncthreads();
  if (tid == 0) {
    unsigned long long kept = 0ull;
    for (int w = 0; w < kNucleusThreads / 32; ++w) kept += warp_part[w];
    const uint4 rnd = philox4x32_10(
        make_uint4(static_cast<uint32_t>(offset), static_cast<uint32_t>(offset >> 32), static_cast<uint32_t>(row), 0u),
        make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)));
    const double u = (static_cast<double>(rnd.x >> 8) + 0.5) * (1.0 / 16777216.0);
    unsigned long long t = static_cast<unsigned long long>(u * static_cast<double>(kept));
    if (t >= kept) t = kept ? kept - 1 : 0ull;
    s_total = kept;
    s_target = t;  // pick the first kept token (index order) whose inclusive cumulative mass exceeds t
    s_base = 0ull;
    s_pick = -1;
  }
  __syncthreads();

  // ---- index-order scan in tiles of kNucleusThreads tokens
  for (int base = 0; base < V && s_pick < 0; base += kNucleusThreads) {
    const int i = base + tid;
    unsigned long long mine = 0ull;
    float x = 0.f;
    if (i < V) {
      x = ldv(z, i);
      if (f2key(x) >= cut) mine = fixed_mass(x, row_max, inv_temp);
    }
    unsigned long long incl = mine;  // inclusive scan inside the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) warp_part[warp] = incl;
    __syncthreads();
    unsigned long long before = s_base;
    for (int w = 0; w < warp; ++w) before += warp_part[w];
    const unsigned long long lo = before + incl - mine, hi = before + incl;
    if (mine != 0ull && lo <= s_target && s_target < hi) {
      s_pick = i;  // exactly one thread satisfies this
      out_ids[row] = i;
      if (out_logprob) out_logprob[row] = logf(static_cast<float>(static_cast<double>(mine) / static_cast<double>(s_total)));
    }
    __syncthreads();
    if (tid == 0) {
      unsigned long long tile = 0ull;
      for (int w = 0; w < kNucleusThreads / 32; ++w) tile += warp_part[w];
      s_base += tile;
    }
    __syncthreads();
  }
  if (tid == 0 && s_pick < 0) {  // all masses rounded to zero except none kept: fall back to the arg-max
    int best = 0;
    float bv = ldv(z, 0);
    for (int i = 1; i < V; ++i) {
      const float x = ldv(z, i);
      if (x > bv) {
        bv = x;
        best = i;
      }
    }
    out_ids[row] = best;
    if (out_logprob) out_logprob[row] = 0.f;
  }
}

}  // namespace

void sample_nucleus(const void* logits, long long ld, int dtype, int rows, int V, float top_p, float temperature,
                    unsigned long long seed, unsigned long long offset, long long* out_ids, float* out_logprob,
                    cudaStream_t stream) {
  if (rows <= 0) return;
  const float inv_temp = 1.f / temperature;
  if (dtype == 0)
    sample_nucleus_kernel<float><<<rows, kNucleusThreads, 0, stream>>>(static_cast<const float*>(logits), ld, V, top_p,
                                                                       inv_temp, seed, offset, out_ids, out_logprob);
  else if (dtype == 1)
    sample_nucleus_kernel<__nv_bfloat16><<<rows, kNucleusThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, V, top_p, inv_temp, seed, offset, out_ids, out_logprob);
  else
    sample_nucleus_kernel<__half><<<rows, kNucleusThreads, 0, stream>>>(static_cast<const __half*>(logits), ld, V, top_p,
                                                                        inv_temp, seed, offset, out_ids, out_logprob);
}

void sample_topk_topp(const void* logits, long long ld, int dtype, int rows, int V, int top_k, float top_p,
                      float temperature, unsigned long long seed, unsigned long long offset, long long* out_ids,
                      float* out_logprob, cudaStream_t stream) {
  if (rows <= 0) return;
  const float inv_temp = 1.f / temperature;
  if (dtype == 0)
    sample_topk_topp_kernel<float><<<rows, kThreads, 0, stream>>>(static_cast<const float*>(logits), ld, V, top_k,
                                                                  top_p, inv_temp, seed, offset, out_ids, out_logprob);
  else if (dtype == 1)
    sample_topk_topp_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), ld,
                                                                          V, top_k, top_p, inv_temp, seed, offset,
                                                                          out_ids, out_logprob);
  else
    sample_topk_topp_kernel<__half><<<rows, kThreads, 0, stream>>>(static_cast<const __half*>(logits), ld, V, top_k,
                                                                   top_p, inv_temp, seed, offset, out_ids, out_logprob);
}

int sample_topk_limit() { return 1024; }

}  // namespace rlk
