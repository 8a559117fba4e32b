// Temperature / top-k / top-p sampling, one CTA per row of logits.
//
//   1. exact k-th largest logit by 4-pass radix select on order-preserving 32-bit keys
//      (integer histograms in shared memory: counts are exact, so the threshold is deterministic);
//   2. candidates (> threshold, plus ties) gathered into shared memory and bitonic-sorted by
//      (logit descending, index ascending) -- a total order, so the gather order does not matter;
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

template <typename T>
__global__ void __launch_bounds__(kThreads)
sample_topk_topp_kernel(const T* __restrict__ logits, long long ld, int V, int top_k, float top_p, float inv_temp,
                        unsigned long long seed, unsigned long long offset, long long* __restrict__ out_ids,
                        float* __restrict__ out_logprob) {
  __shared__ unsigned int hist[256];
  __shared__ unsigned long long cand[kCap];
  __shared__ float prob[kCap];
  __shared__ float warp_tot[kThreads / 32];
  __shared__ unsigned int s_prefix, s_remaining, s_count, s_nkeep;
  __shared__ float s_mass;

  const int row = blockIdx.x;
  const T* z = logits + static_cast<long long>(row) * ld;
  const int tid = threadIdx.x;
  const int k = top_k < 1 ? 1 : (top_k > V ? V : top_k);

  // ---- 1. radix select: key of the k-th largest element
  if (tid == 0) {
    s_prefix = 0;
    s_remaining = static_cast<unsigned int>(k);
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < V; i += kThreads) {
      const uint32_t key = f2key(ldv(z, i));
      if ((key & himask) == prefix) atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned int need = s_remaining;
      int b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= need) break;
        need -= hist[b];
      }
      s_prefix = prefix | (static_cast<uint32_t>(b) << shift);
      s_remaining = need;
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;

  // ---- 2. gather candidates with key >= kth, then sort (key desc, index asc)
  if (tid == 0) s_count = 0;
  __syncthreads();
  for (int i = tid; i < V; i += kThreads) {
    const uint32_t key = f2key(ldv(z, i));
    if (key >= kth) {
      const unsigned int slot = atomicAdd(&s_count, 1u);
      if (slot < kCap) cand[slot] = (static_cast<unsigned long long>(key) << 32) | (0xffffffffu - static_cast<uint32_t>(i));
    }
  }
  __syncthreads();
  const int n = static_cast<int>(s_count < static_cast<unsigned int>(kCap) ? s_count : kCap);
  for (int i = n + tid; i < kCap; i += kThreads) cand[i] = 0ull;
  __syncthreads();
  // bitonic sort, descending, kCap elements (2 per thread)
  for (int size = 2; size <= kCap; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = tid; t < kCap / 2; t += kThreads) {
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

  // ---- 3. softmax over candidates + inclusive scan (fixed tree) + top-p cut
  const float zmax = key2f(static_cast<uint32_t>(cand[0] >> 32));
  float e0 = 0.f, e1 = 0.f;
  {
    const int i0 = 2 * tid, i1 = 2 * tid + 1;
    if (i0 < n) e0 = expf((key2f(static_cast<uint32_t>(cand[i0] >> 32)) - zmax) * inv_temp);
    if (i1 < n) e1 = expf((key2f(static_cast<uint32_t>(cand[i1] >> 32)) - zmax) * inv_temp);
  }
  float incl = e0 + e1;  // thread total, then warp inclusive scan
  const int lane = tid & 31, warp = tid >> 5;
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

}  // namespace

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
