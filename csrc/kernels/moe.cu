// Mixture-of-experts support kernels (Qwen3-MoE style: softmax over all experts, top-k, renormalise):
//   moe_topk           : per token, the k largest router probabilities (ties -> lower expert id) and their
//                        renormalised weights; one warp per token, fixed-order reductions.
//   moe_topk_backward  : gradient of those weights with respect to the logits (softmax over the selected logits).
//   moe_gather_rows    : dst[slot] = scale[slot] * src[src_row[slot]]  (src_row < 0 -> zero row).  With peer
//                        destination pointers this is the all-to-all DISPATCH: every rank stores the rows it
//                        routes to expert e directly into the owning rank's expert-grouped buffer over NVLink.
//   moe_combine        : out[t] = sum_j w[t, j] * src[slot[t, j]] in fixed j order (deterministic); `src` may
//                        live on a peer (the all-to-all COMBINE is this kernel reading peer memory).
//   moe_rowdot         : d w[t, j] = <dout[t], y[slot[t, j]]>.
// The reference has no MoE code (its README only shows a log-prob benchmark on Qwen3-30B-A3B).
#include "../common/ptx.cuh"
#include "kernels.h"

namespace rlk {

namespace {

__global__ void moe_topk_kernel(const float* __restrict__ logits, int tokens, int experts, int k,
                                int* __restrict__ idx, float* __restrict__ weight) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const float* row = logits + static_cast<long long>(t) * experts;
  // softmax statistics over all experts (experts <= 32 * 16)
  float v[16];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < experts ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[i] = (lane + 32 * i) < experts ? expf(v[i] - mx) : -1.f;  // probabilities (unnormalised); -1 = absent
    if (v[i] > 0.f) sum += v[i];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  float picked_sum = 0.f;
  float my_w = 0.f;
  int my_e = 0;
  for (int j = 0; j < k; ++j) {
    float best = -2.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best || (v[i] == best && e < best_e)) {
        best = v[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) v[best_e >> 5] = -1.f;  // remove the winner
    picked_sum += best;
    if (lane == j) {
      my_w = best;
      my_e = best_e;
    }
  }
  if (lane < k) {
    idx[static_cast<long long>(t) * k + lane] = my_e;
    weight[static_cast<long long>(t) * k + lane] = my_w / picked_sum;
  }
  (void)sum;
}

// Gradient of the renormalised top-k weights with respect to the router logits.  The weights are a softmax over the
// k selected logits, so d logit[e_i] = w_i * (dw_i - sum_j w_j dw_j) and every unselected logit gets zero.  One warp
// per token writes the whole row (zeros and the k values).
__global__ void moe_topk_bwd_kernel(const int* __restrict__ idx, const float* __restrict__ weight,
                                    const float* __restrict__ dweight, int tokens, int experts, int k,
                                    float* __restrict__ dlogits) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const long long base = static_cast<long long>(t) * k;
  const float w = lane < k ? weight[base + lane] : 0.f;
  const float dw = lane < k ? dweight[base + lane] : 0.f;
  float dot = w * dw;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
  float* row = dlogits + static_cast<long long>(t) * experts;
  for (int e = lane; e < experts; e += 32) row[e] = 0.f;
  __syncwarp();
  if (lane < k) {
    const int e = idx[base + lane];
    if (e >= 0 && e < experts) row[e] = w * (dw - dot);
  }
}

__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ src, long long ld_src,
                                       const int* __restrict__ src_row, const float* __restrict__ scale,
                                       __nv_bfloat16* __restrict__ dst, long long ld_dst, int slots, int h8,
                                       long long src_rows, uint32_t* err) {
  const int slot = blockIdx.x;
  if (slot >= slots) return;
  const int r = src_row[slot];
  if (r >= 0 && !RLK_INDEX_OK(r, src_rows, err, 500u, 1)) return;
  uint4* out = reinterpret_cast<uint4*>(dst + static_cast<long long>(slot) * ld_dst);
  if (r < 0) {
    for (int i = threadIdx.x; i < h8; i += blockDim.x) out[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* in = reinterpret_cast<const uint4*>(src + static_cast<long long>(r) * ld_src);
  const float s = scale ? scale[slot] : 1.f;
  for (int i = threadIdx.x; i < h8; i += blockDim.x) {
    uint4 q = in[i];
    if (scale) {
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        h[j] = __floats2bfloat162_rn(f.x * s, f.y * s);
      }
    }
    out[i] = q;
  }
}

__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ src, long long ld_src, const int* __restrict__ slot,
                                   const float* __restrict__ weight, int k, __nv_bfloat16* __restrict__ out,
                                   long long ld_out, int tokens, int h8, long long src_rows, uint32_t* err) {
  const int t = blockIdx.x;
  if (t >= tokens) return;
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(t) * ld_out);
  for (int i = threadIdx.x; i < h8; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int j = 0; j < k; ++j) {  // fixed order
      const int s = slot[static_cast<long long>(t) * k + j];
      if (s < 0) continue;
      if (src_rows > 0 && !RLK_INDEX_OK(s, src_rows, err, 501u, 1)) continue;
      const float w = weight ? weight[static_cast<long long>(t) * k + j] : 1.f;
      const uint4 q = reinterpret_cast<const uint4*>(src + static_cast<long long>(s) * ld_src)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = fmaf(w, f.x, acc[2 * e]);
        acc[2 * e + 1] = fmaf(w, f.y, acc[2 * e + 1]);
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    dst[i] = o;
  }
}

__global__ void moe_rowdot_kernel(const __nv_bfloat16* __restrict__ a, long long ld_a, const __nv_bfloat16* __restrict__ b,
                                  long long ld_b, const int* __restrict__ slot, int k, int tokens, int h8,
                                  float* __restrict__ out) {
  const int pair = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (pair >= tokens * k) return;
  const int t = pair / k;
  const int s = slot[pair];
  float acc = 0.f;
  if (s >= 0) {
    const uint4* pa = reinterpret_cast<const uint4*>(a + static_cast<long long>(t) * ld_a);
    const uint4* pb = reinterpret_cast<const uint4*>(b + static_cast<long long>(s) * ld_b);
    for (int i = lane; i < h8; i += 32) {
      const uint4 x = pa[i], y = pb[i];
      const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&x);
      const __nv_bfloat162* hy = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(hx[e]), g = __bfloat1622float2(hy[e]);
        acc = fmaf(f.x, g.x, acc);
        acc = fmaf(f.y, g.y, acc);
      }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) out[pair] = acc;
}

struct PeerBases {
  void* p[8];
};

// Expert-parallel DISPATCH: assignment a (one CTA each) copies row src[token[a]] (times scale[a] if given)
// into rank dest_rank[a]'s slot buffer at row dest_slot[a] with plain stores over NVLink.
__global__ void moe_scatter_rows_peer_kernel(const __nv_bfloat16* __restrict__ src, long long ld_src,
                                             const int* __restrict__ token, const int* __restrict__ dest_rank,
                                             const int* __restrict__ dest_slot, const float* __restrict__ scale,
                                             PeerBases dst, long long ld_dst, int assignments, int h8) {
  const int a = blockIdx.x;
  if (a >= assignments) return;
  const uint4* in = reinterpret_cast<const uint4*>(src + static_cast<long long>(token[a]) * ld_src);
  uint4* out = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(dst.p[dest_rank[a]]) +
                                        static_cast<long long>(dest_slot[a]) * ld_dst);
  const float s = scale ? scale[a] : 1.f;
  for (int i = threadIdx.x; i < h8; i += blockDim.x) {
    uint4 q = in[i];
    if (scale) {
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        h[j] = __floats2bfloat162_rn(f.x * s, f.y * s);
      }
    }
    out[i] = q;
  }
}

// Expert-parallel COMBINE: out[t] = sum_j w[t, j] * buffer_{rank[t, j]}[slot[t, j]] read from the peers in
// fixed j order.
__global__ void moe_combine_peer_kernel(PeerBases src, long long ld_src, const int* __restrict__ rank,
                                        const int* __restrict__ slot, const float* __restrict__ weight, int k,
                                        __nv_bfloat16* __restrict__ out, long long ld_out, int tokens, int h8) {
  const int t = blockIdx.x;
  if (t >= tokens) return;
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(t) * ld_out);
  for (int i = threadIdx.x; i < h8; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int j = 0; j < k; ++j) {
      const long long a = static_cast<long long>(t) * k + j;
      const float w = weight ? weight[a] : 1.f;
      const uint4 q = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(src.p[rank[a]]) +
                                                      static_cast<long long>(slot[a]) * ld_src)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = fmaf(w, f.x, acc[2 * e]);
        acc[2 * e + 1] = fmaf(w, f.y, acc[2 * e + 1]);
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    dst[i] = o;
  }
}

// ---------------------------------------------------------------------------------------------
// Dispatch plan in three small kernels (instead of a dozen framework index ops): assignments are
// grouped expert by expert, every expert block padded to 128 rows, order inside an expert = assignment
// order (so every later summation order is fixed).
//   count : per 256-assignment chunk, histogram over experts                     -> chunk_hist [chunks, E]
//   scan  : per expert, exclusive prefix over the chunks (in place) and totals; padded expert offsets;
//           expert id of every 128-row tile (unused tail tiles get `unused_group`)
//   place : slot of every assignment = offsets[e] + prefix[chunk, e] + rank inside the chunk;
//           src_row[slot] = token
// ---------------------------------------------------------------------------------------------
constexpr int kPlanChunk = 256;

__global__ void moe_plan_count_kernel(const int* __restrict__ idx, int assignments, int experts, int* __restrict__ chunk_hist) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int a = blockIdx.x * kPlanChunk + threadIdx.x;
  if (a < assignments) atomicAdd(&hist[idx[a]], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) chunk_hist[blockIdx.x * experts + e] = hist[e];
}

__global__ void moe_plan_scan_kernel(int* __restrict__ chunk_hist, int chunks, int experts, int num_tiles, int unused_group,
                                     int* __restrict__ offsets, int* __restrict__ counts, int* __restrict__ tile_group) {
  extern __shared__ int off_s[];  // experts + 1
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < chunks; ++c) {
      const int v = chunk_hist[c * experts + e];
      chunk_hist[c * experts + e] = run;  // assignments of this expert in earlier chunks
      run += v;
    }
    counts[e] = run;
    const int blocks = run > 0 ? (run + 127) / 128 : 1;
    off_s[e + 1] = blocks * 128;  // padded size, turned into offsets below
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    off_s[0] = 0;
    for (int e = 0; e < experts; ++e) off_s[e + 1] += off_s[e];
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = off_s[e];
  for (int t = threadIdx.x; t < num_tiles; t += blockDim.x) {
    const int row = t * 128;
    int lo = 0, hi = experts;  // first expert whose end is beyond `row`
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (off_s[mid + 1] > row) hi = mid;
      else lo = mid + 1;
    }
    tile_group[t] = lo < experts ? lo : unused_group;
  }
}

__global__ void moe_plan_place_kernel(const int* __restrict__ idx, int assignments, int k, int experts,
                                      const int* __restrict__ chunk_prefix, const int* __restrict__ offsets,
                                      int* __restrict__ slot, int* __restrict__ src_row) {
  __shared__ int e_s[kPlanChunk];
  const int a = blockIdx.x * kPlanChunk + threadIdx.x;
  const int e = a < assignments ? idx[a] : -1;
  e_s[threadIdx.x] = e;
  __syncthreads();
  if (a >= assignments) return;
  int rank = 0;
  for (int j = 0; j < threadIdx.x; ++j) rank += (e_s[j] == e) ? 1 : 0;
  const int s = offsets[e] + chunk_prefix[blockIdx.x * experts + e] + rank;
  slot[a] = s;
  src_row[s] = a / k;
}

PeerBases make_bases(void* const* p, int world) {
  PeerBases b;
  for (int r = 0; r < 8; ++r) b.p[r] = r < world ? p[r] : nullptr;
  return b;
}

}  // namespace

void moe_build_plan(const int* idx, int assignments, int k, int experts, int num_slots, int unused_group, int* chunk_hist,
                    int* offsets, int* counts, int* tile_group, int* slot, int* src_row, cudaStream_t stream) {
  if (assignments <= 0) return;
  const int chunks = (assignments + kPlanChunk - 1) / kPlanChunk;
  moe_plan_count_kernel<<<chunks, kPlanChunk, experts * sizeof(int), stream>>>(idx, assignments, experts, chunk_hist);
  moe_plan_scan_kernel<<<1, 512, (experts + 1) * sizeof(int), stream>>>(chunk_hist, chunks, experts, num_slots / 128,
                                                                       unused_group, offsets, counts, tile_group);
  moe_plan_place_kernel<<<chunks, kPlanChunk, 0, stream>>>(idx, assignments, k, experts, chunk_hist, offsets, slot, src_row);
}

void moe_scatter_rows_peer(const __nv_bfloat16* src, long long ld_src, const int* token, const int* dest_rank,
                           const int* dest_slot, const float* scale, void* const* dst, int world, long long ld_dst,
                           int assignments, int hidden, cudaStream_t stream) {
  if (assignments <= 0) return;
  moe_scatter_rows_peer_kernel<<<assignments, 128, 0, stream>>>(src, ld_src, token, dest_rank, dest_slot, scale,
                                                                make_bases(dst, world), ld_dst, assignments, hidden / 8);
}

void moe_combine_peer(void* const* src, int world, long long ld_src, const int* rank, const int* slot, const float* weight,
                      int k, __nv_bfloat16* out, long long ld_out, int tokens, int hidden, cudaStream_t stream) {
  if (tokens <= 0) return;
  moe_combine_peer_kernel<<<tokens, 128, 0, stream>>>(make_bases(src, world), ld_src, rank, slot, weight, k, out, ld_out,
                                                      tokens, hidden / 8);
}

void moe_topk(const float* logits, int tokens, int experts, int k, int* idx, float* weight, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int threads = 128;
  moe_topk_kernel<<<(tokens * 32 + threads - 1) / threads, threads, 0, stream>>>(logits, tokens, experts, k, idx, weight);
}

void moe_topk_backward(const int* idx, const float* weight, const float* dweight, int tokens, int experts, int k,
                       float* dlogits, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int threads = 128;
  moe_topk_bwd_kernel<<<(tokens * 32 + threads - 1) / threads, threads, 0, stream>>>(idx, weight, dweight, tokens, experts,
                                                                                  k, dlogits);
}

void moe_gather_rows(const __nv_bfloat16* src, long long ld_src, const int* src_row, const float* scale,
                     __nv_bfloat16* dst, long long ld_dst, int slots, int hidden, cudaStream_t stream, long long src_rows,
                     uint32_t* err) {
  if (slots <= 0) return;
  moe_gather_rows_kernel<<<slots, 128, 0, stream>>>(src, ld_src, src_row, scale, dst, ld_dst, slots, hidden / 8, src_rows,
                                                    err);
}

void moe_combine(const __nv_bfloat16* src, long long ld_src, const int* slot, const float* weight, int k,
                 __nv_bfloat16* out, long long ld_out, int tokens, int hidden, cudaStream_t stream, long long src_rows,
                 uint32_t* err) {
  if (tokens <= 0) return;
  moe_combine_kernel<<<tokens, 128, 0, stream>>>(src, ld_src, slot, weight, k, out, ld_out, tokens, hidden / 8, src_rows,
                                                 err);
}

void moe_rowdot(const __nv_bfloat16* a, long long ld_a, const __nv_bfloat16* b, long long ld_b, const int* slot, int k,
                int tokens, int hidden, float* out, cudaStream_t stream) {
  if (tokens <= 0) return;
  const int threads = 128;
  const long long warps = static_cast<long long>(tokens) * k;
  moe_rowdot_kernel<<<static_cast<unsigned int>((warps * 32 + threads - 1) / threads), threads, 0, stream>>>(
      a, ld_a, b, ld_b, slot, k, tokens, hidden / 8, out);
}

}  // namespace rlk
