// Log-prob-space RL losses: group-normalised advantages, clipped-surrogate + k3-KL (GRPO / PPO),
// and DPO.  All reductions are two-level with a fixed block count and a fixed summation order, so
// the scalars are bitwise reproducible for a given shape.
//
// Reference: group normalisation is a Triton kernel (rl_engine/kernels/ops/triton/loss/
// grpo_loss.py:30-55); the surrogate / masked means are ~10 torch ops (same file :185-214); PPO and
// DPO tails do not exist there.
#include "../common/ptx.cuh"
#include "kernels.h"

namespace rlk {

namespace {

// ------------------------------------------------------------------------- group advantages
// One warp per group (CSR bounds).  Population variance, clamped at eps^2 before the sqrt.
__global__ void group_adv_kernel(const float* __restrict__ rewards, const long long* __restrict__ bounds,
                                 int num_groups, long long uniform, float eps, float* __restrict__ adv,
                                 long long n_rewards RLK_DBG_PARAM) {
  const int g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (g >= num_groups) return;
  const long long b0 = bounds ? bounds[g] : g * uniform;
  const long long b1 = bounds ? bounds[g + 1] : (g + 1) * uniform;
  // CSR group bounds come from the caller: [b0, b1) must lie inside the reward vector
  if (!RLK_INDEX_OK(b0, n_rewards + 1, RLK_DBG_ERR, 640u, 1) || !RLK_INDEX_OK(b1, n_rewards + 1, RLK_DBG_ERR, 640u, 2) ||
      !RLK_INDEX_OK(b1 - b0, n_rewards + 1, RLK_DBG_ERR, 640u, 3))
    return;
  float s = 0.f, q = 0.f;
  for (long long i = b0 + lane; i < b1; i += 32) {
    const float r = rewards[i];
    s += r;
    q = fmaf(r, r, q);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, off);
    q += __shfl_xor_sync(0xffffffffu, q, off);
  }
  const float n = static_cast<float>(b1 - b0);
  const float mean = s / n;
  const float var = fmaxf(q / n - mean * mean, eps * eps);
  const float inv = 1.f / sqrtf(var);
  for (long long i = b0 + lane; i < b1; i += 32) adv[i] = (rewards[i] - mean) * inv;
}

// ------------------------------------------------------------------- clipped surrogate + KL
constexpr int kLossThreads = 256;
constexpr int kLossBlocks = 256;  // fixed: the reduction tree does not depend on the input size

__device__ __forceinline__ float3 block_sum3(float3 v, float3* smem) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, off);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, off);
    v.z += __shfl_xor_sync(0xffffffffu, v.z, off);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float3 r = smem[0];
  for (int w = 1; w < kLossThreads / 32; ++w) {
    r.x += smem[w].x;
    r.y += smem[w].y;
    r.z += smem[w].z;
  }
  __syncthreads();
  return r;
}

// Per token i (row b = i / T): adv = adv_tok ? adv_tok[i] : adv_seq[b].
// Writes per-token unit gradients d(pl_i)/d(logp_i) and d(kl_i)/d(logp_i), and block partials.
__global__ void __launch_bounds__(kLossThreads)
surrogate_fwd_kernel(const float* __restrict__ logp, const float* __restrict__ ref_logp,
                     const float* __restrict__ old_logp, const float* __restrict__ adv_seq,
                     const float* __restrict__ adv_tok, const unsigned char* __restrict__ mask, long long n,
                     long long T, float clip_lo, float clip_hi, float* __restrict__ d_pl, float* __restrict__ d_kl,
                     float* __restrict__ ratio_out, float* __restrict__ kl_out, float3* __restrict__ partials) {
  __shared__ float3 red[kLossThreads / 32];
  const long long per_block = (n + kLossBlocks - 1) / kLossBlocks;
  const long long begin = blockIdx.x * per_block;
  const long long end = begin + per_block < n ? begin + per_block : n;
  float3 acc = make_float3(0.f, 0.f, 0.f);
  for (long long i = begin + threadIdx.x; i < end; i += kLossThreads) {
    float dpl = 0.f, dkl = 0.f, ratio = 1.f, kl = 0.f;
    if (mask[i]) {
      const float lp = logp[i];
      const float a = adv_tok ? adv_tok[i] : adv_seq[i / T];
      ratio = expf(lp - old_logp[i]);
      const float unclipped = ratio * a;
      const float clipped = fminf(fmaxf(ratio, clip_lo), clip_hi) * a;
      const float pl = -fminf(unclipped, clipped);
      dpl = (unclipped <= clipped) ? -unclipped : 0.f;
      float e = 1.f, d = 0.f;
      if (ref_logp) {
        d = ref_logp[i] - lp;
        e = expf(d);
      }
      kl = e - d - 1.f;
      dkl = 1.f - e;
      acc.x += pl;
      acc.y += kl;
      acc.z += 1.f;
    }
    d_pl[i] = dpl;
    d_kl[i] = dkl;
    if (ratio_out) ratio_out[i] = ratio;
    if (kl_out) kl_out[i] = kl;
  }
  acc = block_sum3(acc, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = acc;
}

// out = {loss, policy_loss, kl, count}
__global__ void surrogate_finish_kernel(const float3* __restrict__ partials, float beta, float* __restrict__ out) {
  if (threadIdx.x != 0) return;
  float pl = 0.f, kl = 0.f, cnt = 0.f;
  for (int b = 0; b < kLossBlocks; ++b) {
    pl += partials[b].x;
    kl += partials[b].y;
    cnt += partials[b].z;
  }
  const float denom = fmaxf(cnt, 1e-8f);
  const float policy_loss = pl / denom;
  const float klm = kl / denom;
  out[0] = policy_loss + beta * klm;
  out[1] = policy_loss;
  out[2] = klm;
  out[3] = cnt;
}

// grad_logp[i] = ((g_loss + g_pl) * d_pl[i] + (g_loss * beta + g_kl) * d_kl[i]) / count
__global__ void surrogate_bwd_kernel(const float* __restrict__ d_pl, const float* __restrict__ d_kl,
                                     const float* __restrict__ stats, const float* __restrict__ g3, float beta,
                                     long long n, float* __restrict__ grad_logp) {
  const float inv = 1.f / fmaxf(stats[3], 1e-8f);
  const float c_pl = (g3[0] + g3[1]) * inv;
  const float c_kl = (g3[0] * beta + g3[2]) * inv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    grad_logp[i] = c_pl * d_pl[i] + c_kl * d_kl[i];
  }
}

// ------------------------------------------------------------------------------------- DPO
// h = beta * ((pc - pr) - (rc - rr)); loss_i = -(1-ls) logsig(h) - ls logsig(-h); mean over pairs.
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__global__ void dpo_kernel(const float* __restrict__ pc, const float* __restrict__ pr, const float* __restrict__ rc,
                           const float* __restrict__ rr, int n, float beta, float ls, float* __restrict__ out_loss,
                           float* __restrict__ chosen_reward, float* __restrict__ rejected_reward,
                           float* __restrict__ dh) {
  // single block: n (pairs) is small; fixed-order strided sum then fixed tree
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float h = beta * ((pc[i] - pr[i]) - (rc[i] - rr[i]));
    acc += -(1.f - ls) * log_sigmoid(h) - ls * log_sigmoid(-h);
    const float sig = 1.f / (1.f + expf(-h));
    // d loss_i / d h = -(1-ls) (1 - sig) + ls * sig
    dh[i] = (-(1.f - ls) * (1.f - sig) + ls * sig) * beta / static_cast<float>(n);
    chosen_reward[i] = beta * (pc[i] - rc[i]);
    rejected_reward[i] = beta * (pr[i] - rr[i]);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t += red[w];
    out_loss[0] = t / static_cast<float>(n);
  }
}

}  // namespace

void group_advantages(const float* rewards, const long long* bounds, int num_groups, long long uniform, float eps,
                      float* adv, long long n_rewards, cudaStream_t stream) {
  if (num_groups <= 0) return;
  const int threads = 128;
  const int blocks = (num_groups * 32 + threads - 1) / threads;
  group_adv_kernel<<<blocks, threads, 0, stream>>>(rewards, bounds, num_groups, uniform, eps, adv,
                                                   n_rewards RLK_DBG_ARG);
}

int surrogate_partial_floats() { return kLossBlocks * 3; }

void surrogate_forward(const SurrogateFwdArgs& a, cudaStream_t stream) {
  surrogate_fwd_kernel<<<kLossBlocks, kLossThreads, 0, stream>>>(
      a.logp, a.ref_logp, a.old_logp, a.adv_seq, a.adv_tok, a.mask, a.n, a.T, 1.f - a.clip_eps, 1.f + a.clip_eps,
      a.d_pl, a.d_kl, a.ratio_out, a.kl_out, reinterpret_cast<float3*>(a.partials));
  surrogate_finish_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const float3*>(a.partials), a.beta, a.out4);
}

void surrogate_backward(const float* d_pl, const float* d_kl, const float* stats, const float* g3, float beta,
                        long long n, float* grad_logp, cudaStream_t stream) {
  if (n <= 0) return;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 1184) blocks = 1184;
  surrogate_bwd_kernel<<<static_cast<int>(blocks), threads, 0, stream>>>(d_pl, d_kl, stats, g3, beta, n, grad_logp);
}

void dpo_forward(const float* pc, const float* pr, const float* rc, const float* rr, int n, float beta, float ls,
                 float* out_loss, float* chosen_reward, float* rejected_reward, float* dh, cudaStream_t stream) {
  if (n <= 0) return;
  dpo_kernel<<<1, 256, 0, stream>>>(pc, pr, rc, rr, n, beta, ls, out_loss, chosen_reward, rejected_reward, dh);
}

}  // namespace rlk
