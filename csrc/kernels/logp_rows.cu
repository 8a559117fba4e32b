// Selected-token log-prob over materialised logits: out[row] = z[row, t] - logsumexp(z[row, :]).
//
// One CTA streams one (active) row exactly once with 16-byte loads, each thread keeping an online
// (max, sum-exp) pair in the log2 domain; pairs are merged by a fixed shuffle tree and a fixed
// warp order, so results are bitwise reproducible and do not depend on the batch.  Replaces the
// reference's two-pass and online SIMT kernels and its experimental TMA variant
// (csrc/fused_logp_kernel.cu:111-206, csrc/cuda/fused_logp_sm90.cu:11-108) with one kernel; the
// nine-method Python contract (dense / indexed, typed / fp32 output) maps onto `row_indices` and
// the two dtype switches below.  An out-of-range target id yields 0 like the reference
// (csrc/fused_logp_kernel.cu:149-154).
#include "../common/ptx.cuh"
#include "kernels.h"

#include <cuda_fp16.h>

namespace rlk {

namespace {

constexpr int kThreads = 256;

struct MS {
  float m2, s;
};
__device__ __forceinline__ MS ms_merge(MS a, MS b) {
  const float m = fmaxf(a.m2, b.m2);
  if (m == -INFINITY) return MS{m, 0.f};
  return MS{m, a.s * fast_exp2(a.m2 - m) + b.s * fast_exp2(b.m2 - m)};
}
__device__ __forceinline__ void ms_push(MS& a, float z) {
  const float y = z * kLog2e;
  if (y <= a.m2) {
    a.s += fast_exp2(y - a.m2);
  } else {
    a.s = a.s * fast_exp2(a.m2 - y) + 1.f;
    a.m2 = y;
  }
}

template <typename T>
__device__ __forceinline__ float to_f(T x);
template <>
__device__ __forceinline__ float to_f<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }

template <typename T>
__device__ __forceinline__ T from_f(float x);
template <>
__device__ __forceinline__ float from_f<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

__device__ __forceinline__ void store_out(void* out, long long i, int out_dtype, float v) {
  if (out_dtype == 0) static_cast<float*>(out)[i] = v;
  else if (out_dtype == 1) static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
  else static_cast<__half*>(out)[i] = __float2half_rn(v);
}

// Block-wide fixed-order merge of per-thread (m2, s); result valid in every thread.
__device__ __forceinline__ MS block_merge(MS v, MS* smem) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    MS o;
    o.m2 = __shfl_xor_sync(0xffffffffu, v.m2, off);
    o.s = __shfl_xor_sync(0xffffffffu, v.s, off);
    v = ms_merge(v, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  MS r = smem[0];
  for (int w = 1; w < kThreads / 32; ++w) r = ms_merge(r, smem[w]);
  __syncthreads();
  return r;
}

// One 16-byte vector into the running (max, sum): the vector's maximum is found first, so the running sum is rescaled
// at most once per vector (rarely, after the first few vectors) and every element costs one fused multiply-add and one
// exp2 -- no compare / select / branch per element, which is what limited this kernel before the tensor of exps did.
template <int N>
__device__ __forceinline__ void ms_push_vec(MS& a, const float (&z)[N]) {
  float top = z[0];
#pragma unroll
  for (int j = 1; j < N; ++j) top = fmaxf(top, z[j]);
  const float y = top * kLog2e;
  if (y > a.m2) {
    a.s *= fast_exp2(a.m2 - y);  // exp2(-inf) = 0 on the first vector
    a.m2 = y;
  }
  if (a.m2 == -INFINITY) return;  // nothing but -inf so far: the sum stays 0
  const float neg_m = -a.m2;
  float part = 0.f;
#pragma unroll
  for (int j = 0; j < N; ++j) part += fast_exp2(fmaf(z[j], kLog2e, neg_m));
  a.s += part;
}

template <typename T>
__device__ __forceinline__ MS stream_row(const T* __restrict__ row, int V) {
  constexpr int kVec = 16 / sizeof(T);
  MS acc{-INFINITY, 0.f};
  // peel until 16-byte aligned
  int head = static_cast<int>(((16 - (reinterpret_cast<uintptr_t>(row) & 15u)) & 15u) / sizeof(T));
  if (head > V) head = V;
  for (int i = threadIdx.x; i < head; i += kThreads) ms_push(acc, to_f(row[i]));
  const int body = (V - head) / kVec;
  const uint4* p = reinterpret_cast<const uint4*>(row + head);
  int i = threadIdx.x;
  // two vectors per iteration: both loads are issued before either is consumed
  for (; i + kThreads < body; i += 2 * kThreads) {
    const uint4 q0 = __ldcs(p + i), q1 = __ldcs(p + i + kThreads);
    const T* e0 = reinterpret_cast<const T*>(&q0);
    const T* e1 = reinterpret_cast<const T*>(&q1);
    float z0[kVec], z1[kVec];
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      z0[j] = to_f(e0[j]);
      z1[j] = to_f(e1[j]);
    }
    ms_push_vec(acc, z0);
    ms_push_vec(acc, z1);
  }
  for (; i < body; i += kThreads) {
    const uint4 q = __ldcs(p + i);
    const T* e = reinterpret_cast<const T*>(&q);
    float z[kVec];
#pragma unroll
    for (int j = 0; j < kVec; ++j) z[j] = to_f(e[j]);
    ms_push_vec(acc, z);
  }
  for (int t = head + body * kVec + threadIdx.x; t < V; t += kThreads) ms_push(acc, to_f(row[t]));
  return acc;
}

// Two rows of the same length streamed side by side (policy and reference logits): both rows' loads are in flight
// together and each element is visited once.  Falls back to two separate sweeps if the rows are not both 16-byte aligned.
template <typename T>
__device__ __forceinline__ void stream_two_rows(const T* __restrict__ a, const T* __restrict__ b, int V, MS& acc_a,
                                                MS& acc_b) {
  constexpr int kVec = 16 / sizeof(T);
  if (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15u) != 0) {
    acc_a = stream_row(a, V);
    acc_b = stream_row(b, V);
    return;
  }
  acc_a = MS{-INFINITY, 0.f};
  acc_b = MS{-INFINITY, 0.f};
  const int body = V / kVec;
  const uint4* pa = reinterpret_cast<const uint4*>(a);
  const uint4* pb = reinterpret_cast<const uint4*>(b);
  for (int i = threadIdx.x; i < body; i += kThreads) {
    const uint4 qa = __ldcs(pa + i), qb = __ldcs(pb + i);
    const T* ea = reinterpret_cast<const T*>(&qa);
    const T* eb = reinterpret_cast<const T*>(&qb);
    float za[kVec], zb[kVec];
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      za[j] = to_f(ea[j]);
      zb[j] = to_f(eb[j]);
    }
    ms_push_vec(acc_a, za);
    ms_push_vec(acc_b, zb);
  }
  for (int t = body * kVec + threadIdx.x; t < V; t += kThreads) {
    ms_push(acc_a, to_f(a[t]));
    ms_push(acc_b, to_f(b[t]));
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) logp_rows_kernel(const T* __restrict__ logits, long long ld,
                                                             const long long* __restrict__ ids,
                                                             const long long* __restrict__ row_indices, int V,
                                                             void* __restrict__ out, int out_dtype, float inv_temp,
                                                             long long total_rows RLK_DBG_PARAM) {
  __shared__ MS red[kThreads / 32];
  const long long row = row_indices ? row_indices[blockIdx.x] : static_cast<long long>(blockIdx.x);
  // a gathered row index outside the logits (debug-bounds builds report it and skip the row)
  if (total_rows > 0 && !RLK_INDEX_OK(row, total_rows, RLK_DBG_ERR, 630u, 1)) return;
  const T* src = logits + row * ld;
  MS acc = stream_row(src, V);
  acc = block_merge(acc, red);
  if (threadIdx.x == 0) {
    const long long t = ids[row];
    float r = 0.f;
    if (t >= 0 && t < V) {
      const float lse = (acc.m2 + log2f(acc.s)) * kLn2;
      r = to_f(src[t]) - lse;
    }
    (void)inv_temp;
    store_out(out, row, out_dtype, r);
  }
}

}  // namespace

void logp_rows(const LogpRowsArgs& a, cudaStream_t stream) {
  if (a.launch_rows <= 0) return;
  const dim3 grid(a.launch_rows);
  switch (a.in_dtype) {
    case 0:
      logp_rows_kernel<float><<<grid, kThreads, 0, stream>>>(static_cast<const float*>(a.logits), a.ld, a.ids,
                                                             a.row_indices, a.V, a.out, a.out_dtype, 1.f,
                                                             a.total_rows RLK_DBG_ARG);
      break;
    case 1:
      logp_rows_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(a.logits), a.ld,
                                                                     a.ids, a.row_indices, a.V, a.out, a.out_dtype,
                                                                     1.f, a.total_rows RLK_DBG_ARG);
      break;
    default:
      logp_rows_kernel<__half><<<grid, kThreads, 0, stream>>>(static_cast<const __half*>(a.logits), a.ld, a.ids,
                                                              a.row_indices, a.V, a.out, a.out_dtype, 1.f,
                                                              a.total_rows RLK_DBG_ARG);
      break;
  }
}

// ---------------------------------------------------------------------------------------------
// ratio / KL front end over logits (policy and reference rows streamed once, side by side).
//   d = logp_ref - logp_pi ; ratio = exp(logp_pi - old) ; kl = exp(d) - d - 1
// Inactive rows: ratio 1, kl 0.  Saves logp_pi and lse_pi for the backward.
// Reference: Triton kernels rl_engine/kernels/ops/triton/loss/ratio_kl.py:21-122.
// ---------------------------------------------------------------------------------------------
namespace {

template <typename T>
__global__ void __launch_bounds__(kThreads) ratio_kl_fwd_kernel(const T* __restrict__ pol, const T* __restrict__ ref,
                                                                long long ld_p, long long ld_r,
                                                                const long long* __restrict__ ids,
                                                                const unsigned char* __restrict__ mask,
                                                                const float* __restrict__ old_logp, int V,
                                                                float* __restrict__ ratio, float* __restrict__ kl,
                                                                float* __restrict__ save_d, float* __restrict__ save_lse,
                                                                float* __restrict__ save_lp,
                                                                unsigned int* __restrict__ bad_id_flag) {
  __shared__ MS red[kThreads / 32];
  const long long row = blockIdx.x;
  if (!mask[row]) {
    if (threadIdx.x == 0) {
      ratio[row] = 1.f;
      kl[row] = 0.f;
      save_d[row] = 0.f;
      save_lse[row] = 0.f;
      save_lp[row] = 0.f;
    }
    return;
  }
  const T* prow = pol + row * ld_p;
  const T* rrow = ref ? ref + row * ld_r : nullptr;  // null: reference == policy (d = 0, kl = 0)
  MS a, b;
  if (rrow) {
    stream_two_rows(prow, rrow, V, a, b);
    a = block_merge(a, red);
    b = block_merge(b, red);
  } else {
    a = block_merge(stream_row(prow, V), red);
    b = a;
  }
  if (threadIdx.x == 0) {
    long long t = ids[row];
    if (t < 0 || t >= V) {
      atomicOr(bad_id_flag, 1u);
      t = 0;
    }
    const float lse_p = (a.m2 + log2f(a.s)) * kLn2;
    const float lse_r = (b.m2 + log2f(b.s)) * kLn2;
    const float lp = to_f(prow[t]) - lse_p;
    const float lr = rrow ? to_f(rrow[t]) - lse_r : lp;
    const float d = lr - lp;
    ratio[row] = expf(lp - old_logp[row]);
    kl[row] = expf(d) - d - 1.f;
    save_d[row] = d;
    save_lse[row] = lse_p;
    save_lp[row] = lp;
  }
}

// dlogits[row, j] = coef * (onehot_j - softmax_j), coef = g_ratio * ratio + g_kl * (1 - exp(d))
template <typename T>
__global__ void __launch_bounds__(kThreads) ratio_kl_bwd_kernel(const T* __restrict__ pol, long long ld_p,
                                                                const long long* __restrict__ ids,
                                                                const unsigned char* __restrict__ mask,
                                                                const float* __restrict__ g_ratio,
                                                                const float* __restrict__ g_kl,
                                                                const float* __restrict__ ratio,
                                                                const float* __restrict__ save_d,
                                                                const float* __restrict__ save_lse, int V,
                                                                T* __restrict__ grad, long long ld_g) {
  const long long row = blockIdx.x;
  T* grow = grad + row * ld_g;
  if (!mask[row]) {
    for (int i = threadIdx.x; i < V; i += kThreads) grow[i] = from_f<T>(0.f);
    return;
  }
  const float coef = g_ratio[row] * ratio[row] + g_kl[row] * (1.f - expf(save_d[row]));
  const float lse2 = save_lse[row] * kLog2e;
  long long t = ids[row];
  if (t < 0 || t >= V) t = 0;
  const T* prow = pol + row * ld_p;
  for (int i = threadIdx.x; i < V; i += kThreads) {
    const float p = fast_exp2(fmaf(to_f(prow[i]), kLog2e, -lse2));
    float g = -coef * p;
    if (i == t) g += coef;
    grow[i] = from_f<T>(g);
  }
}

}  // namespace

void ratio_kl_forward(const RatioKlFwdArgs& a, cudaStream_t stream) {
  if (a.rows <= 0) return;
#define RLK_LAUNCH(T)                                                                                          \
  ratio_kl_fwd_kernel<T><<<a.rows, kThreads, 0, stream>>>(static_cast<const T*>(a.policy), static_cast<const T*>(a.ref), \
                                                          a.ld_policy, a.ld_ref, a.ids, a.mask, a.old_logp, a.V,      \
                                                          a.ratio, a.kl, a.save_d, a.save_lse, a.save_lp, a.bad_id_flag)
  if (a.dtype == 0) RLK_LAUNCH(float);
  else if (a.dtype == 1) RLK_LAUNCH(__nv_bfloat16);
  else RLK_LAUNCH(__half);
#undef RLK_LAUNCH
}

void ratio_kl_backward(const RatioKlBwdArgs& a, cudaStream_t stream) {
  if (a.rows <= 0) return;
#define RLK_LAUNCH(T)                                                                                         \
  ratio_kl_bwd_kernel<T><<<a.rows, kThreads, 0, stream>>>(static_cast<const T*>(a.policy), a.ld_policy, a.ids, a.mask, \
                                                          a.g_ratio, a.g_kl, a.ratio, a.save_d, a.save_lse, a.V,     \
                                                          static_cast<T*>(a.grad), a.ld_grad)
  if (a.dtype == 0) RLK_LAUNCH(float);
  else if (a.dtype == 1) RLK_LAUNCH(__nv_bfloat16);
  else RLK_LAUNCH(__half);
#undef RLK_LAUNCH
}

}  // namespace rlk
