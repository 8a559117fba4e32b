// Memory-bound transformer ops for sm_100a: RMSNorm, SiLU / SwiGLU, RoPE, embedding, fused AdamW.
// All use 16-byte accesses, fp32 math, and fixed-order reductions (bitwise reproducible and
// independent of the batch: a row's result depends only on that row).
//
// The reference has only PyTorch definitions of these (rl_engine/kernels/ops/pytorch/norm/
// rms_norm.py:52-70, activation/swiglu.py:38-86, linear/embedding.py:35-51) and no RoPE or optimiser.
#include "../common/ptx.cuh"
#include "kernels.h"

#include <cuda_fp16.h>

namespace rlk {

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float ldf<__half>(const __half* p, long long i) { return __half2float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void stf<__half>(__half* p, long long i, float v) { p[i] = __float2half_rn(v); }

// Vector of 16 bytes of T
template <typename T> struct Vec16 {
  static constexpr int kN = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ float get(int j) const { return ldf(reinterpret_cast<const T*>(&raw), j); }
  __device__ __forceinline__ void set(int j, float v) { stf(reinterpret_cast<T*>(&raw), j, v); }
};

constexpr int kNormThreads = 128;

__device__ __forceinline__ float block_sum_128(float v, float* smem) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
  __syncthreads();
  const float r = (smem[0] + smem[1]) + (smem[2] + smem[3]);
  __syncthreads();
  return r;
}

// ---------------------------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w ; out dtype TO (x.dtype or fp32); optionally saves rstd.
template <typename T, typename TW, typename TO>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const T* __restrict__ x, long long ldx, const TW* __restrict__ w, TO* __restrict__ y, long long ldy,
                   int D, float eps, float* __restrict__ rstd_out) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  const T* xr = x + row * ldx;
  TO* yr = y + row * ldy;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += kNormThreads) {
    const float v = ldf(xr, i);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum_128(ss, red);
  const float rstd = rsqrtf(ss / static_cast<float>(D) + eps);
  if (rstd_out && threadIdx.x == 0) rstd_out[row] = rstd;
  for (int i = threadIdx.x; i < D; i += kNormThreads) stf(yr, i, ldf(xr, i) * rstd * ldf(w, i));
}

// dx = rstd * (w*dy - x * rstd^2 * mean(w*dy*x)); per-row-chunk partial dw written to dw_part[chunk, D].
// Rows per CTA: kNormBwdRowsMax for long inputs (few, large partial-sum chunks), fewer for short ones so that the grid
// still covers the machine several times over (a CTA walks its rows one after the other).
constexpr int kNormBwdRowsMax = 64;
constexpr int kNormBwdRowsMin = 8;
template <typename T, typename TW>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const T* __restrict__ x, long long ldx, const TW* __restrict__ w, const T* __restrict__ dy,
                   long long lddy, const float* __restrict__ rstd, T* __restrict__ dx, long long lddx, int rows, int D,
                   float* __restrict__ dw_part, int rows_per_cta) {
  __shared__ float red[4];
  extern __shared__ float dw_acc[];  // [D]
  for (int i = threadIdx.x; i < D; i += kNormThreads) dw_acc[i] = 0.f;
  const long long r0 = static_cast<long long>(blockIdx.x) * rows_per_cta;
  const long long r1 = r0 + rows_per_cta < rows ? r0 + rows_per_cta : rows;
  for (long long row = r0; row < r1; ++row) {
    const T* xr = x + row * ldx;
    const T* gr = dy + row * lddy;
    T* dr = dx + row * lddx;
    const float rs = rstd[row];
    float dot = 0.f;
    for (int i = threadIdx.x; i < D; i += kNormThreads) dot = fmaf(ldf(gr, i) * ldf(w, i), ldf(xr, i), dot);
    dot = block_sum_128(dot, red);
    const float c = dot * rs * rs / static_cast<float>(D);
    for (int i = threadIdx.x; i < D; i += kNormThreads) {
      const float xv = ldf(xr, i), gv = ldf(gr, i);
      stf(dr, i, rs * (gv * ldf(w, i) - xv * c));
      dw_acc[i] = fmaf(gv, xv * rs, dw_acc[i]);  // each thread owns its columns: no race
    }
  }
  float* out = dw_part + static_cast<long long>(blockIdx.x) * D;
  for (int i = threadIdx.x; i < D; i += kNormThreads) out[i] = dw_acc[i];
}

// bf16 fast paths (x, w, y all bf16; D % 8 == 0; 16-byte aligned rows): 16-byte loads, row kept in
// registers between the two sweeps.  Same reduction order as the generic kernels? No: the per-thread
// partial sums cover different elements, so these are used consistently for every bf16 call instead.
constexpr int kNormVecMax = 4;  // up to 4 x 8 elements per thread -> D <= 4096 in registers
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_bf16_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
                        __nv_bfloat16* __restrict__ y, long long ldy, int D, float eps, float* __restrict__ rstd_out) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * ldy);
  const int n8 = D / 8;
  uint4 buf[kNormVecMax];
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < kNormVecMax; ++v) {
    const int i = threadIdx.x + v * kNormThreads;
    if (i < n8) {
      buf[v] = xr[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&buf[v]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
    }
  }
  ss = block_sum_128(ss, red);
  const float rstd = rsqrtf(ss / static_cast<float>(D) + eps);
  if (rstd_out && threadIdx.x == 0) rstd_out[row] = rstd;
#pragma unroll
  for (int v = 0; v < kNormVecMax; ++v) {
    const int i = threadIdx.x + v * kNormThreads;
    if (i < n8) {
      const uint4 wv = wr[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&buf[v]);
      const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]), g = __bfloat1622float2(wh[j]);
        oh[j] = __floats2bfloat162_rn(f.x * rstd * g.x, f.y * rstd * g.y);
      }
      yr[i] = o;
    }
  }
}

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_bf16_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
                        const __nv_bfloat16* __restrict__ dy, long long lddy, const float* __restrict__ rstd,
                        __nv_bfloat16* __restrict__ dx, long long lddx, int rows, int D, float* __restrict__ dw_part,
                        int rows_per_cta) {
  __shared__ float red[4];
  const int n8 = D / 8;
  float dwacc[kNormVecMax][8];
  float wreg[kNormVecMax][8];
#pragma unroll
  for (int v = 0; v < kNormVecMax; ++v) {
    const int i = threadIdx.x + v * kNormThreads;
    uint4 wv = make_uint4(0, 0, 0, 0);
    if (i < n8) wv = reinterpret_cast<const uint4*>(w)[i];
    const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(wh[j]);
      wreg[v][2 * j] = g.x;
      wreg[v][2 * j + 1] = g.y;
      dwacc[v][2 * j] = 0.f;
      dwacc[v][2 * j + 1] = 0.f;
    }
  }
  const long long r0 = static_cast<long long>(blockIdx.x) * rows_per_cta;
  const long long r1 = r0 + rows_per_cta < rows ? r0 + rows_per_cta : rows;
  for (long long row = r0; row < r1; ++row) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * lddy);
    uint4* dr = reinterpret_cast<uint4*>(dx + row * lddx);
    const float rs = rstd[row];
    float xf[kNormVecMax][8], gf[kNormVecMax][8];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < kNormVecMax; ++v) {
      const int i = threadIdx.x + v * kNormThreads;
      if (i < n8) {
        const uint4 xv = xr[i], gv = gr[i];
        const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = __bfloat1622float2(xh[j]), b = __bfloat1622float2(gh[j]);
          xf[v][2 * j] = a.x; xf[v][2 * j + 1] = a.y;
          gf[v][2 * j] = b.x; gf[v][2 * j + 1] = b.y;
          dot = fmaf(b.x * wreg[v][2 * j], a.x, dot);
          dot = fmaf(b.y * wreg[v][2 * j + 1], a.y, dot);
        }
      }
    }
    dot = block_sum_128(dot, red);
    const float c = dot * rs * rs / static_cast<float>(D);
#pragma unroll
    for (int v = 0; v < kNormVecMax; ++v) {
      const int i = threadIdx.x + v * kNormThreads;
      if (i < n8) {
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float d0 = rs * (gf[v][2 * j] * wreg[v][2 * j] - xf[v][2 * j] * c);
          const float d1 = rs * (gf[v][2 * j + 1] * wreg[v][2 * j + 1] - xf[v][2 * j + 1] * c);
          oh[j] = __floats2bfloat162_rn(d0, d1);
          dwacc[v][2 * j] = fmaf(gf[v][2 * j], xf[v][2 * j] * rs, dwacc[v][2 * j]);
          dwacc[v][2 * j + 1] = fmaf(gf[v][2 * j + 1], xf[v][2 * j + 1] * rs, dwacc[v][2 * j + 1]);
        }
        dr[i] = o;
      }
    }
  }
  float* out = dw_part + static_cast<long long>(blockIdx.x) * D;
#pragma unroll
  for (int v = 0; v < kNormVecMax; ++v) {
    const int i = threadIdx.x + v * kNormThreads;
    if (i < n8) {
      reinterpret_cast<float4*>(out + i * 8)[0] = make_float4(dwacc[v][0], dwacc[v][1], dwacc[v][2], dwacc[v][3]);
      reinterpret_cast<float4*>(out + i * 8)[1] = make_float4(dwacc[v][4], dwacc[v][5], dwacc[v][6], dwacc[v][7]);
    }
  }
}

inline bool bf16_vec_ok(const void* a, long long lda, int D) {
  return D % 8 == 0 && D <= 8 * kNormVecMax * kNormThreads && lda % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15u) == 0;
}

template <typename TW>
__global__ void colsum_kernel(const float* __restrict__ part, int chunks, int D, TW* __restrict__ dw) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= D) return;
  float s = 0.f;
  for (int c = 0; c < chunks; ++c) s += part[static_cast<long long>(c) * D + i];
  stf(dw, i, s);
}

// ------------------------------------------------------------------------------ SiLU / SwiGLU
template <typename T, typename TO>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gate, long long ldg, const T* __restrict__ up, long long ldu,
                                  TO* __restrict__ out, long long ldo, long long rows, int F) {
  const long long total = rows * F;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / F;
    const int c = static_cast<int>(idx - r * F);
    const float g = ldf(gate, r * ldg + c);
    const float s = g / (1.f + expf(-g));
    const float u = up ? ldf(up, r * ldu + c) : 1.f;
    stf(out, r * ldo + c, s * u);
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ gate, long long ldg, const T* __restrict__ up, long long ldu,
                                  const T* __restrict__ dy, long long lddy, T* __restrict__ dgate, long long lddg,
                                  T* __restrict__ dup, long long lddu, long long rows, int F) {
  const long long total = rows * F;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / F;
    const int c = static_cast<int>(idx - r * F);
    const float g = ldf(gate, r * ldg + c);
    const float sig = 1.f / (1.f + expf(-g));
    const float silu = g * sig;
    const float d = ldf(dy, r * lddy + c);
    const float u = up ? ldf(up, r * ldu + c) : 1.f;
    stf(dgate, r * lddg + c, d * u * sig * (1.f + g * (1.f - sig)));
    if (dup) stf(dup, r * lddu + c, d * silu);
  }
}

// Packed bf16 SwiGLU: gu = [gate | up] of width 2F per row (the output of one fused gate/up GEMM).
// 16-byte accesses; F % 8 == 0.  The backward writes d(gu) in place of two separate tensors, so no
// strided scatter / zero-fill is needed to rebuild the packed gradient.
__global__ void swiglu_packed_fwd_kernel(const __nv_bfloat16* __restrict__ gu, long long ldgu,
                                         __nv_bfloat16* __restrict__ out, long long ldo, long long rows, int F) {
  const int f8 = F / 8;
  const long long total = rows * f8;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / f8;
    const int c = static_cast<int>(idx - r * f8) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * ldgu + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * ldgu + F + c);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 gf = __bfloat1622float2(gp[i]), uf = __bfloat1622float2(up[i]);
      op[i] = __floats2bfloat162_rn(gf.x / (1.f + __expf(-gf.x)) * uf.x, gf.y / (1.f + __expf(-gf.y)) * uf.y);
    }
    *reinterpret_cast<uint4*>(out + r * ldo + c) = o;
  }
}

__global__ void swiglu_packed_bwd_kernel(const __nv_bfloat16* __restrict__ gu, long long ldgu,
                                         const __nv_bfloat16* __restrict__ dy, long long lddy,
                                         __nv_bfloat16* __restrict__ dgu, long long lddgu, long long rows, int F) {
  const int f8 = F / 8;
  const long long total = rows * f8;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / f8;
    const int c = static_cast<int>(idx - r * f8) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * ldgu + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * ldgu + F + c);
    const uint4 d = *reinterpret_cast<const uint4*>(dy + r * lddy + c);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    const __nv_bfloat162* dp = reinterpret_cast<const __nv_bfloat162*>(&d);
    uint4 og, ou;
    __nv_bfloat162* ogp = reinterpret_cast<__nv_bfloat162*>(&og);
    __nv_bfloat162* oup = reinterpret_cast<__nv_bfloat162*>(&ou);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 gf = __bfloat1622float2(gp[i]), uf = __bfloat1622float2(up[i]), df = __bfloat1622float2(dp[i]);
      const float s0 = 1.f / (1.f + __expf(-gf.x)), s1 = 1.f / (1.f + __expf(-gf.y));
      ogp[i] = __floats2bfloat162_rn(df.x * uf.x * s0 * (1.f + gf.x * (1.f - s0)), df.y * uf.y * s1 * (1.f + gf.y * (1.f - s1)));
      oup[i] = __floats2bfloat162_rn(df.x * gf.x * s0, df.y * gf.y * s1);
    }
    *reinterpret_cast<uint4*>(dgu + r * lddgu + c) = og;
    *reinterpret_cast<uint4*>(dgu + r * lddgu + F + c) = ou;
  }
}

// ------------------------------------------------------------------------------------- RoPE
// x: [tokens, heads, D] (token pitch ldt, head pitch D); cos/sin: [max_pos, D/2] fp32.
// out[.., j] = a cos - b sin ; out[.., j + D/2] = b cos + a sin ; sign = -1 gives the inverse (backward).
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, long long ldt, const long long* __restrict__ pos,
                            const float* __restrict__ cs, const float* __restrict__ sn, T* __restrict__ out,
                            long long ldo, long long tokens, int heads, int D, float sign,
                            long long table_rows RLK_DBG_PARAM) {
  const int half = D / 2;
  const long long total = tokens * heads * half;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(idx % half);
    const long long th = idx / half;
    const int h = static_cast<int>(th % heads);
    const long long t = th / heads;
    const long long p = pos[t];
    if (!RLK_INDEX_OK(p, table_rows, RLK_DBG_ERR, 610u, 1)) continue;  // position beyond the cos / sin table
    const float c = cs[p * half + j];
    const float s = sn[p * half + j] * sign;
    const long long base = t * ldt + static_cast<long long>(h) * D;
    const long long obase = t * ldo + static_cast<long long>(h) * D;
    const float a = ldf(x, base + j), b = ldf(x, base + j + half);
    stf(out, obase + j, a * c - b * s);
    stf(out, obase + j + half, b * c + a * s);
  }
}

// bf16 fast path: one thread rotates 8 element pairs (16-byte loads and stores, float4 cos / sin).
__global__ void rope_bf16_vec_kernel(const __nv_bfloat16* __restrict__ x, long long ldt, const long long* __restrict__ pos,
                                     const float* __restrict__ cs, const float* __restrict__ sn,
                                     __nv_bfloat16* __restrict__ out, long long ldo, long long tokens, int heads, int D,
                                     float sign, long long table_rows RLK_DBG_PARAM) {
  const int half = D / 2;
  const int vec_per_head = half / 8;  // threads per (token, head)
  const long long total = tokens * heads * vec_per_head;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(idx % vec_per_head);
    const long long th = idx / vec_per_head;
    const int h = static_cast<int>(th % heads);
    const long long t = th / heads;
    const long long p = pos[t];
    if (!RLK_INDEX_OK(p, table_rows, RLK_DBG_ERR, 611u, 1)) continue;  // position beyond the cos / sin table
    const float4* c4 = reinterpret_cast<const float4*>(cs + p * half + v * 8);
    const float4* s4 = reinterpret_cast<const float4*>(sn + p * half + v * 8);
    const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float s[8] = {s0.x * sign, s0.y * sign, s0.z * sign, s0.w * sign, s1.x * sign, s1.y * sign, s1.z * sign, s1.w * sign};
    const __nv_bfloat16* src = x + t * ldt + static_cast<long long>(h) * D + v * 8;
    __nv_bfloat16* dst = out + t * ldo + static_cast<long long>(h) * D + v * 8;
    const uint4 qa = *reinterpret_cast<const uint4*>(src);
    const uint4 qb = *reinterpret_cast<const uint4*>(src + half);
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&qa);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&qb);
    uint4 oa, ob;
    __nv_bfloat162* ra = reinterpret_cast<__nv_bfloat162*>(&oa);
    __nv_bfloat162* rb = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = __bfloat1622float2(pa[i]), b = __bfloat1622float2(pb[i]);
      ra[i] = __floats2bfloat162_rn(a.x * c[2 * i] - b.x * s[2 * i], a.y * c[2 * i + 1] - b.y * s[2 * i + 1]);
      rb[i] = __floats2bfloat162_rn(b.x * c[2 * i] + a.x * s[2 * i], b.y * c[2 * i + 1] + a.y * s[2 * i + 1]);
    }
    *reinterpret_cast<uint4*>(dst) = oa;
    *reinterpret_cast<uint4*>(dst + half) = ob;
  }
}

// -------------------------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const T* __restrict__ table, long long ldw,
                                     T* __restrict__ out, int D, long long vocab RLK_DBG_PARAM) {
  const long long row = blockIdx.x;
  long long id = ids[row];
  (void)RLK_INDEX_OK(id, vocab, RLK_DBG_ERR, 620u, 1);  // release builds read row 0 for an id outside the table
  if (id < 0 || id >= vocab) id = 0;
  const T* src = table + id * ldw;
  T* dst = out + row * static_cast<long long>(D);
  if ((D * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0 &&
      (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
    const int n = D * sizeof(T) / 16;
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = src[i];
  }
}

// Deterministic backward: tokens are pre-sorted by id (stable); CTA s sums the rows of segment s in
// that order and writes one table row.  No atomics.
template <typename T, typename TG>
__global__ void embedding_bwd_kernel(const long long* __restrict__ seg_ids, const long long* __restrict__ seg_start,
                                     const long long* __restrict__ order, const T* __restrict__ dy, int D,
                                     TG* __restrict__ dtable, long long ldw, long long dy_rows,
                                     long long table_rows RLK_DBG_PARAM) {
  const long long s = blockIdx.x;
  const long long b0 = seg_start[s], b1 = seg_start[s + 1];
  const long long id = seg_ids[s];
  if (!RLK_INDEX_OK(id, table_rows, RLK_DBG_ERR, 621u, 1)) return;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float acc = 0.f;
    for (long long k = b0; k < b1; ++k) {
      if (!RLK_INDEX_OK(order[k], dy_rows, RLK_DBG_ERR, 621u, 2)) continue;
      acc += ldf(dy, order[k] * static_cast<long long>(D) + i);
    }
    stf(dtable, id * ldw + i, acc);
  }
}

// ------------------------------------------------------------------------------ fused AdamW
// p (bf16 or fp32), optional fp32 master copy, g (bf16 or fp32), m / v fp32.  Decoupled weight decay.
template <typename TP, typename TG>
__global__ void adamw_kernel(TP* __restrict__ p, float* __restrict__ master, const TG* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v, long long n, float lr, float b1, float b2,
                             float eps, float wd, float bc1, float bc2, float grad_scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float gi = ldf(g, i) * grad_scale;
    float w = master ? master[i] : ldf(p, i);
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float denom = sqrtf(vi * (1.f / bc2)) + eps;
    w = w * (1.f - lr * wd) - lr * (mi * (1.f / bc1)) / denom;
    if (master) master[i] = w;
    stf(p, i, w);
  }
}

// The fp32 master weight of a bf16 parameter, stored as the parameter itself plus a 16-bit residual:
//   master_bits = (bf16_bits << 16) + sign_extend(residual).
// The parameter is the master rounded to bf16 (ties away from zero in magnitude, one integer add), so the residual
// always fits 16 bits and the pair reproduces every bit of the fp32 value: the optimiser has exact fp32-master
// arithmetic at 2 extra bytes per parameter instead of 4.
__device__ __forceinline__ float master_from_split(unsigned short hi, short residual) {
  return __uint_as_float((static_cast<unsigned int>(hi) << 16) + static_cast<unsigned int>(static_cast<int>(residual)));
}
__device__ __forceinline__ void master_to_split(float w, unsigned short& hi, short& residual) {
  const unsigned int bits = __float_as_uint(w);
  const unsigned int up = (bits + 0x8000u) >> 16;  // round half away from zero (in magnitude)
  hi = static_cast<unsigned short>(up);
  residual = static_cast<short>(static_cast<int>(bits - (up << 16)));
}

// Eight elements per thread and iteration through 16-byte accesses.  kMaster: 0 none (bf16 parameter is the state),
// 1 fp32 master, 2 bf16 parameter + 16-bit residual.  TG: gradient type (bf16 or fp32).
template <typename TG, int kMaster>
__global__ void __launch_bounds__(256)
adamw_bf16_vec_kernel(__nv_bfloat16* __restrict__ p, float* __restrict__ master, short* __restrict__ residual,
                      const TG* __restrict__ g, float* __restrict__ m, float* __restrict__ v, long long n8, float lr,
                      float b1, float b2, float eps, float wd, float bc1, float bc2, float grad_scale) {
  const float inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2, decay = 1.f - lr * wd;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * 8;
    float gj[8], w[8], mm[8], vv[8];
    if constexpr (sizeof(TG) == 4) {
      const float4 a = reinterpret_cast<const float4*>(g + e)[0], b = reinterpret_cast<const float4*>(g + e)[1];
      gj[0] = a.x; gj[1] = a.y; gj[2] = a.z; gj[3] = a.w; gj[4] = b.x; gj[5] = b.y; gj[6] = b.z; gj[7] = b.w;
    } else {
      const uint4 q = *reinterpret_cast<const uint4*>(g + e);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = __bfloat1622float2(h[j]);
        gj[2 * j] = x.x;
        gj[2 * j + 1] = x.y;
      }
    }
    uint4 pq = *reinterpret_cast<const uint4*>(p + e);
    unsigned short* ph = reinterpret_cast<unsigned short*>(&pq);
    uint4 rq = make_uint4(0, 0, 0, 0);
    short* rh = reinterpret_cast<short*>(&rq);
    if constexpr (kMaster == 1) {
      const float4 a = reinterpret_cast<const float4*>(master + e)[0], b = reinterpret_cast<const float4*>(master + e)[1];
      w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    } else if constexpr (kMaster == 2) {
      rq = *reinterpret_cast<const uint4*>(residual + e);
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = master_from_split(ph[j], rh[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = __uint_as_float(static_cast<unsigned int>(ph[j]) << 16);
    }
    {
      const float4 a = reinterpret_cast<const float4*>(m + e)[0], b = reinterpret_cast<const float4*>(m + e)[1];
      mm[0] = a.x; mm[1] = a.y; mm[2] = a.z; mm[3] = a.w; mm[4] = b.x; mm[5] = b.y; mm[6] = b.z; mm[7] = b.w;
      const float4 c = reinterpret_cast<const float4*>(v + e)[0], d = reinterpret_cast<const float4*>(v + e)[1];
      vv[0] = c.x; vv[1] = c.y; vv[2] = c.z; vv[3] = c.w; vv[4] = d.x; vv[5] = d.y; vv[6] = d.z; vv[7] = d.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gi = gj[j] * grad_scale;
      mm[j] = b1 * mm[j] + (1.f - b1) * gi;
      vv[j] = b2 * vv[j] + (1.f - b2) * gi * gi;
      const float denom = sqrtf(vv[j] * inv_bc2) + eps;
      w[j] = w[j] * decay - lr * (mm[j] * inv_bc1) / denom;
    }
    reinterpret_cast<float4*>(m + e)[0] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(m + e)[1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
    reinterpret_cast<float4*>(v + e)[0] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    reinterpret_cast<float4*>(v + e)[1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    if constexpr (kMaster == 1) {
      reinterpret_cast<float4*>(master + e)[0] = make_float4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<float4*>(master + e)[1] = make_float4(w[4], w[5], w[6], w[7]);
    }
    if constexpr (kMaster == 2) {
#pragma unroll
      for (int j = 0; j < 8; ++j) master_to_split(w[j], ph[j], rh[j]);
      *reinterpret_cast<uint4*>(residual + e) = rq;
      *reinterpret_cast<uint4*>(p + e) = pq;
    } else {
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pq);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(w[2 * j], w[2 * j + 1]);
      *reinterpret_cast<uint4*>(p + e) = pq;
    }
  }
}

// Scalar form of the residual representation (tails and unaligned buffers).
template <typename TG>
__global__ void adamw_residual_kernel(__nv_bfloat16* __restrict__ p, short* __restrict__ residual,
                                      const TG* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                                      long long n, float lr, float b1, float b2, float eps, float wd, float bc1,
                                      float bc2, float grad_scale) {
  unsigned short* pb = reinterpret_cast<unsigned short*>(p);
  const float inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2, decay = 1.f - lr * wd;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float gi = ldf(g, i) * grad_scale;
    float w = master_from_split(pb[i], residual[i]);
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    w = w * decay - lr * (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps);
    master_to_split(w, pb[i], residual[i]);
  }
}

// Merge of two partial attention results over disjoint key sets by their log-sum-exp, for decoding with packed
// queries: o1 / o2 are [n * rep rows, Hkv, 128] (row = sequence * rep + query head within its key / value group),
// l1 / l2 are [Hkv, n * rep]; out is [n, Hkv * rep * 128] in the model's head order (head = kv head * rep + j).
__global__ void attn_merge2_kernel(const __nv_bfloat16* __restrict__ o1, const float* __restrict__ l1,
                                   const __nv_bfloat16* __restrict__ o2, const float* __restrict__ l2,
                                   __nv_bfloat16* __restrict__ out, long long rows, int hkv, int rep) {
  const long long total = rows * hkv * 16;  // 16 vectors of 8 elements per (row, head)
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(idx & 15);
    const long long rh = idx >> 4;
    const int h = static_cast<int>(rh % hkv);
    const long long r = rh / hkv;
    const float a = l1[h * rows + r], b = l2[h * rows + r];
    const float top = fmaxf(a, b);
    float w1 = top == -INFINITY ? 0.f : __expf(a - top), w2 = top == -INFINITY ? 0.f : __expf(b - top);
    const float inv = (w1 + w2) > 0.f ? 1.f / (w1 + w2) : 0.f;
    w1 *= inv;
    w2 *= inv;
    const uint4 q1 = reinterpret_cast<const uint4*>(o1 + (r * hkv + h) * 128)[v];
    const uint4 q2 = reinterpret_cast<const uint4*>(o2 + (r * hkv + h) * 128)[v];
    const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&q1);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&q2);
    uint4 res;
    __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(p1[i]), y = __bfloat1622float2(p2[i]);
      pr[i] = __floats2bfloat162_rn(x.x * w1 + y.x * w2, x.y * w1 + y.y * w2);
    }
    const long long seq = r / rep;
    const int j = static_cast<int>(r - seq * rep);
    reinterpret_cast<uint4*>(out + (seq * hkv * rep + static_cast<long long>(h) * rep + j) * 128)[v] = res;
  }
}

inline int grid_for(long long total, int threads) {
  long long b = (total + threads - 1) / threads;
  const long long cap = 148LL * 16;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

#define RLK_DISPATCH_T(code, ...)                          \
  do {                                                     \
    if ((code) == 0) { using T = float; __VA_ARGS__; }      \
    else if ((code) == 1) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else { using T = __half; __VA_ARGS__; }                \
  } while (0)

void rmsnorm_forward(const void* x, long long ldx, int x_dtype, const void* w, int w_dtype, void* y, long long ldy,
                     bool out_fp32, long long rows, int D, float eps, float* rstd, cudaStream_t stream) {
  if (rows <= 0) return;
  if (x_dtype == 1 && w_dtype == 1 && !out_fp32 && bf16_vec_ok(x, ldx, D) && bf16_vec_ok(y, ldy, D) &&
      bf16_vec_ok(w, 8, D)) {
    rmsnorm_fwd_bf16_kernel<<<rows, kNormThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), ldx,
                                                               static_cast<const __nv_bfloat16*>(w),
                                                               static_cast<__nv_bfloat16*>(y), ldy, D, eps, rstd);
    return;
  }
  RLK_DISPATCH_T(x_dtype, {
    using TX = T;
    RLK_DISPATCH_T(w_dtype, {
      using TW = T;
      if (out_fp32)
        rmsnorm_fwd_kernel<TX, TW, float><<<rows, kNormThreads, 0, stream>>>(
            static_cast<const TX*>(x), ldx, static_cast<const TW*>(w), static_cast<float*>(y), ldy, D, eps, rstd);
      else
        rmsnorm_fwd_kernel<TX, TW, TX><<<rows, kNormThreads, 0, stream>>>(
            static_cast<const TX*>(x), ldx, static_cast<const TW*>(w), static_cast<TX*>(y), ldy, D, eps, rstd);
    });
  });
}

int rmsnorm_bwd_rows_per_cta(long long rows) {
  const long long target_ctas = 148LL * 8;
  long long r = (rows + target_ctas - 1) / target_ctas;
  if (r < kNormBwdRowsMin) r = kNormBwdRowsMin;
  if (r > kNormBwdRowsMax) r = kNormBwdRowsMax;
  return static_cast<int>(r);
}

int rmsnorm_bwd_chunks(long long rows, int rows_per_cta) {
  if (rows_per_cta <= 0) rows_per_cta = rmsnorm_bwd_rows_per_cta(rows);
  return static_cast<int>((rows + rows_per_cta - 1) / rows_per_cta);
}

void rmsnorm_backward(const void* x, long long ldx, int x_dtype, const void* w, int w_dtype, const void* dy,
                      long long lddy, const float* rstd, void* dx, long long lddx, long long rows, int D,
                      float* dw_part, void* dw, cudaStream_t stream, int rows_per_cta) {
  if (rows <= 0) return;
  if (rows_per_cta <= 0) rows_per_cta = rmsnorm_bwd_rows_per_cta(rows);
  const int chunks = rmsnorm_bwd_chunks(rows, rows_per_cta);
  if (x_dtype == 1 && w_dtype == 1 && bf16_vec_ok(x, ldx, D) && bf16_vec_ok(dy, lddy, D) && bf16_vec_ok(dx, lddx, D) &&
      bf16_vec_ok(w, 8, D)) {
    rmsnorm_bwd_bf16_kernel<<<chunks, kNormThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(w),
        static_cast<const __nv_bfloat16*>(dy), lddy, rstd, static_cast<__nv_bfloat16*>(dx), lddx,
        static_cast<int>(rows), D, dw_part, rows_per_cta);
    colsum_kernel<__nv_bfloat16><<<(D + 255) / 256, 256, 0, stream>>>(dw_part, chunks, D, static_cast<__nv_bfloat16*>(dw));
    return;
  }
  RLK_DISPATCH_T(x_dtype, {
    using TX = T;
    RLK_DISPATCH_T(w_dtype, {
      using TW = T;
      auto k = rmsnorm_bwd_kernel<TX, TW>;
      if (D * 4 > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, D * 4);
      k<<<chunks, kNormThreads, D * sizeof(float), stream>>>(static_cast<const TX*>(x), ldx, static_cast<const TW*>(w),
                                                            static_cast<const TX*>(dy), lddy, rstd,
                                                            static_cast<TX*>(dx), lddx, static_cast<int>(rows), D,
                                                            dw_part, rows_per_cta);
      colsum_kernel<TW><<<(D + 255) / 256, 256, 0, stream>>>(dw_part, chunks, D, static_cast<TW*>(dw));
    });
  });
}

void swiglu_forward(const void* gate, long long ldg, const void* up, long long ldu, int dtype, void* out, long long ldo,
                    bool out_fp32, long long rows, int F, cudaStream_t stream) {
  if (rows <= 0 || F <= 0) return;
  const int threads = 256;
  const int grid = grid_for(rows * F, threads);
  RLK_DISPATCH_T(dtype, {
    if (out_fp32)
      swiglu_fwd_kernel<T, float><<<grid, threads, 0, stream>>>(static_cast<const T*>(gate), ldg,
                                                                static_cast<const T*>(up), ldu,
                                                                static_cast<float*>(out), ldo, rows, F);
    else
      swiglu_fwd_kernel<T, T><<<grid, threads, 0, stream>>>(static_cast<const T*>(gate), ldg,
                                                            static_cast<const T*>(up), ldu, static_cast<T*>(out), ldo,
                                                            rows, F);
  });
}

void swiglu_backward(const void* gate, long long ldg, const void* up, long long ldu, const void* dy, long long lddy,
                     int dtype, void* dgate, long long lddg, void* dup, long long lddu, long long rows, int F,
                     cudaStream_t stream) {
  if (rows <= 0 || F <= 0) return;
  const int threads = 256;
  const int grid = grid_for(rows * F, threads);
  RLK_DISPATCH_T(dtype, {
    swiglu_bwd_kernel<T><<<grid, threads, 0, stream>>>(static_cast<const T*>(gate), ldg, static_cast<const T*>(up), ldu,
                                                       static_cast<const T*>(dy), lddy, static_cast<T*>(dgate), lddg,
                                                       static_cast<T*>(dup), lddu, rows, F);
  });
}

void swiglu_packed_forward(const __nv_bfloat16* gu, long long ldgu, __nv_bfloat16* out, long long ldo, long long rows, int F,
                           cudaStream_t stream) {
  if (rows <= 0 || F <= 0) return;
  swiglu_packed_fwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, stream>>>(gu, ldgu, out, ldo, rows, F);
}

void swiglu_packed_backward(const __nv_bfloat16* gu, long long ldgu, const __nv_bfloat16* dy, long long lddy,
                            __nv_bfloat16* dgu, long long lddgu, long long rows, int F, cudaStream_t stream) {
  if (rows <= 0 || F <= 0) return;
  swiglu_packed_bwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, stream>>>(gu, ldgu, dy, lddy, dgu, lddgu, rows, F);
}

void attn_merge2(const void* o1, const float* l1, const void* o2, const float* l2, void* out, long long rows, int hkv,
                 int rep, cudaStream_t stream) {
  if (rows <= 0) return;
  attn_merge2_kernel<<<grid_for(rows * hkv * 16, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(o1), l1, static_cast<const __nv_bfloat16*>(o2), l2,
      static_cast<__nv_bfloat16*>(out), rows, hkv, rep);
}

void rope_apply(const void* x, long long ldt, int dtype, const long long* pos, const float* cos_t, const float* sin_t,
                void* out, long long ldo, long long tokens, int heads, int D, bool inverse, long long table_rows,
                cudaStream_t stream) {
  if (tokens <= 0) return;
  const int threads = 256;
  const bool vec_ok = dtype == 1 && D % 16 == 0 && ldt % 8 == 0 && ldo % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0 &&
                      (reinterpret_cast<uintptr_t>(cos_t) & 15u) == 0 && (reinterpret_cast<uintptr_t>(sin_t) & 15u) == 0;
  if (vec_ok) {
    rope_bf16_vec_kernel<<<grid_for(tokens * heads * (D / 16), threads), threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), ldt, pos, cos_t, sin_t, static_cast<__nv_bfloat16*>(out), ldo, tokens, heads, D,
        inverse ? -1.f : 1.f, table_rows RLK_DBG_ARG);
    return;
  }
  const int grid = grid_for(tokens * heads * (D / 2), threads);
  RLK_DISPATCH_T(dtype, {
    rope_kernel<T><<<grid, threads, 0, stream>>>(static_cast<const T*>(x), ldt, pos, cos_t, sin_t,
                                                 static_cast<T*>(out), ldo, tokens, heads, D, inverse ? -1.f : 1.f,
                                                 table_rows RLK_DBG_ARG);
  });
}

void embedding_forward(const long long* ids, const void* table, long long ldw, int dtype, void* out, long long rows,
                       int D, long long vocab, cudaStream_t stream) {
  if (rows <= 0) return;
  RLK_DISPATCH_T(dtype, {
    embedding_fwd_kernel<T><<<rows, 128, 0, stream>>>(ids, static_cast<const T*>(table), ldw, static_cast<T*>(out), D,
                                                      vocab RLK_DBG_ARG);
  });
}

void embedding_backward(const long long* seg_ids, const long long* seg_start, long long segments,
                        const long long* order, const void* dy, int dy_dtype, int D, void* dtable, bool table_fp32,
                        long long ldw, long long dy_rows, long long table_rows, cudaStream_t stream) {
  if (segments <= 0) return;
  RLK_DISPATCH_T(dy_dtype, {
    if (table_fp32)
      embedding_bwd_kernel<T, float><<<segments, 128, 0, stream>>>(seg_ids, seg_start, order,
                                                                   static_cast<const T*>(dy), D,
                                                                   static_cast<float*>(dtable), ldw, dy_rows,
                                                                   table_rows RLK_DBG_ARG);
    else
      embedding_bwd_kernel<T, T><<<segments, 128, 0, stream>>>(seg_ids, seg_start, order, static_cast<const T*>(dy), D,
                                                               static_cast<T*>(dtable), ldw, dy_rows,
                                                               table_rows RLK_DBG_ARG);
  });
}

void adamw_step(void* p, int p_dtype, float* master, short* residual, const void* g, int g_dtype, float* m, float* v,
                long long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, float grad_scale,
                cudaStream_t stream) {
  if (n <= 0) return;
  const int threads = 256;
  long long done = 0;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                         reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(master) |
                         reinterpret_cast<uintptr_t>(residual);
  if (p_dtype == 1 && g_dtype != 2 && (bits & 15) == 0 && n >= 8) {
    const long long n8 = n / 8;
    const int grid = grid_for(n8, threads);
    __nv_bfloat16* pb = static_cast<__nv_bfloat16*>(p);
#define RLK_ADAMW_VEC(TG, MODE)                                                                                    \
  adamw_bf16_vec_kernel<TG, MODE><<<grid, threads, 0, stream>>>(pb, master, residual, static_cast<const TG*>(g), m, v, \
                                                                 n8, lr, b1, b2, eps, wd, bc1, bc2, grad_scale)
    const int mode = residual ? 2 : (master ? 1 : 0);
    if (g_dtype == 0) {
      if (mode == 2) RLK_ADAMW_VEC(float, 2); else if (mode == 1) RLK_ADAMW_VEC(float, 1); else RLK_ADAMW_VEC(float, 0);
    } else {
      if (mode == 2) RLK_ADAMW_VEC(__nv_bfloat16, 2); else if (mode == 1) RLK_ADAMW_VEC(__nv_bfloat16, 1); else RLK_ADAMW_VEC(__nv_bfloat16, 0);
    }
#undef RLK_ADAMW_VEC
    done = n8 * 8;
  }
  const long long rest = n - done;
  if (rest <= 0) return;
  const int grid = grid_for(rest, threads);
  if (residual) {  // bf16 parameters only (checked by the binding)
    __nv_bfloat16* pb = static_cast<__nv_bfloat16*>(p) + done;
    RLK_DISPATCH_T(g_dtype, {
      adamw_residual_kernel<T><<<grid, threads, 0, stream>>>(pb, residual + done, static_cast<const T*>(g) + done, m + done,
                                                             v + done, rest, lr, b1, b2, eps, wd, bc1, bc2, grad_scale);
    });
    return;
  }
  RLK_DISPATCH_T(p_dtype, {
    using TP = T;
    RLK_DISPATCH_T(g_dtype, {
      adamw_kernel<TP, T><<<grid, threads, 0, stream>>>(static_cast<TP*>(p) + done, master ? master + done : nullptr,
                                                        static_cast<const T*>(g) + done, m + done, v + done, rest, lr,
                                                        b1, b2, eps, wd, bc1, bc2, grad_scale);
    });
  });
}


// ---- per-head RMSNorm of q and k inside a packed qkv buffer (Qwen3-style q/k norm, head_dim 128) -------------------
// qkv [T, (hq + 2 hkv) * 128] bf16.  Forward: out = qkv with every q head row normalised with w_q [128] and every k
// head row with w_k [128]; v rows are copied.  One half-warp per (token, head) row: 16 lanes x 8 elements.  The
// composition it replaces (two strided slices made contiguous, two generic RMSNorm launches, one concatenation) moves
// the buffer about five times and runs the wide-row kernels on 128-element rows.
namespace {

constexpr int kQkHead = 128;

// Sum over the 16 lanes of this thread's half of the warp.  The two halves of a warp work on different rows and may
// take different branches, so the shuffle names only the lanes of its own half.
__device__ __forceinline__ float half_warp_sum(float v) {
  const unsigned int mask = 0xffffu << (threadIdx.x & 16);
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) v += __shfl_xor_sync(mask, v, off);
  return v;
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return q;
}

__global__ void __launch_bounds__(256)
qk_norm_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld, __nv_bfloat16* __restrict__ out, long long ldo,
                   const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk, long long tokens, int hq,
                   int hkv, float eps) {
  const int heads = hq + 2 * hkv;
  const long long rows = tokens * heads;
  const int sub = threadIdx.x & 15;
  const long long first = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 4;
  const long long stride = (static_cast<long long>(gridDim.x) * blockDim.x) >> 4;
  for (long long row = first; row < rows; row += stride) {  // uniform per half-warp
    const long long t = row / heads;
    const int h = static_cast<int>(row - t * heads);
    const uint4 raw = *reinterpret_cast<const uint4*>(qkv + t * ld + h * kQkHead + sub * 8);
    uint4 res = raw;
    if (h < hq + hkv) {
      float x[8];
      unpack_bf16x8(raw, x);
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(x[j], x[j], ss);
      ss = half_warp_sum(ss);
      const float rstd = rsqrtf(ss * (1.f / kQkHead) + eps);
      float w[8];
      unpack_bf16x8(*reinterpret_cast<const uint4*>((h < hq ? wq : wk) + sub * 8), w);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = x[j] * rstd * w[j];
      res = pack_bf16x8(x);
    }
    *reinterpret_cast<uint4*>(out + t * ldo + h * kQkHead + sub * 8) = res;
  }
}

// dqkv from d(out); per-block partial weight gradients part[block][2][128] (q then k), summed later in block order.
__global__ void __launch_bounds__(256)
qk_norm_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld, const __nv_bfloat16* __restrict__ dout,
                   long long ldg, __nv_bfloat16* __restrict__ dqkv, long long ldd, const __nv_bfloat16* __restrict__ wq,
                   const __nv_bfloat16* __restrict__ wk, long long tokens, int hq, int hkv, float eps,
                   float* __restrict__ part) {
  __shared__ float red[16][2][kQkHead];  // one slab per half-warp of the block
  const int heads = hq + 2 * hkv;
  const long long rows = tokens * heads;
  const int sub = threadIdx.x & 15, hw = threadIdx.x >> 4;
  const long long first = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 4;
  const long long stride = (static_cast<long long>(gridDim.x) * blockDim.x) >> 4;
  float gq[8], gk[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) gq[j] = gk[j] = 0.f;
  float wqf[8], wkf[8];
  unpack_bf16x8(*reinterpret_cast<const uint4*>(wq + sub * 8), wqf);
  unpack_bf16x8(*reinterpret_cast<const uint4*>(wk + sub * 8), wkf);
  for (long long row = first; row < rows; row += stride) {
    const long long t = row / heads;
    const int h = static_cast<int>(row - t * heads);
    const uint4 graw = *reinterpret_cast<const uint4*>(dout + t * ldg + h * kQkHead + sub * 8);
    uint4 res = graw;
    if (h < hq + hkv) {
      float x[8], dy[8];
      unpack_bf16x8(*reinterpret_cast<const uint4*>(qkv + t * ld + h * kQkHead + sub * 8), x);
      unpack_bf16x8(graw, dy);
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(x[j], x[j], ss);
      ss = half_warp_sum(ss);
      const float rstd = rsqrtf(ss * (1.f / kQkHead) + eps);
      const bool is_q = h < hq;
      float dot = 0.f, xh[8], dyw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[j] = x[j] * rstd;
        dyw[j] = dy[j] * (is_q ? wqf[j] : wkf[j]);
        dot = fmaf(dyw[j], xh[j], dot);
      }
      dot = half_warp_sum(dot) * (1.f / kQkHead);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        x[j] = rstd * (dyw[j] - xh[j] * dot);
        if (is_q) gq[j] = fmaf(dy[j], xh[j], gq[j]);
        else gk[j] = fmaf(dy[j], xh[j], gk[j]);
      }
      res = pack_bf16x8(x);
    }
    *reinterpret_cast<uint4*>(dqkv + t * ldd + h * kQkHead + sub * 8) = res;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    red[hw][0][sub * 8 + j] = gq[j];
    red[hw][1][sub * 8 + j] = gk[j];
  }
  __syncthreads();
  // 256 threads = 2 x 128 columns: sum the 16 half-warp slabs in slab order
  const int which = threadIdx.x >> 7, col = threadIdx.x & 127;
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) acc += red[i][which][col];
  part[(static_cast<long long>(blockIdx.x) * 2 + which) * kQkHead + col] = acc;
}

}  // namespace

int qk_norm_blocks(long long tokens, int heads) {
  const long long half_warps = tokens * heads;
  long long blocks = (half_warps + 15) / 16;
  const long long cap = 148LL * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

void qk_norm_forward(const __nv_bfloat16* qkv, long long ld, __nv_bfloat16* out, long long ldo, const __nv_bfloat16* wq,
                     const __nv_bfloat16* wk, long long tokens, int hq, int hkv, float eps, cudaStream_t stream) {
  if (tokens <= 0) return;
  qk_norm_fwd_kernel<<<qk_norm_blocks(tokens, hq + 2 * hkv), 256, 0, stream>>>(qkv, ld, out, ldo, wq, wk, tokens, hq, hkv, eps);
}

void qk_norm_backward(const __nv_bfloat16* qkv, long long ld, const __nv_bfloat16* dout, long long ldg,
                      __nv_bfloat16* dqkv, long long ldd, const __nv_bfloat16* wq, const __nv_bfloat16* wk,
                      long long tokens, int hq, int hkv, float eps, float* part, cudaStream_t stream) {
  if (tokens <= 0) return;
  qk_norm_bwd_kernel<<<qk_norm_blocks(tokens, hq + 2 * hkv), 256, 0, stream>>>(qkv, ld, dout, ldg, dqkv, ldd, wq, wk, tokens,
                                                                             hq, hkv, eps, part);
}

}  // namespace rlk
