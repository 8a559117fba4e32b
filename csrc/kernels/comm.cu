// Communication kernels over the symmetric heap (plain NVLink peer loads / stores, no NCCL):
//
//   peer_barrier       : all ranks of a node meet; every wait is bounded and reports a timeout in the
//                        error word instead of hanging.
//   zero1_fused_step   : gradient reduce-scatter + scale + AdamW + parameter all-gather in ONE kernel.
//                        Rank r owns elements [lo, hi) of the flat parameter vector: it loads that range
//                        of every peer's bf16 gradient buffer, sums in fixed rank order in fp32, applies
//                        AdamW on its fp32 moments (and optional fp32 master copy) and stores the new
//                        bf16 values into every peer's parameter buffer.
//   peer_sum           : out[i] = sum_r peer_r[i] in fixed rank order (used for the tensor-parallel
//                        grad_hidden reduction of the vocab-parallel LM head).
//   cast_broadcast     : weight sync: read a local buffer, cast dtype, store into every peer's buffer.
//
// In the reference these are, respectively: nothing; DeepSpeed ZeRO (external, deepspeed_trainer.py:
// 115-169); an NCCL all-reduce (ops/pytorch/loss/linear_logp.py:331); and per-tensor cuMemcpyDtoD
// into a VMM allocation (executors/bridge.py:2023-2123).
#include "../common/ptx.cuh"
#include "kernels.h"

#include <cuda_fp16.h>

namespace rlk {

namespace {

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct PeerPtrs {
  void* p[8];
};

// pads[r] points at rank r's signal pad (>= world u32 slots).  Thread r publishes `epoch` into slot
// [my rank] of peer r's pad, then waits until slot [r] of the local pad reaches `epoch`.
__global__ void peer_barrier_kernel(PeerPtrs pads, int rank, int world, unsigned int epoch,
                                    unsigned long long limit_ns, uint32_t* err) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  st_release_sys(static_cast<unsigned int*>(pads.p[r]) + rank, epoch);
  const unsigned int* mine = static_cast<const unsigned int*>(pads.p[rank]) + r;
  const uint64_t t0 = global_timer_ns();
  while (static_cast<int>(ld_acquire_sys(mine) - epoch) < 0) {
    if (global_timer_ns() - t0 > limit_ns) {
      report_error(err, kErrPeerTimeout, 300, static_cast<uint32_t>(r));
      return;
    }
    __nanosleep(100);
  }
}

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return q;
}

// [lo, hi) are element indices, multiples of 8.  m / v / master are indexed from 0 at element lo.
// ``skip_if_set``: the error word of the device barrier that precedes this kernel (or nullptr).  If that barrier
// gave up waiting for a peer, some gradients are not final, so the kernel applies nothing and returns.
// kWorld > 0 fixes the number of ranks at compile time: the loads from all peers are then issued back to back, before
// the first use, so a thread has kWorld remote loads in flight instead of one (a remote load takes microseconds; with
// one in flight per thread the kernel ran at 0.42 of the link bandwidth per direction).  kWorld == 0 is the generic
// form for other rank counts.
template <int kWorld>
__global__ void __launch_bounds__(256)
zero1_fused_step_kernel(PeerPtrs grads, PeerPtrs params, int rank, int world_rt, long long lo, long long hi,
                        float* __restrict__ m, float* __restrict__ v, float* __restrict__ master, float lr, float b1,
                        float b2, float eps, float wd, float bc1, float bc2, float grad_scale,
                        const uint32_t* __restrict__ skip_if_set) {
  if (skip_if_set != nullptr && *skip_if_set != 0u) return;
  const int world = kWorld > 0 ? kWorld : world_rt;
  const float inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2, decay = 1.f - lr * wd;
  const long long n8 = (hi - lo) / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = lo + i * 8;
    float g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = 0.f;
    if constexpr (kWorld > 0) {
      uint4 q[kWorld];
#pragma unroll
      for (int r = 0; r < kWorld; ++r)
        q[r] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(grads.p[r]) + e);
#pragma unroll
      for (int r = 0; r < kWorld; ++r) {  // fixed rank order: bitwise identical on every run and every rank
        float f[8];
        unpack8(q[r], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] += f[j];
      }
    } else {
      for (int r = 0; r < world; ++r) {
        const uint4 q = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(grads.p[r]) + e);
        float f[8];
        unpack8(q, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] += f[j];
      }
    }
    float w[8];
    if (master != nullptr) {
      const float4 a = reinterpret_cast<const float4*>(master + i * 8)[0];
      const float4 b = reinterpret_cast<const float4*>(master + i * 8)[1];
      w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    } else {
      // every rank holds identical parameters; read this rank's own copy
      unpack8(*reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(params.p[rank]) + e), w);
    }
    float mm[8], vv[8];
    {
      const float4 a = reinterpret_cast<const float4*>(m + i * 8)[0], b = reinterpret_cast<const float4*>(m + i * 8)[1];
      mm[0] = a.x; mm[1] = a.y; mm[2] = a.z; mm[3] = a.w; mm[4] = b.x; mm[5] = b.y; mm[6] = b.z; mm[7] = b.w;
      const float4 c = reinterpret_cast<const float4*>(v + i * 8)[0], d = reinterpret_cast<const float4*>(v + i * 8)[1];
      vv[0] = c.x; vv[1] = c.y; vv[2] = c.z; vv[3] = c.w; vv[4] = d.x; vv[5] = d.y; vv[6] = d.z; vv[7] = d.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * grad_scale;
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      const float denom = sqrtf(vv[j] * inv_bc2) + eps;
      w[j] = w[j] * decay - lr * (mm[j] * inv_bc1) / denom;
    }
    reinterpret_cast<float4*>(m + i * 8)[0] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(m + i * 8)[1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
    reinterpret_cast<float4*>(v + i * 8)[0] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    reinterpret_cast<float4*>(v + i * 8)[1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    if (master != nullptr) {
      reinterpret_cast<float4*>(master + i * 8)[0] = make_float4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<float4*>(master + i * 8)[1] = make_float4(w[4], w[5], w[6], w[7]);
    }
    const uint4 packed = pack8(w);
    if constexpr (kWorld > 0) {
#pragma unroll
      for (int r = 0; r < kWorld; ++r) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[r]) + e) = packed;
    } else {
      for (int r = 0; r < world; ++r) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[r]) + e) = packed;
    }
  }
}

// Eight consecutive elements of T (float, bf16 or half) <-> eight floats, by 16- or 32-byte vector accesses.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    unpack8(*reinterpret_cast<const uint4*>(p), f);
  } else {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = __half22float2(h[j]);
      f[2 * j] = x.x;
      f[2 * j + 1] = x.y;
    }
  }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  if constexpr (sizeof(T) == 4) {
    reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    *reinterpret_cast<uint4*>(p) = pack8(f);
  } else {
    uint4 q;
    __half2* h = reinterpret_cast<__half2*>(&q);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
    *reinterpret_cast<uint4*>(p) = q;
  }
}

template <typename T>
__device__ __forceinline__ float load1(const T* p) {
  if constexpr (sizeof(T) == 4) return *p;
  else if constexpr (std::is_same<T, __nv_bfloat16>::value) return __bfloat162float(*p);
  else return __half2float(*p);
}

template <typename T>
__device__ __forceinline__ void store1(T* p, float x) {
  if constexpr (sizeof(T) == 4) *p = x;
  else if constexpr (std::is_same<T, __nv_bfloat16>::value) *p = __float2bfloat16_rn(x);
  else *p = __float2half_rn(x);
}

// out[i] = sum_r src_r[i]; SRC bf16 or float, OUT bf16 or float.  ``n8`` groups of eight elements go through the
// vector path, two groups per thread and iteration so that 2 * world independent 16-byte loads are in flight per
// thread; the last n - 8 * n8 elements are scalar.  The host passes n8 = 0 unless every pointer is 16-byte aligned.
template <typename TS, typename TO>
__global__ void peer_sum_kernel(PeerPtrs srcs, int world, long long n, long long n8, TO* __restrict__ out) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  for (long long i = tid; i < n8; i += 2 * stride) {
    const long long i2 = i + stride;
    const bool two = i2 < n8;
    float acc0[8] = {}, acc1[8] = {};
    for (int r = 0; r < world; ++r) {
      float f0[8], f1[8] = {};
      load8(static_cast<const TS*>(srcs.p[r]) + i * 8, f0);
      if (two) load8(static_cast<const TS*>(srcs.p[r]) + i2 * 8, f1);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc0[j] += f0[j];
        acc1[j] += f1[j];
      }
    }
    store8(out + i * 8, acc0);
    if (two) store8(out + i2 * 8, acc1);
  }
  for (long long i = n8 * 8 + tid; i < n; i += stride) {
    float acc = 0.f;
    for (int r = 0; r < world; ++r) acc += load1(static_cast<const TS*>(srcs.p[r]) + i);
    store1(out + i, acc);
  }
}

// dst_r[i] = cast(src[i]) for every peer r.  Four groups of eight elements per thread and iteration: the loads are
// issued before the first store, so four 16/32-byte loads are in flight per thread.
template <typename TS, typename TD>
__global__ void cast_broadcast_kernel(const TS* __restrict__ src, PeerPtrs dsts, int world, long long n, long long n8) {
  constexpr int kUnroll = 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  for (long long i = tid; i < n8; i += kUnroll * stride) {
    float f[kUnroll][8];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long iu = i + u * stride;
      if (iu < n8) load8(src + iu * 8, f[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long iu = i + u * stride;
      if (iu < n8) {
        for (int r = 0; r < world; ++r) store8(static_cast<TD*>(dsts.p[r]) + iu * 8, f[u]);
      }
    }
  }
  for (long long i = n8 * 8 + tid; i < n; i += stride) {
    const float x = load1(src + i);
    for (int r = 0; r < world; ++r) store1(static_cast<TD*>(dsts.p[r]) + i, x);
  }
}

// Integrity digest of a byte range: sum over its 64-bit little-endian words w_i (the tail zero-padded) of
// (w_i ^ (w_i >> 29)) * ((i + 1) * kDigestMul), all modulo 2^64, with an arithmetic shift.  Wrap-around integer
// addition is associative and commutative, so any partition of the range over threads gives the same 64 bits.
// One pass, 16-byte loads; the result is ADDED into *out (the caller zeroes it).
constexpr unsigned long long kDigestMul = 0x9E3779B97F4A7C15ull;  // == -7046029254386353131 as a signed 64-bit value

__device__ __forceinline__ unsigned long long digest_term(long long w, unsigned long long index) {
  return static_cast<unsigned long long>(w ^ (w >> 29)) * ((index + 1ull) * kDigestMul);
}

__global__ void __launch_bounds__(256)
digest64_kernel(const long long* __restrict__ words, long long n_words, const unsigned char* __restrict__ tail,
                int tail_bytes, unsigned long long* __restrict__ out) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  unsigned long long acc = 0ull;
  const long long pairs = n_words / 2;
  for (long long i = tid; i < pairs; i += stride) {
    const longlong2 w = reinterpret_cast<const longlong2*>(words)[i];
    acc += digest_term(w.x, static_cast<unsigned long long>(2 * i));
    acc += digest_term(w.y, static_cast<unsigned long long>(2 * i + 1));
  }
  if (tid == 0) {
    if (n_words & 1) acc += digest_term(words[n_words - 1], static_cast<unsigned long long>(n_words - 1));
    if (tail_bytes > 0) {
      unsigned long long w = 0ull;
      for (int b = 0; b < tail_bytes; ++b) w |= static_cast<unsigned long long>(tail[b]) << (8 * b);
      acc += digest_term(static_cast<long long>(w), static_cast<unsigned long long>(n_words));
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if ((threadIdx.x & 31) == 0 && acc != 0ull) atomicAdd(out, acc);
}

// ---- many tensors in one launch ---------------------------------------------------------------------------------
// A weight update is hundreds of tensors; one launch per tensor costs more in launch and binding overhead than the
// bytes cost in bandwidth (291 launches for 8 GB: 15.9 ms against 2.9 ms for one).  The segment kernels take a device
// table with one row per tensor and cut the whole update into units of kSegUnit elements; block b handles units b,
// b + gridDim.x, ... and finds a unit's tensor by binary search over the table's running unit count.
struct Segment {
  long long src;         // device address of the tensor's first element
  long long dst;         // byte offset of its copy in the destination window (cast) / result slot (digest)
  long long n;           // elements (cast) / bytes (digest)
  long long first_unit;  // units of all earlier rows
};
constexpr long long kSegUnit = 1 << 15;

__device__ __forceinline__ int find_segment(const Segment* __restrict__ segs, int count, long long unit) {
  int lo = 0, hi = count - 1;
  while (lo < hi) {  // last row whose first_unit <= unit
    const int mid = (lo + hi + 1) >> 1;
    if (segs[mid].first_unit <= unit) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

// dst_base[seg.dst ...] = cast(src tensor) for every row of the table (one destination: this GPU's own window).
template <typename TS, typename TD>
__global__ void __launch_bounds__(256)
cast_segments_kernel(const Segment* __restrict__ segs, int count, long long total_units, unsigned char* __restrict__ dst_base) {
  for (long long unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
    const Segment sg = segs[find_segment(segs, count, unit)];
    const long long e0 = (unit - sg.first_unit) * kSegUnit;
    const long long len = min(kSegUnit, sg.n - e0);
    const TS* src = reinterpret_cast<const TS*>(sg.src) + e0;
    TD* dst = reinterpret_cast<TD*>(dst_base + sg.dst) + e0;
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    const long long n8 = vec ? len / 8 : 0;
    for (long long i = threadIdx.x; i < n8; i += 4 * blockDim.x) {
      float f[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u * blockDim.x < n8) load8(src + (i + u * blockDim.x) * 8, f[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u * blockDim.x < n8) store8(dst + (i + u * blockDim.x) * 8, f[u]);
    }
    for (long long i = n8 * 8 + threadIdx.x; i < len; i += blockDim.x) store1(dst + i, load1(src + i));
  }
}

// results[seg.dst] += digest of the tensor's bytes, for every row of the table (same function as digest64_kernel: the
// terms carry their word index, so any partition into units gives the same 64 bits).
__global__ void __launch_bounds__(256)
digest_segments_kernel(const Segment* __restrict__ segs, int count, long long total_units,
                       unsigned long long* __restrict__ results) {
  constexpr long long kWordsPerUnit = kSegUnit;  // 64-bit words
  for (long long unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
    const Segment sg = segs[find_segment(segs, count, unit)];
    const long long n_words = sg.n / 8;
    const int tail_bytes = static_cast<int>(sg.n - n_words * 8);
    const long long w0 = (unit - sg.first_unit) * kWordsPerUnit;
    const long long w1 = min(w0 + kWordsPerUnit, n_words);
    const long long* words = reinterpret_cast<const long long*>(sg.src);
    unsigned long long acc = 0ull;
    // w0 is even, so pairs of words are 16-byte aligned whenever the tensor is
    for (long long i = w0 + 2 * threadIdx.x; i + 1 < w1; i += 2 * blockDim.x) {
      const longlong2 w = *reinterpret_cast<const longlong2*>(words + i);
      acc += digest_term(w.x, static_cast<unsigned long long>(i));
      acc += digest_term(w.y, static_cast<unsigned long long>(i + 1));
    }
    if (threadIdx.x == 0) {
      if (((w1 - w0) & 1) && w1 > w0) acc += digest_term(words[w1 - 1], static_cast<unsigned long long>(w1 - 1));
      const bool last_unit = w0 + kWordsPerUnit >= n_words;
      if (last_unit && tail_bytes > 0) {
        const unsigned char* tail = reinterpret_cast<const unsigned char*>(sg.src) + n_words * 8;
        unsigned long long w = 0ull;
        for (int b = 0; b < tail_bytes; ++b) w |= static_cast<unsigned long long>(tail[b]) << (8 * b);
        acc += digest_term(static_cast<long long>(w), static_cast<unsigned long long>(n_words));
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0 && acc != 0ull) atomicAdd(results + sg.dst, acc);
  }
}

PeerPtrs make_ptrs(void* const* p, int world) {
  PeerPtrs out;
  for (int r = 0; r < 8; ++r) out.p[r] = r < world ? p[r] : nullptr;
  return out;
}

// Number of 8-element groups that may use vector accesses: all of them if every pointer is 16-byte aligned, else none.
long long vector_groups(void* const* ptrs, int world, const void* other, long long n) {
  uintptr_t bits = reinterpret_cast<uintptr_t>(other);
  for (int r = 0; r < world; ++r) bits |= reinterpret_cast<uintptr_t>(ptrs[r]);
  return (bits & 15) == 0 ? n / 8 : 0;
}

int capped_grid(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = 148LL * 8;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

void peer_barrier(void* const* pads, int rank, int world, unsigned int epoch, unsigned long long limit_ns, uint32_t* err,
                  cudaStream_t stream) {
  peer_barrier_kernel<<<1, 32, 0, stream>>>(make_ptrs(pads, world), rank, world, epoch, limit_ns, err);
}

void zero1_fused_step(void* const* grads, void* const* params, int rank, int world, long long lo, long long hi, float* m,
                      float* v, float* master, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                      float grad_scale, const uint32_t* skip_if_set, int max_blocks, cudaStream_t stream) {
  if (hi <= lo) return;
  int grid = capped_grid((hi - lo) / 8, 256);
  if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;
#define RLK_ZERO1(W)                                                                                              \
  zero1_fused_step_kernel<W><<<grid, 256, 0, stream>>>(make_ptrs(grads, world), make_ptrs(params, world), rank, world, \
                                                       lo, hi, m, v, master, lr, b1, b2, eps, wd, bc1, bc2,          \
                                                       grad_scale, skip_if_set)
  switch (world) {
    case 1: RLK_ZERO1(1); break;
    case 2: RLK_ZERO1(2); break;
    case 4: RLK_ZERO1(4); break;
    case 8: RLK_ZERO1(8); break;
    default: RLK_ZERO1(0); break;
  }
#undef RLK_ZERO1
}

void weight_digest64(const void* data, long long nbytes, unsigned long long* out, cudaStream_t stream) {
  if (nbytes <= 0) return;
  const long long n_words = nbytes / 8;
  const int tail = static_cast<int>(nbytes % 8);
  const int grid = capped_grid(n_words / 2 + 1, 256);
  digest64_kernel<<<grid, 256, 0, stream>>>(static_cast<const long long*>(data), n_words,
                                            static_cast<const unsigned char*>(data) + n_words * 8, tail, out);
}

void peer_sum(void* const* srcs, int world, long long n, bool src_fp32, void* out, bool out_fp32, cudaStream_t stream) {
  if (n <= 0) return;
  const PeerPtrs p = make_ptrs(srcs, world);
  const long long n8 = vector_groups(srcs, world, out, n);
  const int grid = capped_grid(n8 > 0 ? (n8 + 1) / 2 : n, 256);
  if (src_fp32) {
    if (out_fp32) peer_sum_kernel<float, float><<<grid, 256, 0, stream>>>(p, world, n, n8, static_cast<float*>(out));
    else peer_sum_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>(p, world, n, n8, static_cast<__nv_bfloat16*>(out));
  } else {
    if (out_fp32) peer_sum_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(p, world, n, n8, static_cast<float*>(out));
    else peer_sum_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(p, world, n, n8, static_cast<__nv_bfloat16*>(out));
  }
}

void cast_broadcast(const void* src, int src_dtype, void* const* dsts, int dst_dtype, int world, long long n,
                    cudaStream_t stream) {
  if (n <= 0) return;
  const PeerPtrs p = make_ptrs(dsts, world);
  const long long n8 = vector_groups(dsts, world, src, n);
  const int grid = capped_grid(n8 > 0 ? (n8 + 3) / 4 : n, 256);
#define RLK_CB(TS, TD) \
  cast_broadcast_kernel<TS, TD><<<grid, 256, 0, stream>>>(static_cast<const TS*>(src), p, world, n, n8)
  if (src_dtype == 0) {
    if (dst_dtype == 0) RLK_CB(float, float);
    else if (dst_dtype == 1) RLK_CB(float, __nv_bfloat16);
    else RLK_CB(float, __half);
  } else if (src_dtype == 1) {
    if (dst_dtype == 0) RLK_CB(__nv_bfloat16, float);
    else if (dst_dtype == 1) RLK_CB(__nv_bfloat16, __nv_bfloat16);
    else RLK_CB(__nv_bfloat16, __half);
  } else {
    if (dst_dtype == 0) RLK_CB(__half, float);
    else if (dst_dtype == 1) RLK_CB(__half, __nv_bfloat16);
    else RLK_CB(__half, __half);
  }
#undef RLK_CB
}

void cast_segments(const void* table, int count, long long total_units, int src_dtype, int dst_dtype, void* dst_base,
                   cudaStream_t stream) {
  if (count <= 0 || total_units <= 0) return;
  const int grid = static_cast<int>(total_units < 148LL * 8 ? total_units : 148LL * 8);
  const Segment* segs = static_cast<const Segment*>(table);
  unsigned char* dst = static_cast<unsigned char*>(dst_base);
#define RLK_CS(TS, TD) cast_segments_kernel<TS, TD><<<grid, 256, 0, stream>>>(segs, count, total_units, dst)
  if (src_dtype == 0) {
    if (dst_dtype == 0) RLK_CS(float, float);
    else if (dst_dtype == 1) RLK_CS(float, __nv_bfloat16);
    else RLK_CS(float, __half);
  } else if (src_dtype == 1) {
    if (dst_dtype == 0) RLK_CS(__nv_bfloat16, float);
    else if (dst_dtype == 1) RLK_CS(__nv_bfloat16, __nv_bfloat16);
    else RLK_CS(__nv_bfloat16, __half);
  } else {
    if (dst_dtype == 0) RLK_CS(__half, float);
    else if (dst_dtype == 1) RLK_CS(__half, __nv_bfloat16);
    else RLK_CS(__half, __half);
  }
#undef RLK_CS
}

void digest_segments(const void* table, int count, long long total_units, unsigned long long* results, cudaStream_t stream) {
  if (count <= 0 || total_units <= 0) return;
  const int grid = static_cast<int>(total_units < 148LL * 8 ? total_units : 148LL * 8);
  digest_segments_kernel<<<grid, 256, 0, stream>>>(static_cast<const Segment*>(table), count, total_units, results);
}

}  // namespace rlk
