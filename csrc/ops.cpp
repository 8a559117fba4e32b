// Python bindings (module rl_engine._C).  This is the only translation unit that sees torch; it
// validates tensors, allocates outputs on the caller's device and launches on the current stream.
// Reference counterpart: csrc/ops.cpp:1-99 (pybind of 11-13 functions, launches on the default stream).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdlib>

#include <atomic>
#include <optional>
#include <vector>

#include "common/trace.h"
#include "kernels/kernels.h"
#include "runtime/runtime.h"

namespace {

using torch::Tensor;
std::atomic<long long> g_launches{0};

int dtype_code(const Tensor& t) {
  switch (t.scalar_type()) {
    case torch::kFloat32: return 0;
    case torch::kBFloat16: return 1;
    case torch::kFloat16: return 2;
    default: TORCH_CHECK(false, "rl_engine: unsupported dtype ", t.scalar_type(), " (float32, bfloat16, float16 only)");
  }
}

void check_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), "rl_engine: ", name, " must be a CUDA tensor");
}
void check_rowmajor(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, "rl_engine: ", name, " must be 2-D with unit inner stride");
}

// One 4-word error record per device, allocated on first use.
Tensor& error_word(int device) {
  static std::vector<Tensor> words(64);
  if (!words[device].defined()) {
    words[device] = torch::zeros({4}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
    // debug-bounds builds: kernels without an error-word parameter report checked indices here
    rlk::bind_debug_error_word(device, reinterpret_cast<uint32_t*>(words[device].data_ptr<int>()));
  }
  return words[device];
}

cudaStream_t stream_of(const Tensor& t) {
#if defined(RLK_DEBUG_BOUNDS)
  error_word(t.get_device());  // make sure the word exists before any launch on this device
#endif
  return at::cuda::getCurrentCUDAStream(t.get_device()).stream();
}
uint32_t* err_ptr(const Tensor& like) { return reinterpret_cast<uint32_t*>(error_word(like.get_device()).data_ptr<int>()); }

int sm_count_of(int device) {
  static std::vector<int> cache(64, 0);
  if (cache[device] == 0) cache[device] = at::cuda::getDeviceProperties(device)->multiProcessorCount;
  return cache[device];
}

void after_launch(int n = 1) {
  g_launches += n;
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------ GEMM
// Default tile engine of the plain GEMM: CTA pairs (256 x 256 tiles, cta_group::2) or single CTAs.
// RLK_GEMM_PAIR=0/1 overrides the built-in default; gemm(..., pair=0/1) overrides both for one call.
bool gemm_pair_default() {
  static const int value = [] {
    const char* env = std::getenv("RLK_GEMM_PAIR");
    if (env != nullptr && env[0] != '\0') return env[0] != '0' ? 1 : 0;
    return 1;
  }();
  return value != 0;
}

Tensor gemm(const Tensor& a, const Tensor& b, bool a_mn, bool b_mn, std::optional<Tensor> out, bool out_fp32,
            bool accumulate, double alpha, int64_t pair) {
  check_rowmajor(a, "a");
  check_rowmajor(b, "b");
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16, "rl_engine.gemm: bf16 operands only");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "rl_engine.gemm: contraction sizes differ (", K, " vs ", Kb, ")");
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0, "rl_engine.gemm: operand row pitch must be a multiple of 8 elements");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0,
              "rl_engine.gemm: operands must be 16-byte aligned");
  Tensor d;
  if (out.has_value()) {
    d = *out;
    check_rowmajor(d, "out");
    TORCH_CHECK(d.size(0) == M && d.size(1) == N, "rl_engine.gemm: out has the wrong shape");
    TORCH_CHECK(d.scalar_type() == (out_fp32 ? torch::kFloat32 : torch::kBFloat16), "rl_engine.gemm: out dtype mismatch");
  } else {
    TORCH_CHECK(!accumulate, "rl_engine.gemm: accumulate needs an explicit out tensor");
    d = torch::empty({M, N}, a.options().dtype(out_fp32 ? torch::kFloat32 : torch::kBFloat16));
  }
  if (M == 0 || N == 0) return d;
  if (K == 0) {
    if (!accumulate) d.zero_();
    return d;
  }
  rlk::GemmArgs g;
  g.A = reinterpret_cast<const __nv_bfloat16*>(a.data_ptr());
  g.B = reinterpret_cast<const __nv_bfloat16*>(b.data_ptr());
  g.D = d.data_ptr();
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.K = static_cast<int>(K);
  g.lda = a.stride(0);
  g.ldb = b.stride(0);
  g.ldd = d.stride(0);
  g.a_mn_major = a_mn;
  g.b_mn_major = b_mn;
  g.out_fp32 = out_fp32;
  g.accumulate = accumulate;
  g.alpha = static_cast<float>(alpha);
  g.sm_count = sm_count_of(a.get_device());
  g.err = err_ptr(a);
  // Default engine: CTA pairs, except for a single 128-row tile (nothing to pair).  Measured in seconds-long loops
  // under the power cap on B200 (T = 16384 and 32768 tokens, Llama-3-8B linears, forward / dgrad / wgrad): with
  // rasterisation groups of at least eight 256-row tiles the pair engine is as fast or faster than the single-CTA
  // engine on every shape (up to 12 % on the gate/up weight gradient), although it runs at a lower clock.
  const bool pair_suits = M > 128;
  g.cta_pair = pair < 0 ? (gemm_pair_default() && pair_suits) : pair != 0;
  rlk::gemm_bf16(g, stream_of(a));
  after_launch();
  return d;
}

// x [rows, cols] bf16 -> (e4m3 codes [rows, cols] as uint8, fp32 scale per row) with x ~= code * scale.
std::vector<Tensor> quantize_fp8_rows(const Tensor& x) {
  check_rowmajor(x, "x");
  TORCH_CHECK(x.scalar_type() == torch::kBFloat16, "rl_engine.quantize_fp8_rows: bf16 input only");
  TORCH_CHECK(x.size(1) % 16 == 0, "rl_engine.quantize_fp8_rows: the row length must be a multiple of 16");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor q = torch::empty({x.size(0), x.size(1)}, x.options().dtype(torch::kUInt8));
  Tensor scale = torch::empty({x.size(0)}, x.options().dtype(torch::kFloat32));
  if (x.numel()) {
    rlk::quantize_rows_e4m3(x.data_ptr(), x.stride(0), x.size(0), static_cast<int>(x.size(1)), q.data_ptr(), q.stride(0),
                            scale.data_ptr<float>(), stream_of(x));
    after_launch();
  }
  return {q, scale};
}

// D[M, N] bf16 = (A_q[M, K] @ B_q[N, K]^T) * scale_a[:, None] * scale_b[None, :]; e4m3 codes as uint8.
Tensor gemm_fp8(const Tensor& a_q, const Tensor& scale_a, const Tensor& b_q, const Tensor& scale_b, int64_t pair) {
  check_rowmajor(a_q, "a_q");
  check_rowmajor(b_q, "b_q");
  TORCH_CHECK(a_q.scalar_type() == torch::kUInt8 && b_q.scalar_type() == torch::kUInt8,
              "rl_engine.gemm_fp8: operands are e4m3 codes stored as uint8");
  TORCH_CHECK(a_q.size(1) == b_q.size(1), "rl_engine.gemm_fp8: contraction sizes differ");
  TORCH_CHECK(a_q.stride(0) % 16 == 0 && b_q.stride(0) % 16 == 0, "rl_engine.gemm_fp8: row pitch must be a multiple of 16 bytes");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(a_q.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(b_q.data_ptr()) % 16 == 0,
              "rl_engine.gemm_fp8: operands must be 16-byte aligned");
  auto check_scale = [](const Tensor& s, int64_t n, const char* name) {
    TORCH_CHECK(s.is_cuda() && s.scalar_type() == torch::kFloat32 && s.is_contiguous() && s.numel() == n,
                "rl_engine.gemm_fp8: ", name, " must be a contiguous float32 vector with one entry per row");
  };
  check_scale(scale_a, a_q.size(0), "scale_a");
  check_scale(scale_b, b_q.size(0), "scale_b");
  const c10::cuda::CUDAGuard guard(a_q.device());
  const int64_t M = a_q.size(0), N = b_q.size(0), K = a_q.size(1);
  Tensor d = torch::empty({M, N}, a_q.options().dtype(torch::kBFloat16));
  if (M == 0 || N == 0) return d;
  if (K == 0) return d.zero_();
  rlk::gemm_fp8_rowscaled(a_q.data_ptr(), a_q.stride(0), scale_a.data_ptr<float>(), b_q.data_ptr(), b_q.stride(0),
                          scale_b.data_ptr<float>(), d.data_ptr(), d.stride(0), static_cast<int>(M), static_cast<int>(N),
                          static_cast<int>(K), pair < 0 ? (gemm_pair_default() && M > 128) : pair != 0,
                          sm_count_of(a_q.get_device()), err_ptr(a_q), stream_of(a_q));
  after_launch();
  return d;
}

// --------------------------------------------------------------- tensor-parallel fused linears
void fill_peers(void** dst, const std::vector<uint64_t>& src, const char* what) {
  TORCH_CHECK(!src.empty() && src.size() <= 8, "rl_engine.tp: need 1..8 addresses for ", what);
  for (size_t i = 0; i < 8; ++i) dst[i] = i < src.size() ? reinterpret_cast<void*>(src[i]) : nullptr;
  for (auto a : src) TORCH_CHECK(a != 0 && a % 16 == 0, "rl_engine.tp: bad peer address for ", what);
}

// out[M, N] = allgather_rows(x_local) * B^T, the gather fused into the GEMM kernel.
Tensor tp_ag_gemm(const Tensor& x_local, const Tensor& b, bool b_mn, int64_t rank, std::vector<uint64_t> gathered,
                  std::vector<uint64_t> ready, int64_t epoch, int64_t chunks, double wait_ms) {
  check_rowmajor(x_local, "x_local");
  check_rowmajor(b, "b");
  TORCH_CHECK(x_local.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16, "rl_engine.tp_ag_gemm: bf16 only");
  const c10::cuda::CUDAGuard guard(x_local.device());
  const int64_t world = static_cast<int64_t>(gathered.size());
  const int64_t rows = x_local.size(0), K = x_local.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == K, "rl_engine.tp_ag_gemm: contraction sizes differ");
  TORCH_CHECK(rows > 0 && rows % 128 == 0, "rl_engine.tp_ag_gemm: local rows must be a positive multiple of 128");
  TORCH_CHECK(chunks >= 1 && K % (8 * chunks) == 0, "rl_engine.tp_ag_gemm: K must be a multiple of 8 * chunks");
  TORCH_CHECK(N % 8 == 0, "rl_engine.tp_ag_gemm: N must be a multiple of 8 (the output is written by TMA)");
  TORCH_CHECK(x_local.stride(0) % 8 == 0 && b.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(x_local.data_ptr()) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0,
              "rl_engine.tp_ag_gemm: operands must be 16-byte aligned with row pitch % 8 == 0");
  TORCH_CHECK(ready.size() == gathered.size() && rank >= 0 && rank < world, "rl_engine.tp_ag_gemm: bad rank / peer lists");
  Tensor out = torch::empty({rows * world, N}, x_local.options());
  rlk::TpAgGemmArgs a;
  a.x_local = reinterpret_cast<const __nv_bfloat16*>(x_local.data_ptr());
  a.ldx = x_local.stride(0);
  a.rows_local = static_cast<int>(rows);
  a.K = static_cast<int>(K);
  a.N = static_cast<int>(N);
  a.B = reinterpret_cast<const __nv_bfloat16*>(b.data_ptr());
  a.ldb = b.stride(0);
  a.b_mn = b_mn;
  a.C = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  a.ldc = out.stride(0);
  a.rank = static_cast<int>(rank);
  a.world = static_cast<int>(world);
  a.epoch = static_cast<unsigned int>(epoch);
  a.chunks = static_cast<int>(chunks);
  fill_peers(a.gathered, gathered, "gathered");
  fill_peers(a.ready, ready, "ready");
  a.wait_ns = static_cast<unsigned long long>(wait_ms * 1e6);
  a.sm_count = sm_count_of(x_local.get_device());
  a.err = err_ptr(x_local);
  rlk::tp_ag_gemm(a, stream_of(x_local));
  after_launch();
  return out;
}

// out[M / W, N] = reduce_scatter_rows(a * B^T), the reduction fused into the GEMM kernel.
Tensor tp_gemm_rs(const Tensor& a_in, const Tensor& b, bool b_mn, int64_t rank, std::vector<uint64_t> partial,
                  std::vector<uint64_t> counters, int64_t target, double wait_ms) {
  check_rowmajor(a_in, "a");
  check_rowmajor(b, "b");
  TORCH_CHECK(a_in.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16, "rl_engine.tp_gemm_rs: bf16 only");
  const c10::cuda::CUDAGuard guard(a_in.device());
  const int64_t world = static_cast<int64_t>(partial.size());
  const int64_t M = a_in.size(0), K = a_in.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == K, "rl_engine.tp_gemm_rs: contraction sizes differ");
  TORCH_CHECK(M % (128 * world) == 0 && M > 0, "rl_engine.tp_gemm_rs: rows must be a positive multiple of 128 * world");
  TORCH_CHECK(N % 8 == 0, "rl_engine.tp_gemm_rs: N must be a multiple of 8");
  TORCH_CHECK(a_in.stride(0) % 8 == 0 && b.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(a_in.data_ptr()) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0,
              "rl_engine.tp_gemm_rs: operands must be 16-byte aligned with row pitch % 8 == 0");
  TORCH_CHECK(counters.size() == partial.size() && rank >= 0 && rank < world, "rl_engine.tp_gemm_rs: bad rank / peer lists");
  Tensor out = torch::empty({M / world, N}, a_in.options());
  rlk::TpGemmRsArgs g;
  g.A = reinterpret_cast<const __nv_bfloat16*>(a_in.data_ptr());
  g.lda = a_in.stride(0);
  g.rows_local = static_cast<int>(M / world);
  g.K = static_cast<int>(K);
  g.N = static_cast<int>(N);
  g.B = reinterpret_cast<const __nv_bfloat16*>(b.data_ptr());
  g.ldb = b.stride(0);
  g.b_mn = b_mn;
  g.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  g.ldo = out.stride(0);
  g.rank = static_cast<int>(rank);
  g.world = static_cast<int>(world);
  g.target = static_cast<unsigned int>(target);
  fill_peers(g.partial, partial, "partial");
  fill_peers(g.counters, counters, "counters");
  g.wait_ns = static_cast<unsigned long long>(wait_ms * 1e6);
  g.sm_count = sm_count_of(a_in.get_device());
  g.err = err_ptr(a_in);
  rlk::tp_gemm_rs(g, stream_of(a_in));
  after_launch();
  return out;
}

// Grouped GEMM for mixture-of-experts layers (see GemmArgs::group_mode in kernels.h).
//   mode 1: a [rows, K] (rows grouped by expert, 128-row padded blocks), b [G * N, K] (b_mn = false) or
//           [G * K, N] (b_mn = true, used for dX = dY * W_g), tile_group int32 [rows / 128]  -> out [rows, N]
//   mode 2: a [rows, M], b [rows, N], group_offsets int32 [G + 1]  -> out [G * M, N] = per-group a^T b
Tensor grouped_gemm(const Tensor& a, const Tensor& b, int64_t mode, const Tensor& table, int64_t num_groups, bool b_mn,
                    bool out_fp32, std::optional<Tensor> out) {
  check_rowmajor(a, "a");
  check_rowmajor(b, "b");
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16, "grouped_gemm: bf16 operands only");
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == torch::kInt32 && table.is_contiguous(), "grouped_gemm: int32 table on GPU");
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0,
              "grouped_gemm: operands must be 16-byte aligned with 16-byte row pitch");
  const c10::cuda::CUDAGuard guard(a.device());
  rlk::GemmArgs g;
  g.A = reinterpret_cast<const __nv_bfloat16*>(a.data_ptr());
  g.B = reinterpret_cast<const __nv_bfloat16*>(b.data_ptr());
  g.lda = a.stride(0);
  g.ldb = b.stride(0);
  g.out_fp32 = out_fp32;
  g.accumulate = false;
  g.alpha = 1.f;
  g.sm_count = sm_count_of(a.get_device());
  g.err = err_ptr(a);
  g.group_mode = static_cast<int>(mode);
  g.num_groups = static_cast<int>(num_groups);
  Tensor d;
  auto odt = a.options().dtype(out_fp32 ? torch::kFloat32 : torch::kBFloat16);
  if (mode == 1) {
    TORCH_CHECK(a.size(0) % 128 == 0 && table.numel() == a.size(0) / 128, "grouped_gemm(1): rows must be 128-padded, one table entry per tile");
    const int64_t K = a.size(1);
    const int64_t N = b_mn ? b.size(1) : b.size(0) / num_groups;
    TORCH_CHECK(b_mn ? (b.size(0) == num_groups * K) : (b.size(1) == K && b.size(0) == num_groups * N), "grouped_gemm(1): b has the wrong shape");
    TORCH_CHECK(!b_mn || K % 64 == 0, "grouped_gemm(1): contraction size must be a multiple of 64 for stacked MN-major b");
    if (out.has_value()) {  // the caller's buffer (e.g. a window of symmetric memory that peers read afterwards)
      d = *out;
      TORCH_CHECK(d.is_cuda() && d.device() == a.device() && d.dim() == 2 && d.size(0) == a.size(0) && d.size(1) == N &&
                      d.stride(1) == 1 && d.scalar_type() == odt.dtype().toScalarType(),
                  "grouped_gemm(1): out must be [rows, N] of the output dtype on the operands' device");
    } else {
      d = torch::empty({a.size(0), N}, odt);
    }
    g.M = static_cast<int>(a.size(0));
    g.N = static_cast<int>(N);
    g.K = static_cast<int>(K);
    g.a_mn_major = false;
    g.b_mn_major = b_mn;
    g.tile_group = table.data_ptr<int>();
  } else {
    TORCH_CHECK(mode == 2 && a.size(0) == b.size(0) && table.numel() == num_groups + 1, "grouped_gemm(2): bad operands");
    TORCH_CHECK(!out.has_value(), "grouped_gemm(2): out is only supported for the grouped-M mode");
    TORCH_CHECK(a.size(1) % 128 == 0, "grouped_gemm(2): per-group output rows must be a multiple of 128");
    d = torch::empty({num_groups * a.size(1), b.size(1)}, odt);
    g.M = static_cast<int>(a.size(1));
    g.N = static_cast<int>(b.size(1));
    g.K = static_cast<int>(a.size(0));
    g.a_mn_major = true;
    g.b_mn_major = true;
    g.group_offsets = table.data_ptr<int>();
  }
  g.D = d.data_ptr();
  g.ldd = d.stride(0);
  if (d.numel() == 0) return d;
  rlk::gemm_bf16(g, stream_of(a));
  after_launch();
  return d;
}

std::vector<Tensor> moe_topk(const Tensor& logits, int64_t k) {
  check_rowmajor(logits, "router_logits");
  TORCH_CHECK(logits.scalar_type() == torch::kFloat32 && logits.is_contiguous(), "moe_topk: contiguous float32 logits");
  TORCH_CHECK(logits.size(1) <= 512 && k >= 1 && k <= 32 && k <= logits.size(1), "moe_topk: experts <= 512, 1 <= k <= min(32, experts)");
  const c10::cuda::CUDAGuard guard(logits.device());
  Tensor idx = torch::empty({logits.size(0), k}, logits.options().dtype(torch::kInt32));
  Tensor w = torch::empty({logits.size(0), k}, logits.options());
  if (logits.size(0)) {
    rlk::moe_topk(logits.data_ptr<float>(), static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                  static_cast<int>(k), idx.data_ptr<int>(), w.data_ptr<float>(), stream_of(logits));
    after_launch();
  }
  return {idx, w};
}

// d logits [T, E] from the gradient of the renormalised top-k weights [T, k].
Tensor moe_topk_bwd(const Tensor& idx, const Tensor& weight, const Tensor& dweight, int64_t experts) {
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == torch::kInt32 && idx.is_contiguous() && idx.dim() == 2,
              "moe_topk_bwd: idx must be a contiguous int32 CUDA tensor [T, k]");
  TORCH_CHECK(weight.scalar_type() == torch::kFloat32 && weight.is_contiguous() && weight.sizes() == idx.sizes() &&
                  dweight.scalar_type() == torch::kFloat32 && dweight.is_contiguous() && dweight.sizes() == idx.sizes() &&
                  weight.device() == idx.device() && dweight.device() == idx.device(),
              "moe_topk_bwd: weight and dweight must be contiguous float32 tensors shaped like idx on its device");
  TORCH_CHECK(idx.size(1) >= 1 && idx.size(1) <= 32 && experts >= idx.size(1), "moe_topk_bwd: 1 <= k <= min(32, experts)");
  const c10::cuda::CUDAGuard guard(idx.device());
  Tensor dlogits = torch::empty({idx.size(0), experts}, weight.options());
  if (idx.size(0)) {
    rlk::moe_topk_backward(idx.data_ptr<int>(), weight.data_ptr<float>(), dweight.data_ptr<float>(),
                           static_cast<int>(idx.size(0)), static_cast<int>(experts), static_cast<int>(idx.size(1)),
                           dlogits.data_ptr<float>(), stream_of(idx));
    after_launch();
  }
  return dlogits;
}

// (slot [T, k], src_row [S], tile_group [S / 128], offsets [E + 1], counts [E]) for expert ids `idx` int32 [T, k].
std::vector<Tensor> moe_build_plan(const Tensor& idx, int64_t experts, int64_t num_slots, int64_t unused_group) {
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == torch::kInt32 && idx.is_contiguous() && idx.dim() == 2, "moe_build_plan: idx int32 [T, k]");
  TORCH_CHECK(experts >= 1 && experts <= 4096 && num_slots % 128 == 0, "moe_build_plan: 1 <= experts <= 4096, num_slots % 128 == 0");
  const c10::cuda::CUDAGuard guard(idx.device());
  const int64_t a = idx.numel(), k = idx.size(1);
  // every expert block is padded to a multiple of 128 rows (empty experts keep one block): at most a + 128 * experts rows
  TORCH_CHECK(num_slots >= (a + 128 * experts) / 128 * 128, "moe_build_plan: num_slots is below the worst-case padded size");
  auto opt = idx.options();
  Tensor slot = torch::empty({idx.size(0), k}, opt);
  Tensor src_row = torch::full({num_slots}, -1, opt);
  Tensor tile_group = torch::empty({num_slots / 128}, opt);
  Tensor offsets = torch::empty({experts + 1}, opt);
  Tensor counts = torch::empty({experts}, opt);
  const int64_t chunks = (a + 255) / 256;
  Tensor scratch = torch::empty({std::max<int64_t>(chunks, 1) * experts}, opt);
  if (a > 0) {
    rlk::moe_build_plan(idx.data_ptr<int>(), static_cast<int>(a), static_cast<int>(k), static_cast<int>(experts),
                        static_cast<int>(num_slots), static_cast<int>(unused_group), scratch.data_ptr<int>(),
                        offsets.data_ptr<int>(), counts.data_ptr<int>(), tile_group.data_ptr<int>(), slot.data_ptr<int>(),
                        src_row.data_ptr<int>(), stream_of(idx));
    after_launch(3);
  }
  return {slot, src_row, tile_group, offsets, counts};
}

void check_bf16_rows(const Tensor& t, const char* n) {
  check_rowmajor(t, n);
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16 && t.size(1) % 8 == 0 && t.stride(0) % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0,
              "rl_engine.moe: ", n, " must be bf16 rows of a multiple of 8 elements, 16-byte aligned");
}

// dst_ptr == 0: allocate [slots, H] locally; else write to that device address (e.g. a peer's buffer).
Tensor moe_gather_rows(const Tensor& src, const Tensor& src_row, std::optional<Tensor> scale, int64_t dst_ptr,
                       int64_t dst_ld) {
  check_bf16_rows(src, "src");
  TORCH_CHECK(src_row.is_cuda() && src_row.scalar_type() == torch::kInt32 && src_row.is_contiguous(), "src_row: int32 GPU");
  const c10::cuda::CUDAGuard guard(src.device());
  const int64_t slots = src_row.numel(), h = src.size(1);
  Tensor out;
  __nv_bfloat16* dst;
  long long ld;
  if (dst_ptr == 0) {
    out = torch::empty({slots, h}, src.options());
    dst = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
    ld = h;
  } else {
    dst = reinterpret_cast<__nv_bfloat16*>(dst_ptr);
    ld = dst_ld;
  }
  const float* sp = nullptr;
  Tensor sc;
  if (scale.has_value() && scale->defined()) {
    sc = scale->to(torch::kFloat32).contiguous();
    TORCH_CHECK(sc.numel() == slots, "scale must have one entry per slot");
    sp = sc.data_ptr<float>();
  }
  if (slots) {
    rlk::moe_gather_rows(reinterpret_cast<const __nv_bfloat16*>(src.data_ptr()), src.stride(0), src_row.data_ptr<int>(), sp,
                         dst, ld, static_cast<int>(slots), static_cast<int>(h), stream_of(src), src.size(0), err_ptr(src));
    after_launch();
  }
  return out;
}

// src_ptr != 0 reads rows from that device address (e.g. a peer's expert output buffer) with pitch src_ld.
Tensor moe_combine(std::optional<Tensor> src, int64_t src_ptr, int64_t src_ld, int64_t hidden, const Tensor& slot,
                   std::optional<Tensor> weight) {
  TORCH_CHECK(slot.is_cuda() && slot.scalar_type() == torch::kInt32 && slot.is_contiguous() && slot.dim() == 2, "slot: int32 [T, k]");
  const c10::cuda::CUDAGuard guard(slot.device());
  const __nv_bfloat16* sp;
  long long ld;
  if (src.has_value() && src->defined()) {
    check_bf16_rows(*src, "src");
    sp = reinterpret_cast<const __nv_bfloat16*>(src->data_ptr());
    ld = src->stride(0);
    hidden = src->size(1);
  } else {
    TORCH_CHECK(src_ptr != 0 && hidden % 8 == 0, "moe_combine: need src tensor or src_ptr");
    sp = reinterpret_cast<const __nv_bfloat16*>(src_ptr);
    ld = src_ld;
  }
  const float* wp = nullptr;
  Tensor w;
  if (weight.has_value() && weight->defined()) {
    w = weight->to(torch::kFloat32).contiguous();
    TORCH_CHECK(w.numel() == slot.numel(), "weight must match slot");
    wp = w.data_ptr<float>();
  }
  Tensor out = torch::empty({slot.size(0), hidden}, slot.options().dtype(torch::kBFloat16));
  if (slot.size(0)) {
    rlk::moe_combine(sp, ld, slot.data_ptr<int>(), wp, static_cast<int>(slot.size(1)),
                     reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), out.stride(0), static_cast<int>(slot.size(0)),
                     static_cast<int>(hidden), stream_of(slot), (src.has_value() && src->defined()) ? src->size(0) : 0,
                     err_ptr(slot));
    after_launch();
  }
  return out;
}

Tensor moe_rowdot(const Tensor& a, const Tensor& b, const Tensor& slot) {
  check_bf16_rows(a, "a");
  check_bf16_rows(b, "b");
  TORCH_CHECK(slot.is_cuda() && slot.scalar_type() == torch::kInt32 && slot.is_contiguous() && slot.dim() == 2 &&
                  slot.size(0) == a.size(0) && a.size(1) == b.size(1),
              "moe_rowdot: slot int32 [T, k], a [T, H], b [slots, H]");
  const c10::cuda::CUDAGuard guard(a.device());
  Tensor out = torch::empty({slot.size(0), slot.size(1)}, a.options().dtype(torch::kFloat32));
  if (slot.numel()) {
    rlk::moe_rowdot(reinterpret_cast<const __nv_bfloat16*>(a.data_ptr()), a.stride(0),
                    reinterpret_cast<const __nv_bfloat16*>(b.data_ptr()), b.stride(0), slot.data_ptr<int>(),
                    static_cast<int>(slot.size(1)), static_cast<int>(slot.size(0)), static_cast<int>(a.size(1)),
                    out.data_ptr<float>(), stream_of(a));
    after_launch();
  }
  return out;
}

// ------------------------------------------------------------------------- linear -> logprob
std::vector<int64_t> linear_logp_workspace_shape(int64_t n_tokens, int64_t v_local, int64_t world) {
  int items = 0, n_pad = 0, tiles_m = 0;
  rlk::linear_logp_workspace_shape(static_cast<int>(n_tokens), static_cast<int>(v_local), static_cast<int>(world), &items,
                                   &n_pad, &tiles_m);
  return {items, n_pad, tiles_m};
}

std::vector<Tensor> linear_logp_fwd(const Tensor& hidden, const Tensor& weight, const Tensor& target,
                                    std::optional<Tensor> bias, int64_t vocab_start, int64_t rank, int64_t world,
                                    int64_t slot_base, int64_t total_records, std::vector<int64_t> peer_partials, std::vector<int64_t> peer_counters,
                                    int64_t next_counters, int64_t counter_capacity, bool want_lse,
                                    bool want_entropy, double wait_limit_ms, int64_t global_vocab) {
  check_rowmajor(hidden, "hidden");
  check_rowmajor(weight, "weight");
  check_cuda(target, "target");
  TORCH_CHECK(hidden.scalar_type() == torch::kBFloat16 && weight.scalar_type() == torch::kBFloat16,
              "rl_engine.linear_logp: bf16 hidden and weight only");
  TORCH_CHECK(target.scalar_type() == torch::kInt64 && target.is_contiguous() && target.numel() == hidden.size(0),
              "rl_engine.linear_logp: target must be contiguous int64 [N]");
  TORCH_CHECK(hidden.size(1) == weight.size(1), "rl_engine.linear_logp: hidden dim mismatch");
  TORCH_CHECK(hidden.stride(0) % 8 == 0 && weight.stride(0) % 8 == 0, "rl_engine.linear_logp: row pitch must be a multiple of 8");
  TORCH_CHECK(world >= 1 && world <= 8 && rank >= 0 && rank < world, "rl_engine.linear_logp: bad rank/world");
  TORCH_CHECK(static_cast<int64_t>(peer_partials.size()) == world && static_cast<int64_t>(peer_counters.size()) == world,
              "rl_engine.linear_logp: need one partial buffer and one counter array per rank");
  const c10::cuda::CUDAGuard guard(hidden.device());
  const int64_t n = hidden.size(0);
  auto fopt = hidden.options().dtype(torch::kFloat32);
  Tensor logp = torch::empty({n}, fopt);
  Tensor lse = want_lse ? torch::empty({n}, fopt) : Tensor();
  Tensor ent = want_entropy ? torch::empty({n}, fopt) : Tensor();
  Tensor bias_f;
  if (bias.has_value() && bias->defined()) {
    bias_f = bias->to(torch::kFloat32).contiguous();
    TORCH_CHECK(bias_f.numel() == weight.size(0), "rl_engine.linear_logp: bias must have V_local elements");
  }
  if (n == 0) return {logp, lse, ent};
  rlk::LinearLogpFwdArgs a{};
  a.hidden = reinterpret_cast<const __nv_bfloat16*>(hidden.data_ptr());
  a.weight = reinterpret_cast<const __nv_bfloat16*>(weight.data_ptr());
  a.target = target.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(target.data_ptr<int64_t>()) : nullptr;
  a.bias = bias_f.defined() ? bias_f.data_ptr<float>() : nullptr;
  a.n_tokens = static_cast<int>(n);
  a.hidden_dim = static_cast<int>(hidden.size(1));
  a.v_local = static_cast<int>(weight.size(0));
  a.ld_hidden = hidden.stride(0);
  a.ld_weight = weight.stride(0);
  a.vocab_start = vocab_start;
  a.global_vocab = global_vocab;
  a.rank = static_cast<int>(rank);
  a.world = static_cast<int>(world);
  a.slot_base = static_cast<int>(slot_base);
  a.total_records = static_cast<int>(total_records);
  for (int r = 0; r < world; ++r) {
    a.peer_partials[r] = reinterpret_cast<void*>(peer_partials[r]);
    a.peer_counters[r] = reinterpret_cast<unsigned int*>(peer_counters[r]);
  }
  a.next_counters = reinterpret_cast<unsigned int*>(next_counters);
  a.counter_capacity = static_cast<int>(counter_capacity);
  a.logp = logp.data_ptr<float>();
  a.lse = want_lse ? lse.data_ptr<float>() : nullptr;
  a.entropy = want_entropy ? ent.data_ptr<float>() : nullptr;
  a.sm_count = sm_count_of(hidden.get_device());
  a.err = err_ptr(hidden);
  a.wait_limit_ns = static_cast<unsigned long long>(wait_limit_ms * 1e6);
  rlk::linear_logp_forward(a, stream_of(hidden));
  after_launch();
  return {logp, lse, ent};
}

void linear_logp_dz(const Tensor& hidden, const Tensor& weight, const Tensor& target, std::optional<Tensor> bias,
                    const Tensor& lse, const Tensor& grad, int64_t vocab_start, Tensor dz) {
  check_rowmajor(hidden, "hidden");
  check_rowmajor(weight, "weight");
  check_rowmajor(dz, "dz");
  TORCH_CHECK(dz.scalar_type() == torch::kBFloat16 && dz.size(0) >= hidden.size(0) && dz.size(1) == weight.size(0),
              "rl_engine.linear_logp_dz: dz must be bf16 [>=N, V_local]");
  TORCH_CHECK(dz.stride(0) % 8 == 0, "rl_engine.linear_logp_dz: dz row pitch must be a multiple of 8");
  TORCH_CHECK(lse.scalar_type() == torch::kFloat32 && grad.scalar_type() == torch::kFloat32 && lse.is_contiguous() &&
                  grad.is_contiguous(),
              "rl_engine.linear_logp_dz: lse and grad must be contiguous float32");
  TORCH_CHECK(target.scalar_type() == torch::kInt64 && target.is_contiguous(), "target must be contiguous int64");
  const c10::cuda::CUDAGuard guard(hidden.device());
  if (hidden.size(0) == 0) return;
  Tensor bias_f;
  if (bias.has_value() && bias->defined()) bias_f = bias->to(torch::kFloat32).contiguous();
  rlk::LinearLogpDzArgs a{};
  a.hidden = reinterpret_cast<const __nv_bfloat16*>(hidden.data_ptr());
  a.weight = reinterpret_cast<const __nv_bfloat16*>(weight.data_ptr());
  a.target = reinterpret_cast<const long long*>(target.data_ptr<int64_t>());
  a.bias = bias_f.defined() ? bias_f.data_ptr<float>() : nullptr;
  a.lse = lse.data_ptr<float>();
  a.grad = grad.data_ptr<float>();
  a.n_tokens = static_cast<int>(hidden.size(0));
  a.hidden_dim = static_cast<int>(hidden.size(1));
  a.v_local = static_cast<int>(weight.size(0));
  a.ld_hidden = hidden.stride(0);
  a.ld_weight = weight.stride(0);
  a.vocab_start = vocab_start;
  a.dz = reinterpret_cast<__nv_bfloat16*>(dz.data_ptr());
  a.ld_dz = dz.stride(0);
  a.sm_count = sm_count_of(hidden.get_device());
  a.err = err_ptr(hidden);
  rlk::linear_logp_dz(a, stream_of(hidden));
  after_launch();
}

// --------------------------------------------------------------------------- logp over logits
void logp_rows(const Tensor& logits, const Tensor& ids, std::optional<Tensor> row_indices, Tensor out) {
  check_rowmajor(logits, "logits");
  check_cuda(out, "out");
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == torch::kInt64 && ids.is_contiguous() && ids.numel() == logits.size(0),
              "rl_engine.logp_rows: ids must be contiguous int64 [rows]");
  TORCH_CHECK(out.is_contiguous() && out.numel() == logits.size(0), "rl_engine.logp_rows: out must be contiguous [rows]");
  const c10::cuda::CUDAGuard guard(logits.device());
  rlk::LogpRowsArgs a{};
  a.logits = logits.data_ptr();
  a.ld = logits.stride(0);
  a.in_dtype = dtype_code(logits);
  a.ids = reinterpret_cast<const long long*>(ids.data_ptr<int64_t>());
  a.row_indices = nullptr;
  a.launch_rows = static_cast<int>(logits.size(0));
  if (row_indices.has_value() && row_indices->defined()) {
    TORCH_CHECK(row_indices->is_cuda() && row_indices->scalar_type() == torch::kInt64 && row_indices->is_contiguous(),
                "rl_engine.logp_rows: row_indices must be contiguous int64 on the GPU");
    a.row_indices = reinterpret_cast<const long long*>(row_indices->data_ptr<int64_t>());
    a.launch_rows = static_cast<int>(row_indices->numel());
  }
  a.V = static_cast<int>(logits.size(1));
  a.total_rows = logits.size(0);
  a.out = out.data_ptr();
  a.out_dtype = dtype_code(out);
  if (a.launch_rows == 0) return;
  rlk::logp_rows(a, stream_of(logits));
  after_launch();
}

std::vector<Tensor> ratio_kl_fwd(const Tensor& policy, std::optional<Tensor> ref_opt, const Tensor& ids,
                                 const Tensor& mask, const Tensor& old_logp) {
  check_rowmajor(policy, "policy_logits");
  const bool has_ref = ref_opt.has_value() && ref_opt->defined();
  Tensor ref = has_ref ? *ref_opt : policy;
  check_rowmajor(ref, "ref_logits");
  TORCH_CHECK(policy.scalar_type() == ref.scalar_type() && policy.sizes() == ref.sizes(), "policy/ref logits must match");
  const int64_t rows = policy.size(0);
  TORCH_CHECK(ids.scalar_type() == torch::kInt64 && ids.is_contiguous() && ids.numel() == rows, "ids: int64 [rows]");
  TORCH_CHECK(mask.scalar_type() == torch::kBool && mask.is_contiguous() && mask.numel() == rows, "mask: bool [rows]");
  TORCH_CHECK(old_logp.scalar_type() == torch::kFloat32 && old_logp.is_contiguous() && old_logp.numel() == rows,
              "old_logps: float32 [rows]");
  const c10::cuda::CUDAGuard guard(policy.device());
  auto fopt = policy.options().dtype(torch::kFloat32);
  Tensor ratio = torch::empty({rows}, fopt), kl = torch::empty({rows}, fopt), d = torch::empty({rows}, fopt),
         lse = torch::empty({rows}, fopt), lp = torch::empty({rows}, fopt);
  Tensor bad = torch::zeros({1}, policy.options().dtype(torch::kInt32));
  rlk::RatioKlFwdArgs a{};
  a.policy = policy.data_ptr();
  a.ref = has_ref ? ref.data_ptr() : nullptr;
  a.ld_policy = policy.stride(0);
  a.ld_ref = ref.stride(0);
  a.dtype = dtype_code(policy);
  a.ids = reinterpret_cast<const long long*>(ids.data_ptr<int64_t>());
  a.mask = reinterpret_cast<const unsigned char*>(mask.data_ptr<bool>());
  a.old_logp = old_logp.data_ptr<float>();
  a.rows = static_cast<int>(rows);
  a.V = static_cast<int>(policy.size(1));
  a.ratio = ratio.data_ptr<float>();
  a.kl = kl.data_ptr<float>();
  a.save_d = d.data_ptr<float>();
  a.save_lse = lse.data_ptr<float>();
  a.save_lp = lp.data_ptr<float>();
  a.bad_id_flag = reinterpret_cast<unsigned int*>(bad.data_ptr<int>());
  if (rows) {
    rlk::ratio_kl_forward(a, stream_of(policy));
    after_launch();
  }
  return {ratio, kl, d, lse, bad, lp};
}

Tensor ratio_kl_bwd(const Tensor& policy, const Tensor& ids, const Tensor& mask, const Tensor& g_ratio,
                    const Tensor& g_kl, const Tensor& ratio, const Tensor& d, const Tensor& lse) {
  check_rowmajor(policy, "policy_logits");
  const c10::cuda::CUDAGuard guard(policy.device());
  Tensor grad = torch::empty({policy.size(0), policy.size(1)}, policy.options());
  rlk::RatioKlBwdArgs a{};
  a.policy = policy.data_ptr();
  a.ld_policy = policy.stride(0);
  a.dtype = dtype_code(policy);
  a.ids = reinterpret_cast<const long long*>(ids.data_ptr<int64_t>());
  a.mask = reinterpret_cast<const unsigned char*>(mask.data_ptr<bool>());
  Tensor gr = g_ratio.to(torch::kFloat32).contiguous(), gk = g_kl.to(torch::kFloat32).contiguous();
  a.g_ratio = gr.data_ptr<float>();
  a.g_kl = gk.data_ptr<float>();
  a.ratio = ratio.data_ptr<float>();
  a.save_d = d.data_ptr<float>();
  a.save_lse = lse.data_ptr<float>();
  a.rows = static_cast<int>(policy.size(0));
  a.V = static_cast<int>(policy.size(1));
  a.grad = grad.data_ptr();
  a.ld_grad = grad.stride(0);
  if (a.rows) {
    rlk::ratio_kl_backward(a, stream_of(policy));
    after_launch();
  }
  return grad;
}

// ------------------------------------------------------------------------------- RL losses
Tensor group_advantages(const Tensor& rewards, std::optional<Tensor> bounds, int64_t uniform, double eps) {
  check_cuda(rewards, "rewards");
  TORCH_CHECK(rewards.scalar_type() == torch::kFloat32 && rewards.is_contiguous(), "rewards: contiguous float32");
  const c10::cuda::CUDAGuard guard(rewards.device());
  Tensor adv = torch::empty_like(rewards);
  const long long* bptr = nullptr;
  int64_t groups = 0;
  if (bounds.has_value() && bounds->defined()) {
    TORCH_CHECK(bounds->is_cuda() && bounds->scalar_type() == torch::kInt64 && bounds->is_contiguous(), "bounds: int64 GPU");
    bptr = reinterpret_cast<const long long*>(bounds->data_ptr<int64_t>());
    groups = bounds->numel() - 1;
  } else {
    TORCH_CHECK(uniform > 0 && rewards.numel() % uniform == 0, "uniform group size must divide the number of rewards");
    groups = rewards.numel() / uniform;
  }
  if (groups > 0) {
    rlk::group_advantages(rewards.data_ptr<float>(), bptr, static_cast<int>(groups), uniform, static_cast<float>(eps),
                          adv.data_ptr<float>(), rewards.numel(), stream_of(rewards));
    after_launch();
  }
  return adv;
}

std::vector<Tensor> surrogate_fwd(const Tensor& logp, std::optional<Tensor> ref_logp, const Tensor& old_logp,
                                  std::optional<Tensor> adv_seq, std::optional<Tensor> adv_tok, const Tensor& mask,
                                  int64_t T, double clip_eps, double beta, bool want_terms) {
  check_cuda(logp, "logp");
  auto f32c = [](const Tensor& t, const char* n) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.is_contiguous(), n, ": contiguous float32 on GPU");
  };
  f32c(logp, "logp");
  f32c(old_logp, "old_logps");
  TORCH_CHECK(mask.is_cuda() && mask.scalar_type() == torch::kBool && mask.is_contiguous() && mask.numel() == logp.numel(),
              "mask: contiguous bool, same size as logp");
  const c10::cuda::CUDAGuard guard(logp.device());
  const int64_t n = logp.numel();
  auto fopt = logp.options();
  Tensor d_pl = torch::empty({n}, fopt), d_kl = torch::empty({n}, fopt);
  Tensor ratio = want_terms ? torch::empty({n}, fopt) : Tensor();
  Tensor kl = want_terms ? torch::empty({n}, fopt) : Tensor();
  Tensor partials = torch::empty({rlk::surrogate_partial_floats()}, fopt);
  Tensor out4 = torch::empty({4}, fopt);
  rlk::SurrogateFwdArgs a{};
  a.logp = logp.data_ptr<float>();
  a.ref_logp = nullptr;
  if (ref_logp.has_value() && ref_logp->defined()) {
    f32c(*ref_logp, "ref_logps");
    a.ref_logp = ref_logp->data_ptr<float>();
  }
  a.old_logp = old_logp.data_ptr<float>();
  a.adv_seq = nullptr;
  a.adv_tok = nullptr;
  if (adv_tok.has_value() && adv_tok->defined()) {
    f32c(*adv_tok, "advantages");
    TORCH_CHECK(adv_tok->numel() == n, "per-token advantages must match logp");
    a.adv_tok = adv_tok->data_ptr<float>();
  } else {
    TORCH_CHECK(adv_seq.has_value() && adv_seq->defined(), "need per-sequence or per-token advantages");
    f32c(*adv_seq, "sample_advantages");
    TORCH_CHECK(T > 0 && adv_seq->numel() * T == n, "per-sequence advantages must have n / T entries");
    a.adv_seq = adv_seq->data_ptr<float>();
  }
  a.mask = reinterpret_cast<const unsigned char*>(mask.data_ptr<bool>());
  a.n = n;
  a.T = T > 0 ? T : 1;
  a.clip_eps = static_cast<float>(clip_eps);
  a.beta = static_cast<float>(beta);
  a.d_pl = d_pl.data_ptr<float>();
  a.d_kl = d_kl.data_ptr<float>();
  a.ratio_out = want_terms ? ratio.data_ptr<float>() : nullptr;
  a.kl_out = want_terms ? kl.data_ptr<float>() : nullptr;
  a.partials = partials.data_ptr<float>();
  a.out4 = out4.data_ptr<float>();
  rlk::surrogate_forward(a, stream_of(logp));
  after_launch(2);
  return {out4, d_pl, d_kl, ratio, kl};
}

Tensor surrogate_bwd(const Tensor& d_pl, const Tensor& d_kl, const Tensor& out4, const Tensor& g3, double beta) {
  const c10::cuda::CUDAGuard guard(d_pl.device());
  Tensor grad = torch::empty_like(d_pl);
  Tensor g = g3.to(torch::kFloat32).contiguous();
  rlk::surrogate_backward(d_pl.data_ptr<float>(), d_kl.data_ptr<float>(), out4.data_ptr<float>(), g.data_ptr<float>(),
                          static_cast<float>(beta), d_pl.numel(), grad.data_ptr<float>(), stream_of(d_pl));
  after_launch();
  return grad;
}

std::vector<Tensor> dpo_fwd(const Tensor& pc, const Tensor& pr, const Tensor& rc, const Tensor& rr, double beta,
                            double label_smoothing) {
  const c10::cuda::CUDAGuard guard(pc.device());
  auto prep = [](const Tensor& t) { return t.to(torch::kFloat32).contiguous().view({-1}); };
  Tensor a = prep(pc), b = prep(pr), c = prep(rc), d = prep(rr);
  const int64_t n = a.numel();
  TORCH_CHECK(b.numel() == n && c.numel() == n && d.numel() == n, "dpo: all four log-prob vectors must match");
  Tensor loss = torch::zeros({1}, a.options()), cr = torch::empty({n}, a.options()), rj = torch::empty({n}, a.options()),
         dh = torch::empty({n}, a.options());
  rlk::dpo_forward(a.data_ptr<float>(), b.data_ptr<float>(), c.data_ptr<float>(), d.data_ptr<float>(),
                   static_cast<int>(n), static_cast<float>(beta), static_cast<float>(label_smoothing),
                   loss.data_ptr<float>(), cr.data_ptr<float>(), rj.data_ptr<float>(), dh.data_ptr<float>(), stream_of(a));
  after_launch();
  return {loss, cr, rj, dh};
}

// ------------------------------------------------------------------------------ model ops
std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const Tensor& w, double eps, bool out_fp32, bool save_rstd) {
  check_rowmajor(x, "x");
  TORCH_CHECK(w.is_cuda() && w.is_contiguous() && w.numel() == x.size(1), "weight must be contiguous [D]");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty({x.size(0), x.size(1)}, x.options().dtype(out_fp32 ? torch::kFloat32 : x.scalar_type()));
  Tensor rstd = save_rstd ? torch::empty({x.size(0)}, x.options().dtype(torch::kFloat32)) : Tensor();
  if (x.size(0)) {
    rlk::rmsnorm_forward(x.data_ptr(), x.stride(0), dtype_code(x), w.data_ptr(), dtype_code(w), y.data_ptr(), y.stride(0),
                         out_fp32, x.size(0), static_cast<int>(x.size(1)), static_cast<float>(eps),
                         save_rstd ? rstd.data_ptr<float>() : nullptr, stream_of(x));
    after_launch();
  }
  return {y, rstd};
}

void check_qk_norm(const Tensor& qkv, const Tensor& wq, const Tensor& wk, int64_t hq, int64_t hkv, const char* who) {
  check_rowmajor(qkv, who);
  TORCH_CHECK(qkv.scalar_type() == torch::kBFloat16 && hq >= 1 && hkv >= 1 && qkv.size(1) == (hq + 2 * hkv) * 128 &&
                  qkv.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(qkv.data_ptr()) % 16 == 0,
              "qk_norm: ", who, " must be 16-byte aligned bf16 [tokens, (hq + 2 hkv) * 128]");
  for (const Tensor* w : {&wq, &wk})
    TORCH_CHECK(w->is_cuda() && w->scalar_type() == torch::kBFloat16 && w->is_contiguous() && w->numel() == 128 &&
                    reinterpret_cast<uintptr_t>(w->data_ptr()) % 16 == 0 && w->device() == qkv.device(),
                "qk_norm: the norm weights must be 16-byte aligned contiguous bf16 [128] on the buffer's device");
}

// Per-head RMSNorm of the q and k heads of a packed qkv buffer (head_dim 128), v copied: one launch.
Tensor qk_norm_fwd(const Tensor& qkv, const Tensor& wq, const Tensor& wk, int64_t hq, int64_t hkv, double eps) {
  check_qk_norm(qkv, wq, wk, hq, hkv, "qkv");
  const c10::cuda::CUDAGuard guard(qkv.device());
  Tensor out = torch::empty({qkv.size(0), qkv.size(1)}, qkv.options());
  if (qkv.size(0)) {
    rlk::qk_norm_forward(reinterpret_cast<const __nv_bfloat16*>(qkv.data_ptr()), qkv.stride(0),
                         reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), out.stride(0),
                         reinterpret_cast<const __nv_bfloat16*>(wq.data_ptr()),
                         reinterpret_cast<const __nv_bfloat16*>(wk.data_ptr()), qkv.size(0), static_cast<int>(hq),
                         static_cast<int>(hkv), static_cast<float>(eps), stream_of(qkv));
    after_launch();
  }
  return out;
}

// (dqkv, dwq, dwk) from the gradient of qk_norm_fwd's output; the weight gradients are summed over the blocks' partial
// sums in block order (fp32) and returned in bf16.
std::vector<Tensor> qk_norm_bwd(const Tensor& qkv, const Tensor& dout, const Tensor& wq, const Tensor& wk, int64_t hq,
                                int64_t hkv, double eps) {
  check_qk_norm(qkv, wq, wk, hq, hkv, "qkv");
  check_qk_norm(dout, wq, wk, hq, hkv, "dout");
  TORCH_CHECK(dout.size(0) == qkv.size(0) && dout.device() == qkv.device(), "qk_norm_bwd: dout must match qkv");
  const c10::cuda::CUDAGuard guard(qkv.device());
  Tensor dqkv = torch::empty({qkv.size(0), qkv.size(1)}, qkv.options());
  const int blocks = rlk::qk_norm_blocks(qkv.size(0), static_cast<int>(hq + 2 * hkv));
  Tensor part = torch::zeros({blocks, 2, 128}, qkv.options().dtype(torch::kFloat32));
  if (qkv.size(0)) {
    rlk::qk_norm_backward(reinterpret_cast<const __nv_bfloat16*>(qkv.data_ptr()), qkv.stride(0),
                          reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr()), dout.stride(0),
                          reinterpret_cast<__nv_bfloat16*>(dqkv.data_ptr()), dqkv.stride(0),
                          reinterpret_cast<const __nv_bfloat16*>(wq.data_ptr()),
                          reinterpret_cast<const __nv_bfloat16*>(wk.data_ptr()), qkv.size(0), static_cast<int>(hq),
                          static_cast<int>(hkv), static_cast<float>(eps), part.data_ptr<float>(), stream_of(qkv));
    after_launch();
  }
  Tensor dw = part.sum(0);
  return {dqkv, dw[0].to(torch::kBFloat16), dw[1].to(torch::kBFloat16)};
}

std::vector<Tensor> rmsnorm_bwd(const Tensor& x, const Tensor& w, const Tensor& dy, const Tensor& rstd) {
  check_rowmajor(x, "x");
  check_rowmajor(dy, "dy");
  TORCH_CHECK(dy.scalar_type() == x.scalar_type(), "dy dtype must match x");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0), D = x.size(1);
  Tensor dx = torch::empty({rows, D}, x.options());
  Tensor dw = torch::zeros({D}, w.options());
  if (rows) {
    Tensor part = torch::empty({rlk::rmsnorm_bwd_chunks(rows), D}, x.options().dtype(torch::kFloat32));
    rlk::rmsnorm_backward(x.data_ptr(), x.stride(0), dtype_code(x), w.data_ptr(), dtype_code(w), dy.data_ptr(),
                          dy.stride(0), rstd.data_ptr<float>(), dx.data_ptr(), dx.stride(0), rows, static_cast<int>(D),
                          part.data_ptr<float>(), dw.data_ptr(), stream_of(x));
    after_launch(2);
  }
  return {dx, dw};
}

Tensor swiglu_fwd(const Tensor& gate, std::optional<Tensor> up, bool out_fp32) {
  check_rowmajor(gate, "gate");
  const c10::cuda::CUDAGuard guard(gate.device());
  const bool has_up = up.has_value() && up->defined();
  if (has_up) {
    check_rowmajor(*up, "up");
    TORCH_CHECK(up->sizes() == gate.sizes() && up->scalar_type() == gate.scalar_type(), "gate/up must match");
  }
  Tensor out = torch::empty({gate.size(0), gate.size(1)}, gate.options().dtype(out_fp32 ? torch::kFloat32 : gate.scalar_type()));
  if (gate.numel()) {
    rlk::swiglu_forward(gate.data_ptr(), gate.stride(0), has_up ? up->data_ptr() : nullptr, has_up ? up->stride(0) : 0,
                        dtype_code(gate), out.data_ptr(), out.stride(0), out_fp32, gate.size(0),
                        static_cast<int>(gate.size(1)), stream_of(gate));
    after_launch();
  }
  return out;
}

std::vector<Tensor> swiglu_bwd(const Tensor& gate, std::optional<Tensor> up, const Tensor& dy) {
  check_rowmajor(gate, "gate");
  check_rowmajor(dy, "dy");
  TORCH_CHECK(dy.scalar_type() == gate.scalar_type(), "dy dtype must match gate");
  const c10::cuda::CUDAGuard guard(gate.device());
  const bool has_up = up.has_value() && up->defined();
  Tensor dg = torch::empty({gate.size(0), gate.size(1)}, gate.options());
  Tensor du = has_up ? torch::empty({gate.size(0), gate.size(1)}, gate.options()) : Tensor();
  if (gate.numel()) {
    rlk::swiglu_backward(gate.data_ptr(), gate.stride(0), has_up ? up->data_ptr() : nullptr, has_up ? up->stride(0) : 0,
                         dy.data_ptr(), dy.stride(0), dtype_code(gate), dg.data_ptr(), dg.stride(0),
                         has_up ? du.data_ptr() : nullptr, has_up ? du.stride(0) : 0, gate.size(0),
                         static_cast<int>(gate.size(1)), stream_of(gate));
    after_launch();
  }
  return {dg, du};
}

Tensor swiglu_packed_fwd(const Tensor& gu) {
  check_rowmajor(gu, "gate_up");
  TORCH_CHECK(gu.scalar_type() == torch::kBFloat16 && gu.size(1) % 16 == 0 && gu.stride(0) % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(gu.data_ptr()) % 16 == 0,
              "swiglu_packed: bf16 [rows, 2F] with F % 8 == 0 and 16-byte aligned rows");
  const c10::cuda::CUDAGuard guard(gu.device());
  const int64_t F = gu.size(1) / 2;
  Tensor out = torch::empty({gu.size(0), F}, gu.options());
  if (gu.numel()) {
    rlk::swiglu_packed_forward(reinterpret_cast<const __nv_bfloat16*>(gu.data_ptr()), gu.stride(0),
                               reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), out.stride(0), gu.size(0),
                               static_cast<int>(F), stream_of(gu));
    after_launch();
  }
  return out;
}

Tensor swiglu_packed_bwd(const Tensor& gu, const Tensor& dy) {
  check_rowmajor(gu, "gate_up");
  check_rowmajor(dy, "dy");
  TORCH_CHECK(dy.scalar_type() == torch::kBFloat16 && dy.size(0) == gu.size(0) && dy.size(1) * 2 == gu.size(1) &&
                  dy.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(dy.data_ptr()) % 16 == 0,
              "swiglu_packed_bwd: dy must be aligned bf16 [rows, F]");
  const c10::cuda::CUDAGuard guard(gu.device());
  Tensor dgu = torch::empty({gu.size(0), gu.size(1)}, gu.options());
  if (gu.numel()) {
    rlk::swiglu_packed_backward(reinterpret_cast<const __nv_bfloat16*>(gu.data_ptr()), gu.stride(0),
                                reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr()), dy.stride(0),
                                reinterpret_cast<__nv_bfloat16*>(dgu.data_ptr()), dgu.stride(0), gu.size(0),
                                static_cast<int>(gu.size(1) / 2), stream_of(gu));
    after_launch();
  }
  return dgu;
}

// x: [tokens, heads, D] with unit stride on D and stride D on heads
Tensor rope(const Tensor& x, const Tensor& positions, const Tensor& cos_t, const Tensor& sin_t, bool inverse,
            std::optional<Tensor> out_opt) {
  check_cuda(x, "x");
  TORCH_CHECK(x.dim() == 3 && x.stride(2) == 1 && x.stride(1) == x.size(2), "rope: x must be [tokens, heads, D] with packed heads");
  TORCH_CHECK(positions.is_cuda() && positions.scalar_type() == torch::kInt64 && positions.is_contiguous() &&
                  positions.numel() == x.size(0),
              "rope: positions must be contiguous int64 [tokens]");
  TORCH_CHECK(cos_t.scalar_type() == torch::kFloat32 && sin_t.scalar_type() == torch::kFloat32 && cos_t.is_contiguous() &&
                  sin_t.is_contiguous() && cos_t.size(-1) == x.size(2) / 2,
              "rope: cos/sin tables must be contiguous float32 [max_pos, D/2]");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor out;
  if (out_opt.has_value() && out_opt->defined()) {
    out = *out_opt;
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == x.scalar_type() && out.dim() == 3 && out.size(0) == x.size(0) &&
                    out.size(1) == x.size(1) && out.size(2) == x.size(2) && out.stride(2) == 1 &&
                    out.stride(1) == out.size(2),
                "rope: out must match x with packed heads");
  } else {
    out = torch::empty({x.size(0), x.size(1), x.size(2)}, x.options());
  }
  if (x.numel()) {
    rlk::rope_apply(x.data_ptr(), x.stride(0), dtype_code(x), reinterpret_cast<const long long*>(positions.data_ptr<int64_t>()),
                    cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), out.data_ptr(), out.stride(0), x.size(0),
                    static_cast<int>(x.size(1)), static_cast<int>(x.size(2)), inverse, cos_t.size(0), stream_of(x));
    after_launch();
  }
  return out;
}

// Decoding with packed queries: merge the prefix part and the own-keys part of the attention by log-sum-exp.
Tensor attn_merge2(const Tensor& o1, const Tensor& l1, const Tensor& o2, const Tensor& l2, int64_t rep) {
  check_cuda(o1, "o1");
  TORCH_CHECK(o1.scalar_type() == torch::kBFloat16 && o2.scalar_type() == torch::kBFloat16 && o1.dim() == 3 &&
                  o1.size(2) == 128 && o1.is_contiguous() && o2.is_contiguous() && o1.sizes() == o2.sizes(),
              "rl_engine.attn_merge2: o1 / o2 must be contiguous bf16 [rows, heads, 128]");
  const int64_t rows = o1.size(0), hkv = o1.size(1);
  auto ok = [&](const Tensor& l) {
    return l.is_cuda() && l.scalar_type() == torch::kFloat32 && l.is_contiguous() && l.dim() == 2 && l.size(0) == hkv &&
           l.size(1) == rows;
  };
  TORCH_CHECK(ok(l1) && ok(l2), "rl_engine.attn_merge2: l1 / l2 must be contiguous float32 [heads, rows]");
  TORCH_CHECK(rep >= 1 && rows % rep == 0, "rl_engine.attn_merge2: rows must be a multiple of rep");
  const c10::cuda::CUDAGuard guard(o1.device());
  Tensor out = torch::empty({rows / rep, hkv * rep * 128}, o1.options());
  if (rows) {
    rlk::attn_merge2(o1.data_ptr(), l1.data_ptr<float>(), o2.data_ptr(), l2.data_ptr<float>(), out.data_ptr(), rows,
                     static_cast<int>(hkv), static_cast<int>(rep), stream_of(o1));
    after_launch();
  }
  return out;
}

Tensor embedding_fwd(const Tensor& ids, const Tensor& table) {
  check_rowmajor(table, "weight");
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == torch::kInt64 && ids.is_contiguous(), "ids: contiguous int64 GPU");
  const c10::cuda::CUDAGuard guard(table.device());
  Tensor out = torch::empty({ids.numel(), table.size(1)}, table.options());
  if (ids.numel()) {
    rlk::embedding_forward(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), table.data_ptr(), table.stride(0),
                           dtype_code(table), out.data_ptr(), ids.numel(), static_cast<int>(table.size(1)), table.size(0),
                           stream_of(table));
    after_launch();
  }
  return out;
}

// seg_ids [S], seg_start [S+1], order [tokens]: tokens stably sorted by id and run-length encoded.
void embedding_bwd(const Tensor& seg_ids, const Tensor& seg_start, const Tensor& order, const Tensor& dy, Tensor dtable) {
  check_rowmajor(dy, "dy");
  check_rowmajor(dtable, "dtable");
  TORCH_CHECK(dy.is_contiguous(), "dy must be contiguous");
  const c10::cuda::CUDAGuard guard(dy.device());
  const int64_t segs = seg_ids.numel();
  if (segs == 0) return;
  const bool tfp32 = dtable.scalar_type() == torch::kFloat32;
  TORCH_CHECK(tfp32 || dtable.scalar_type() == dy.scalar_type(), "dtable must be float32 or match dy");
  rlk::embedding_backward(reinterpret_cast<const long long*>(seg_ids.data_ptr<int64_t>()),
                          reinterpret_cast<const long long*>(seg_start.data_ptr<int64_t>()), segs,
                          reinterpret_cast<const long long*>(order.data_ptr<int64_t>()), dy.data_ptr(), dtype_code(dy),
                          static_cast<int>(dy.size(1)), dtable.data_ptr(), tfp32, dtable.stride(0), dy.size(0),
                          dtable.size(0), stream_of(dy));
  after_launch();
}

void adamw(Tensor p, std::optional<Tensor> master, const Tensor& g, Tensor m, Tensor v, double lr, double b1, double b2,
           double eps, double wd, int64_t step, double grad_scale) {
  check_cuda(p, "param");
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adamw: contiguous tensors");
  TORCH_CHECK(m.scalar_type() == torch::kFloat32 && v.scalar_type() == torch::kFloat32, "adamw: fp32 moments");
  TORCH_CHECK(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel(), "adamw: size mismatch");
  const c10::cuda::CUDAGuard guard(p.device());
  float* mp = nullptr;
  short* rp = nullptr;
  if (master.has_value() && master->defined()) {
    TORCH_CHECK(master->is_cuda() && master->is_contiguous() && master->numel() == p.numel(),
                "adamw: master must be a contiguous CUDA tensor of the parameter's size");
    if (master->scalar_type() == torch::kInt16) {  // 16-bit residuals of a bf16 parameter
      TORCH_CHECK(p.scalar_type() == torch::kBFloat16, "adamw: int16 residual masters need bfloat16 parameters");
      rp = reinterpret_cast<short*>(master->data_ptr<int16_t>());
    } else {
      TORCH_CHECK(master->scalar_type() == torch::kFloat32, "adamw: master must be float32 or int16 residuals");
      mp = master->data_ptr<float>();
    }
  }
  const float bc1 = 1.f - static_cast<float>(std::pow(b1, static_cast<double>(step)));
  const float bc2 = 1.f - static_cast<float>(std::pow(b2, static_cast<double>(step)));
  if (p.numel()) {
    rlk::adamw_step(p.data_ptr(), dtype_code(p), mp, rp, g.data_ptr(), dtype_code(g), m.data_ptr<float>(), v.data_ptr<float>(),
                    p.numel(), static_cast<float>(lr), static_cast<float>(b1), static_cast<float>(b2),
                    static_cast<float>(eps), static_cast<float>(wd), bc1, bc2, static_cast<float>(grad_scale), stream_of(p));
    after_launch();
  }
}

// ---------------------------------------------------------------------------------- sampler
std::vector<Tensor> sample(const Tensor& logits, int64_t top_k, double top_p, double temperature, int64_t seed,
                           int64_t offset, bool want_logprob) {
  check_rowmajor(logits, "logits");
  // top_k == 0 selects the full-vocabulary nucleus kernel (top-p only / plain temperature sampling)
  TORCH_CHECK(top_k >= 0 && top_k <= rlk::sample_topk_limit(), "rl_engine.sample: top_k must be in [0, ",
              rlk::sample_topk_limit(), "] (0 = no top-k)");
  TORCH_CHECK(top_p > 0.0 && top_p <= 1.0, "rl_engine.sample: top_p must be in (0, 1]");
  TORCH_CHECK(temperature > 0.0, "rl_engine.sample: temperature must be positive");
  const c10::cuda::CUDAGuard guard(logits.device());
  Tensor ids = torch::empty({logits.size(0)}, logits.options().dtype(torch::kInt64));
  Tensor lp = want_logprob ? torch::empty({logits.size(0)}, logits.options().dtype(torch::kFloat32)) : Tensor();
  if (logits.size(0) && top_k == 0) {
    rlk::sample_nucleus(logits.data_ptr(), logits.stride(0), dtype_code(logits), static_cast<int>(logits.size(0)),
                        static_cast<int>(logits.size(1)), static_cast<float>(top_p), static_cast<float>(temperature),
                        static_cast<unsigned long long>(seed), static_cast<unsigned long long>(offset),
                        reinterpret_cast<long long*>(ids.data_ptr<int64_t>()), want_logprob ? lp.data_ptr<float>() : nullptr,
                        stream_of(logits));
    after_launch();
  } else if (logits.size(0)) {
    rlk::sample_topk_topp(logits.data_ptr(), logits.stride(0), dtype_code(logits), static_cast<int>(logits.size(0)),
                          static_cast<int>(logits.size(1)), static_cast<int>(top_k), static_cast<float>(top_p),
                          static_cast<float>(temperature), static_cast<unsigned long long>(seed),
                          static_cast<unsigned long long>(offset), reinterpret_cast<long long*>(ids.data_ptr<int64_t>()),
                          want_logprob ? lp.data_ptr<float>() : nullptr, stream_of(logits));
    after_launch();
  }
  return {ids, lp};
}

// -------------------------------------------------------------------------------- attention
std::vector<Tensor> attention_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& seqs,
                                  const Tensor& tiles, bool causal, double softmax_scale, bool want_lse) {
  auto check3 = [](const Tensor& t, const char* n) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 3 && t.size(2) == 128 &&
                    t.stride(2) == 1 && t.stride(1) == 128,
                "rl_engine.attention: ", n, " must be bf16 [tokens, heads, 128] with packed heads");
    TORCH_CHECK(t.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0,
                "rl_engine.attention: ", n, " must be 16-byte aligned with a 16-byte token pitch");
  };
  check3(q, "q");
  check3(k, "k");
  check3(v, "v");
  TORCH_CHECK(k.size(0) == v.size(0) && k.size(1) == v.size(1), "rl_engine.attention: k and v must match");
  TORCH_CHECK(q.size(1) % k.size(1) == 0, "rl_engine.attention: q heads must be a multiple of kv heads");
  TORCH_CHECK(seqs.is_cuda() && seqs.scalar_type() == torch::kInt32 && seqs.is_contiguous() && seqs.dim() == 2 &&
                  seqs.size(1) == 8,
              "rl_engine.attention: seqs must be int32 [S, 8]");
  TORCH_CHECK(tiles.is_cuda() && tiles.scalar_type() == torch::kInt32 && tiles.is_contiguous() && tiles.dim() == 2 &&
                  tiles.size(1) == 2,
              "rl_engine.attention: tiles must be int32 [n, 2]");
  const c10::cuda::CUDAGuard guard(q.device());
  Tensor out = torch::empty({q.size(0), q.size(1), 128}, q.options());
  Tensor lse = want_lse ? torch::empty({q.size(1), q.size(0)}, q.options().dtype(torch::kFloat32)) : Tensor();
  if (tiles.size(0) == 0) return {out, lse};
  rlk::AttnFwdArgs a{};
  a.q = reinterpret_cast<const __nv_bfloat16*>(q.data_ptr());
  a.k = reinterpret_cast<const __nv_bfloat16*>(k.data_ptr());
  a.v = reinterpret_cast<const __nv_bfloat16*>(v.data_ptr());
  a.ld_q = q.stride(0);
  a.ld_k = k.stride(0);
  a.ld_v = v.stride(0);
  a.total_q = q.size(0);
  a.total_kv = k.size(0);
  a.heads_q = static_cast<int>(q.size(1));
  a.heads_kv = static_cast<int>(k.size(1));
  a.seqs = seqs.data_ptr<int>();
  a.num_seqs = static_cast<int>(seqs.size(0));
  a.sm_count = sm_count_of(q.get_device());
  a.tiles = tiles.data_ptr<int>();
  a.num_tiles = static_cast<int>(tiles.size(0));
  a.causal = causal;
  a.softmax_scale = static_cast<float>(softmax_scale);
  a.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  a.ld_out = out.stride(0);
  a.lse = want_lse ? lse.data_ptr<float>() : nullptr;
  a.lse_head_stride = q.size(0);
  a.err = err_ptr(q);
  rlk::attention_forward(a, stream_of(q));
  after_launch();
  return {out, lse};
}

std::vector<Tensor> attention_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out,
                                  const Tensor& dout, const Tensor& lse, const Tensor& seqs, const Tensor& q_tiles,
                                  const Tensor& kv_items, const Tensor& q_blocks, const Tensor& reduce_jobs,
                                  int64_t num_slots, bool causal, double softmax_scale) {
  auto check3 = [](const Tensor& t, const char* n) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 3 && t.size(2) == 128 &&
                    t.stride(2) == 1 && t.stride(1) == 128 && t.stride(0) % 8 == 0 &&
                    reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0,
                "rl_engine.attention_bwd: ", n, " must be aligned bf16 [tokens, heads, 128] with packed heads");
  };
  check3(q, "q");
  check3(k, "k");
  check3(v, "v");
  check3(out, "out");
  check3(dout, "dout");
  TORCH_CHECK(out.stride(0) == dout.stride(0), "rl_engine.attention_bwd: out and dout must share their token pitch");
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == torch::kFloat32 && lse.is_contiguous() && lse.size(0) == q.size(1) &&
                  lse.size(1) == q.size(0),
              "rl_engine.attention_bwd: lse must be float32 [heads, tokens]");
  auto checki = [](const Tensor& t, int64_t w, const char* n) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt32 && t.is_contiguous() && t.dim() == 2 && t.size(1) == w,
                "rl_engine.attention_bwd: ", n, " must be int32 [n, ", w, "]");
  };
  checki(seqs, 8, "seqs");
  checki(q_tiles, 2, "q_tiles");
  checki(kv_items, 8, "kv_items");
  checki(q_blocks, 4, "q_blocks");
  checki(reduce_jobs, 4, "reduce_jobs");
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t hq = q.size(1), hkv = k.size(1);
  Tensor dq = torch::zeros({q.size(0), hq, 128}, q.options());
  Tensor dk = torch::zeros({k.size(0), hkv, 128}, k.options());
  Tensor dv = torch::zeros({k.size(0), hkv, 128}, k.options());
  Tensor delta = torch::empty({hq, q.size(0)}, lse.options());
  Tensor partials = torch::empty({std::max<int64_t>(num_slots, 1) * hkv * 2 * 128 * 128}, lse.options());
  cudaStream_t stream = stream_of(q);
  rlk::attention_delta(reinterpret_cast<const __nv_bfloat16*>(out.data_ptr()),
                       reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr()), out.stride(0), static_cast<int>(hq),
                       q.size(0), delta.data_ptr<float>(), stream);
  rlk::AttnBwdArgs a{};
  a.q = reinterpret_cast<const __nv_bfloat16*>(q.data_ptr());
  a.k = reinterpret_cast<const __nv_bfloat16*>(k.data_ptr());
  a.v = reinterpret_cast<const __nv_bfloat16*>(v.data_ptr());
  a.dout = reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr());
  a.ld_q = q.stride(0);
  a.ld_k = k.stride(0);
  a.ld_v = v.stride(0);
  a.ld_do = dout.stride(0);
  a.total_q = q.size(0);
  a.total_kv = k.size(0);
  a.heads_q = static_cast<int>(hq);
  a.heads_kv = static_cast<int>(hkv);
  a.seqs = seqs.data_ptr<int>();
  a.q_tiles = q_tiles.data_ptr<int>();
  a.num_q_tiles = static_cast<int>(q_tiles.size(0));
  a.kv_items = kv_items.data_ptr<int>();
  a.num_kv_items = static_cast<int>(kv_items.size(0));
  a.q_blocks = q_blocks.data_ptr<int>();
  a.reduce_jobs = reduce_jobs.data_ptr<int>();
  a.num_reduce_jobs = static_cast<int>(reduce_jobs.size(0));
  a.causal = causal;
  a.softmax_scale = static_cast<float>(softmax_scale);
  a.lse = lse.data_ptr<float>();
  a.delta = delta.data_ptr<float>();
  a.dq = reinterpret_cast<__nv_bfloat16*>(dq.data_ptr());
  a.ld_dq = dq.stride(0);
  a.dk = reinterpret_cast<__nv_bfloat16*>(dk.data_ptr());
  a.dv = reinterpret_cast<__nv_bfloat16*>(dv.data_ptr());
  a.ld_dkv = dk.stride(0);
  a.partials = partials.data_ptr<float>();
  a.err = err_ptr(q);
  rlk::attention_backward_dq(a, stream);
  rlk::attention_backward_dkv(a, stream);
  after_launch(a.num_reduce_jobs > 0 ? 4 : 3);
  return {dq, dk, dv};
}

// ------------------------------------------------------------------------------ diagnostics
std::vector<int64_t> error_state(int64_t device) {
  Tensor w = error_word(static_cast<int>(device)).cpu();
  auto a = w.accessor<int, 1>();
  return {a[0], a[1], a[2], a[3]};
}
void device_stamp(Tensor stamps, int64_t slot) {
  TORCH_CHECK(stamps.is_cuda() && stamps.scalar_type() == torch::kInt64 && stamps.is_contiguous() && slot >= 0 &&
                  slot < stamps.numel(),
              "rl_engine.device_stamp: stamps must be a contiguous int64 CUDA tensor and slot in range");
  const c10::cuda::CUDAGuard guard(stamps.device());
  rlk::device_stamp(reinterpret_cast<unsigned long long*>(stamps.data_ptr<int64_t>()), static_cast<int>(slot), stream_of(stamps));
  after_launch();
}

void reset_error(int64_t device) { error_word(static_cast<int>(device)).zero_(); }
long long launch_count() { return g_launches.load(); }
}  // namespace
namespace rlk {
void count_launch(int n) { g_launches += n; }
}  // namespace rlk
namespace {

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "rl_engine native sm_100a kernels";
#ifdef RLK_ATTN_PROFILE
  m.def("attention_profile", [] {
    std::vector<unsigned long long> v(16);
    rlk::attention_profile_read(v.data());
    rlk::attention_profile_reset();
    return v;
  });
  m.def("attention_bwd_profile", [] {
    std::vector<unsigned long long> v(16);
    rlk::attention_bwd_profile_read(v.data());
    return v;
  });
#endif
  m.def("device_stamp", &device_stamp);
  m.def("trace_enabled", [] { return rlk::trace_enabled(); });
  m.def("gemm", rlk::traced("rlk::gemm", &gemm), py::arg("a"), py::arg("b"), py::arg("a_mn") = false, py::arg("b_mn") = false,
        py::arg("out") = py::none(), py::arg("out_fp32") = false, py::arg("accumulate") = false, py::arg("alpha") = 1.0,
        py::arg("pair") = -1);
  m.def("grouped_gemm", rlk::traced("rlk::grouped_gemm", &grouped_gemm), py::arg("a"), py::arg("b"), py::arg("mode"),
        py::arg("table"), py::arg("num_groups"), py::arg("b_mn"), py::arg("out_fp32"), py::arg("out") = py::none());
  m.def("tp_ag_gemm", rlk::traced("rlk::tp_ag_gemm", &tp_ag_gemm));
  m.def("tp_gemm_rs", rlk::traced("rlk::tp_gemm_rs", &tp_gemm_rs));
  m.def("moe_topk", rlk::traced("rlk::moe_topk", &moe_topk));
  m.def("moe_topk_bwd", rlk::traced("rlk::moe_topk_bwd", &moe_topk_bwd));
  m.def("moe_build_plan", rlk::traced("rlk::moe_build_plan", &moe_build_plan));
  m.def("moe_gather_rows", rlk::traced("rlk::moe_gather_rows", &moe_gather_rows), py::arg("src"), py::arg("src_row"), py::arg("scale") = py::none(),
        py::arg("dst_ptr") = 0, py::arg("dst_ld") = 0);
  m.def("moe_combine", rlk::traced("rlk::moe_combine", &moe_combine), py::arg("src"), py::arg("src_ptr"), py::arg("src_ld"), py::arg("hidden"), py::arg("slot"),
        py::arg("weight") = py::none());
  m.def("moe_rowdot", rlk::traced("rlk::moe_rowdot", &moe_rowdot));
  m.def("linear_logp_workspace_shape", rlk::traced("rlk::linear_logp_workspace_shape", &linear_logp_workspace_shape));
  m.def("linear_logp_fwd", rlk::traced("rlk::linear_logp_fwd", &linear_logp_fwd), py::arg("hidden"), py::arg("weight"),
        py::arg("target"), py::arg("bias"), py::arg("vocab_start"), py::arg("rank"), py::arg("world"),
        py::arg("slot_base"), py::arg("total_records"), py::arg("peer_partials"), py::arg("peer_counters"),
        py::arg("next_counters"), py::arg("counter_capacity"), py::arg("want_lse"), py::arg("want_entropy"),
        py::arg("wait_limit_ms"), py::arg("global_vocab") = 0);
  m.def("linear_logp_dz", rlk::traced("rlk::linear_logp_dz", &linear_logp_dz));
  m.def("logp_rows", rlk::traced("rlk::logp_rows", &logp_rows));
  m.def("ratio_kl_fwd", rlk::traced("rlk::ratio_kl_fwd", &ratio_kl_fwd));
  m.def("ratio_kl_bwd", rlk::traced("rlk::ratio_kl_bwd", &ratio_kl_bwd));
  m.def("group_advantages", rlk::traced("rlk::group_advantages", &group_advantages));
  m.def("surrogate_fwd", rlk::traced("rlk::surrogate_fwd", &surrogate_fwd));
  m.def("surrogate_bwd", rlk::traced("rlk::surrogate_bwd", &surrogate_bwd));
  m.def("dpo_fwd", rlk::traced("rlk::dpo_fwd", &dpo_fwd));
  m.def("quantize_fp8_rows", rlk::traced("rlk::quantize_fp8_rows", &quantize_fp8_rows));
  m.def("gemm_fp8", rlk::traced("rlk::gemm_fp8", &gemm_fp8), py::arg("a_q"), py::arg("scale_a"), py::arg("b_q"),
        py::arg("scale_b"), py::arg("pair") = -1);
  m.def("attn_merge2", rlk::traced("rlk::attn_merge2", &attn_merge2));
  m.def("rmsnorm_fwd", rlk::traced("rlk::rmsnorm_fwd", &rmsnorm_fwd));
  m.def("qk_norm_fwd", rlk::traced("rlk::qk_norm_fwd", &qk_norm_fwd));
  m.def("qk_norm_bwd", rlk::traced("rlk::qk_norm_bwd", &qk_norm_bwd));
  m.def("rmsnorm_bwd", rlk::traced("rlk::rmsnorm_bwd", &rmsnorm_bwd));
  m.def("swiglu_fwd", rlk::traced("rlk::swiglu_fwd", &swiglu_fwd));
  m.def("swiglu_bwd", rlk::traced("rlk::swiglu_bwd", &swiglu_bwd));
  m.def("swiglu_packed_fwd", rlk::traced("rlk::swiglu_packed_fwd", &swiglu_packed_fwd));
  m.def("swiglu_packed_bwd", rlk::traced("rlk::swiglu_packed_bwd", &swiglu_packed_bwd));
  m.def("rope", rlk::traced("rlk::rope", &rope), py::arg("x"), py::arg("positions"), py::arg("cos"), py::arg("sin"), py::arg("inverse") = false,
        py::arg("out") = py::none());
  m.def("embedding_fwd", rlk::traced("rlk::embedding_fwd", &embedding_fwd));
  m.def("embedding_bwd", rlk::traced("rlk::embedding_bwd", &embedding_bwd));
  m.def("adamw", rlk::traced("rlk::adamw", &adamw));
  m.def("sample", rlk::traced("rlk::sample", &sample));
  m.def("attention_fwd", rlk::traced("rlk::attention_fwd", &attention_fwd));
  m.def("attention_bwd", rlk::traced("rlk::attention_bwd", &attention_bwd));
  m.def("error_state", rlk::traced("rlk::error_state", &error_state));
  m.def("reset_error", rlk::traced("rlk::reset_error", &reset_error));
  m.def("launch_count", rlk::traced("rlk::launch_count", &launch_count));
  rlk::bind_runtime(m);
}
