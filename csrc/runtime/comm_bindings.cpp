// Python bindings of the peer-memory communication kernels.  Peer buffers are passed as raw device
// addresses (ints) obtained from SymmetricHeap.ptrs(); local tensors as torch tensors.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include <cmath>
#include <type_traits>
#include <vector>

#include "../kernels/kernels.h"
#include "../common/trace.h"
#include "runtime.h"

namespace rlk {

namespace {

using torch::Tensor;

std::vector<void*> to_ptrs(const std::vector<uint64_t>& addrs) {
  TORCH_CHECK(!addrs.empty() && addrs.size() <= 8, "rl_engine: need 1..8 peer addresses");
  std::vector<void*> out;
  for (auto a : addrs) {
    TORCH_CHECK(a != 0, "rl_engine: null peer address");
    out.push_back(reinterpret_cast<void*>(a));
  }
  return out;
}

int dtype_code(torch::ScalarType t) {
  if (t == torch::kFloat32) return 0;
  if (t == torch::kBFloat16) return 1;
  if (t == torch::kFloat16) return 2;
  TORCH_CHECK(false, "rl_engine: unsupported dtype");
}

cudaStream_t cur_stream(int device) { return at::cuda::getCurrentCUDAStream(device).stream(); }

void py_peer_barrier(std::vector<uint64_t> pads, int64_t rank, int64_t epoch, double limit_ms, Tensor err_word) {
  const c10::cuda::CUDAGuard guard(err_word.device());
  auto p = to_ptrs(pads);
  peer_barrier(p.data(), static_cast<int>(rank), static_cast<int>(p.size()), static_cast<unsigned int>(epoch),
               static_cast<unsigned long long>(limit_ms * 1e6), reinterpret_cast<uint32_t*>(err_word.data_ptr<int>()),
               cur_stream(err_word.get_device()));
}

void py_zero1_fused_step(std::vector<uint64_t> grads, std::vector<uint64_t> params, int64_t lo, int64_t hi, Tensor m,
                         Tensor v, std::optional<Tensor> master, double lr, double b1, double b2, double eps, double wd,
                         int64_t step, double grad_scale, int64_t rank, std::optional<Tensor> barrier_err,
                         int64_t max_blocks) {
  TORCH_CHECK(rank >= 0 && rank < static_cast<int64_t>(params.size()), "rl_engine.zero1: rank out of range");
  TORCH_CHECK(lo % 8 == 0 && hi % 8 == 0 && hi >= lo, "rl_engine.zero1: shard bounds must be multiples of 8");
  TORCH_CHECK(m.is_cuda() && m.scalar_type() == torch::kFloat32 && m.is_contiguous() && m.numel() >= hi - lo &&
                  v.scalar_type() == torch::kFloat32 && v.is_contiguous() && v.numel() >= hi - lo,
              "rl_engine.zero1: moments must be contiguous float32 of the shard size");
  TORCH_CHECK(grads.size() == params.size(), "rl_engine.zero1: need one gradient and one parameter buffer per rank");
  const c10::cuda::CUDAGuard guard(m.device());
  float* mp = nullptr;
  if (master.has_value() && master->defined()) {
    TORCH_CHECK(master->scalar_type() == torch::kFloat32 && master->is_contiguous() && master->numel() >= hi - lo,
                "rl_engine.zero1: master shard must be contiguous float32");
    mp = master->data_ptr<float>();
  }
  auto g = to_ptrs(grads);
  auto p = to_ptrs(params);
  const float bc1 = 1.f - static_cast<float>(std::pow(b1, static_cast<double>(step)));
  const float bc2 = 1.f - static_cast<float>(std::pow(b2, static_cast<double>(step)));
  const uint32_t* skip = nullptr;
  if (barrier_err.has_value() && barrier_err->defined()) {
    TORCH_CHECK(barrier_err->is_cuda() && barrier_err->scalar_type() == torch::kInt32 && barrier_err->numel() >= 1,
                "rl_engine.zero1: barrier_err must be the int32 error word of the preceding barrier");
    skip = reinterpret_cast<const uint32_t*>(barrier_err->data_ptr<int>());
  }
  zero1_fused_step(g.data(), p.data(), static_cast<int>(rank), static_cast<int>(g.size()), lo, hi, m.data_ptr<float>(),
                   v.data_ptr<float>(), mp, static_cast<float>(lr), static_cast<float>(b1), static_cast<float>(b2),
                   static_cast<float>(eps), static_cast<float>(wd), bc1, bc2, static_cast<float>(grad_scale), skip,
                   static_cast<int>(max_blocks), cur_stream(m.get_device()));
}

void py_peer_sum(std::vector<uint64_t> srcs, int64_t n, bool src_fp32, Tensor out) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.numel() >= n, "rl_engine.peer_sum: out too small");
  const c10::cuda::CUDAGuard guard(out.device());
  auto s = to_ptrs(srcs);
  peer_sum(s.data(), static_cast<int>(s.size()), n, src_fp32, out.data_ptr(), out.scalar_type() == torch::kFloat32,
           cur_stream(out.get_device()));
}

void py_cast_broadcast(const Tensor& src, std::vector<uint64_t> dsts, int64_t dst_dtype_code) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous(), "rl_engine.cast_broadcast: src must be a contiguous CUDA tensor");
  const c10::cuda::CUDAGuard guard(src.device());
  auto d = to_ptrs(dsts);
  cast_broadcast(src.data_ptr(), dtype_code(src.scalar_type()), d.data(), static_cast<int>(dst_dtype_code),
                 static_cast<int>(d.size()), src.numel(), cur_stream(src.get_device()));
}

// digests[slot] += digest of the bytes of ``t`` (contiguous, 16-byte aligned); ``digests`` is int64 on the same device.
void py_weight_digest(const Tensor& t, Tensor digests, int64_t slot) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "rl_engine.weight_digest: contiguous CUDA tensor expected");
  TORCH_CHECK(digests.is_cuda() && digests.scalar_type() == torch::kInt64 && digests.is_contiguous() && slot >= 0 &&
                  slot < digests.numel() && digests.get_device() == t.get_device(),
              "rl_engine.weight_digest: digests must be a contiguous int64 tensor on the tensor's device");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, "rl_engine.weight_digest: data must be 16-byte aligned");
  const c10::cuda::CUDAGuard guard(t.device());
  weight_digest64(t.data_ptr(), static_cast<long long>(t.numel()) * static_cast<long long>(t.element_size()),
                  reinterpret_cast<unsigned long long*>(digests.data_ptr<int64_t>()) + slot, cur_stream(t.get_device()));
}

void check_segment_table(const Tensor& table, const char* who) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == torch::kInt64 && table.is_contiguous() && table.dim() == 2 &&
                  table.size(1) == 4,
              "rl_engine.", who, ": table must be a contiguous CUDA int64 tensor [tensors, 4]");
}

// One launch for a whole update: every row of ``table`` (source address, destination byte offset, elements, units of
// the earlier rows; 32768 elements per unit) is cast from ``src_dtype`` to ``dst_dtype`` into ``dst_base + offset``.
void py_cast_segments(const Tensor& table, int64_t total_units, int64_t src_dtype_code, int64_t dst_dtype_code,
                      uint64_t dst_base) {
  check_segment_table(table, "cast_segments");
  TORCH_CHECK(src_dtype_code >= 0 && src_dtype_code <= 2 && dst_dtype_code >= 0 && dst_dtype_code <= 2,
              "rl_engine.cast_segments: dtype codes are 0 (float32), 1 (bfloat16), 2 (float16)");
  const c10::cuda::CUDAGuard guard(table.device());
  cast_segments(table.data_ptr(), static_cast<int>(table.size(0)), total_units, static_cast<int>(src_dtype_code),
                static_cast<int>(dst_dtype_code), reinterpret_cast<void*>(dst_base), cur_stream(table.get_device()));
}

// digests[row.slot] += digest of the row's bytes, for every row of ``table`` (source address, slot, bytes, units of the
// earlier rows; 32768 64-bit words per unit).  Every source must be 16-byte aligned.
void py_digest_segments(const Tensor& table, int64_t total_units, Tensor digests) {
  check_segment_table(table, "digest_segments");
  TORCH_CHECK(digests.is_cuda() && digests.scalar_type() == torch::kInt64 && digests.is_contiguous() &&
                  digests.get_device() == table.get_device(),
              "rl_engine.digest_segments: digests must be a contiguous int64 tensor on the table's device");
  const c10::cuda::CUDAGuard guard(table.device());
  digest_segments(table.data_ptr(), static_cast<int>(table.size(0)), total_units,
                  reinterpret_cast<unsigned long long*>(digests.data_ptr<int64_t>()), cur_stream(table.get_device()));
}

// Copy-engine transfer of ``nbytes`` from ``src`` to a device address that may live on a peer GPU (a mapped window of
// the symmetric heap), in stream order.  Plain bytes need no SM: the copy engines reach the NVLink rate where
// store loops from the SMs measured 0.4 of it.
void py_peer_copy(uint64_t dst, const Tensor& src, int64_t nbytes) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous(), "rl_engine.peer_copy: src must be a contiguous CUDA tensor");
  TORCH_CHECK(nbytes >= 0 && nbytes <= static_cast<int64_t>(src.numel()) * static_cast<int64_t>(src.element_size()),
              "rl_engine.peer_copy: nbytes exceeds the source tensor");
  if (nbytes == 0) return;
  const c10::cuda::CUDAGuard guard(src.device());
  C10_CUDA_CHECK(cudaMemcpyAsync(reinterpret_cast<void*>(dst), src.data_ptr(), static_cast<size_t>(nbytes),
                                 cudaMemcpyDeviceToDevice, cur_stream(src.get_device())));
}

void check_rows(const Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 2 && t.stride(1) == 1 && t.size(1) % 8 == 0 &&
                  t.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0,
              "rl_engine.moe: ", n, " must be aligned bf16 rows");
}
void check_i32(const Tensor& t, int64_t n, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt32 && t.is_contiguous() && t.numel() == n, "rl_engine.moe: ", name,
              " must be contiguous int32 with ", n, " entries");
}

void py_moe_scatter_rows_peer(const Tensor& src, const Tensor& token, const Tensor& dest_rank, const Tensor& dest_slot,
                              std::optional<Tensor> scale, std::vector<uint64_t> dst, int64_t ld_dst) {
  check_rows(src, "src");
  const int64_t n = token.numel();
  check_i32(token, n, "token");
  check_i32(dest_rank, n, "dest_rank");
  check_i32(dest_slot, n, "dest_slot");
  const c10::cuda::CUDAGuard guard(src.device());
  auto d = to_ptrs(dst);
  Tensor sc;
  const float* sp = nullptr;
  if (scale.has_value() && scale->defined()) {
    sc = scale->to(torch::kFloat32).contiguous();
    TORCH_CHECK(sc.numel() == n, "scale must have one entry per assignment");
    sp = sc.data_ptr<float>();
  }
  moe_scatter_rows_peer(reinterpret_cast<const __nv_bfloat16*>(src.data_ptr()), src.stride(0), token.data_ptr<int>(),
                        dest_rank.data_ptr<int>(), dest_slot.data_ptr<int>(), sp, d.data(), static_cast<int>(d.size()), ld_dst,
                        static_cast<int>(n), static_cast<int>(src.size(1)), cur_stream(src.get_device()));
}

Tensor py_moe_combine_peer(std::vector<uint64_t> src, int64_t ld_src, int64_t hidden, const Tensor& rank, const Tensor& slot,
                           std::optional<Tensor> weight) {
  TORCH_CHECK(slot.dim() == 2 && hidden % 8 == 0, "moe_combine_peer: slot [T, k], hidden % 8 == 0");
  check_i32(slot, slot.numel(), "slot");
  check_i32(rank, slot.numel(), "rank");
  const c10::cuda::CUDAGuard guard(slot.device());
  auto s = to_ptrs(src);
  Tensor w;
  const float* wp = nullptr;
  if (weight.has_value() && weight->defined()) {
    w = weight->to(torch::kFloat32).contiguous();
    TORCH_CHECK(w.numel() == slot.numel(), "weight must match slot");
    wp = w.data_ptr<float>();
  }
  Tensor out = torch::empty({slot.size(0), hidden}, slot.options().dtype(torch::kBFloat16));
  moe_combine_peer(s.data(), static_cast<int>(s.size()), ld_src, rank.data_ptr<int>(), slot.data_ptr<int>(), wp,
                   static_cast<int>(slot.size(1)), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), out.stride(0),
                   static_cast<int>(slot.size(0)), static_cast<int>(hidden), cur_stream(slot.get_device()));
  return out;
}

}  // namespace

// Every binding below launches exactly one kernel: count it, (with RLK_NVTX=1) put it in a range, and raise if the
// launch itself was refused (bad configuration, attribute not set on this device, ...).
template <typename R, typename... Args>
auto counted(const char* name, R (*fn)(Args...)) {
  return [name, fn](Args... args) -> R {
    TraceRange range(name);
    count_launch(1);
    if constexpr (std::is_void_v<R>) {
      fn(std::forward<Args>(args)...);
      C10_CUDA_KERNEL_LAUNCH_CHECK();
    } else {
      R out = fn(std::forward<Args>(args)...);
      C10_CUDA_KERNEL_LAUNCH_CHECK();
      return out;
    }
  };
}

void bind_comm(pybind11::module_& m) {
  m.def("moe_scatter_rows_peer", counted("rlk::moe_scatter_rows_peer", &py_moe_scatter_rows_peer));
  m.def("moe_combine_peer", counted("rlk::moe_combine_peer", &py_moe_combine_peer));
  m.def("peer_barrier", counted("rlk::peer_barrier", &py_peer_barrier));
  m.def("zero1_fused_step", counted("rlk::zero1_fused_step", &py_zero1_fused_step));
  m.def("peer_sum", counted("rlk::peer_sum", &py_peer_sum));
  m.def("cast_broadcast", counted("rlk::cast_broadcast", &py_cast_broadcast));
  m.def("weight_digest", counted("rlk::weight_digest", &py_weight_digest));
  m.def("cast_segments", counted("rlk::cast_segments", &py_cast_segments));
  m.def("digest_segments", counted("rlk::digest_segments", &py_digest_segments));
  m.def("peer_copy", &py_peer_copy);
}

}  // namespace rlk
