// See no_alloc.h.  The scratch array, the once-per-device address look-up and the entry point live in
// this one file; the kernels themselves are the ones behind the regular RMSNorm backward.
#include "no_alloc.h"

#include <mutex>
#include <string>

#include "kernels.h"

namespace {

// Device-side storage for the partial weight-gradient sums.  In host code this name is only a handle
// for the runtime: its device address must be obtained with cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_scratch[RLK_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
constexpr int kRowsPerCta = 64;  // fixed here (the regular entry point adapts it to the row count): scratch need = ceil(rows / 64) * dim
float* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mutex;
thread_local std::string g_last_error;

// Resolve the scratch address for the current device, once.
int scratch_for_current_device(float** out) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
    g_last_error = std::string("cudaGetDevice failed: ") + cudaGetErrorString(e);
    return RLK_NOALLOC_CUDA_ERROR;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[device] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      g_last_error = std::string("cudaGetSymbolAddress failed: ") + cudaGetErrorString(e);
      return RLK_NOALLOC_CUDA_ERROR;
    }
    g_scratch_ptr[device] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[device];
  return RLK_NOALLOC_OK;
}

}  // namespace

extern "C" long long rlk_rmsnorm_backward_noalloc_scratch_floats(long long rows, int dim) {
  if (rows <= 0 || dim <= 0) return 0;
  return static_cast<long long>(rlk::rmsnorm_bwd_chunks(rows, kRowsPerCta)) * dim;
}

extern "C" const char* rlk_noalloc_last_error(void) { return g_last_error.c_str(); }

extern "C" int rlk_rmsnorm_backward_noalloc(const void* x, const void* weight, const void* dy, const float* rstd, void* dx,
                                            void* dweight, long long rows, int dim, long long ld, int x_dtype,
                                            int w_dtype, cudaStream_t stream) {
  if (!x || !weight || !dy || !rstd || !dx || !dweight || rows <= 0 || dim <= 0 || ld < dim || x_dtype < 0 ||
      x_dtype > 2 || w_dtype < 0 || w_dtype > 2) {
    g_last_error = "null pointer, non-positive size, ld < dim or unknown dtype code";
    return RLK_NOALLOC_BAD_ARGUMENT;
  }
  if (static_cast<long long>(dim) * 4 > RLK_NOALLOC_MAX_ROW_BYTES) {
    g_last_error = "dim * 4 bytes exceeds the " + std::to_string(RLK_NOALLOC_MAX_ROW_BYTES) +
                   "-byte shared-memory row buffer of the kernel";
    return RLK_NOALLOC_BAD_ARGUMENT;
  }
  if (rlk_rmsnorm_backward_noalloc_scratch_floats(rows, dim) > RLK_NOALLOC_SCRATCH_FLOATS) {
    g_last_error = "problem needs " + std::to_string(rlk_rmsnorm_backward_noalloc_scratch_floats(rows, dim)) +
                   " scratch floats; the built-in scratch holds " + std::to_string(RLK_NOALLOC_SCRATCH_FLOATS);
    return RLK_NOALLOC_TOO_LARGE;
  }
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != RLK_NOALLOC_OK) return rc;
  // Drop a launch error that an earlier, unrelated call left behind, so that what is read after the launches below
  // belongs to them; then read AND clear the result, so that a failure here is not blamed on the host's next call.
  (void)cudaGetLastError();
  rlk::rmsnorm_backward(x, ld, x_dtype, weight, w_dtype, dy, ld, rstd, dx, ld, rows, dim, scratch, dweight, stream,
                        kRowsPerCta);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_error = std::string("launch failed: ") + cudaGetErrorString(e);
    return RLK_NOALLOC_CUDA_ERROR;
  }
  return RLK_NOALLOC_OK;
}
