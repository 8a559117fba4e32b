// Allocation-free entry point.  This has no counterpart in the reference project.
//
// Some callers cannot allocate device memory at the moment they need a kernel: code running inside
// a CUDA stream capture (cudaMalloc is illegal while capturing), a serving loop that runs with its
// memory pool frozen, or a host thread that was handed a stream but not an allocator (a C or Rust
// runtime linking this library without PyTorch).  For them, one kernel that normally needs a scratch
// buffer from the caller -- the RMSNorm backward, whose per-row-chunk partial sums of the weight
// gradient live in scratch -- is exposed with the scratch held inside the library instead.
//
// Contract
//   * The scratch is a file-scope device array of RLK_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU
//     that loads the library holds it from load until the process exits.
//   * A call needs ceil(rows / 64) * dim floats of scratch.  Larger problems are rejected with
//     RLK_NOALLOC_TOO_LARGE and nothing is launched; use the regular entry point (caller-provided
//     scratch) for those.
//   * The first call on a device resolves the device address of the scratch array
//     (cudaGetSymbolAddress).  Make that first call outside of any stream capture.
//   * Rows of more than 12288 elements (dim * 4 bytes above 48 KB) on the generic path -- anything but
//     bfloat16 x with bfloat16 weight -- need the kernel's opt-in shared-memory size: EVERY such call
//     sets that attribute (a host-side call on the kernel for that dtype pair, no allocation), not only
//     the first.  dim * 4 bytes above RLK_NOALLOC_MAX_ROW_BYTES cannot run at all and is rejected with
//     RLK_NOALLOC_BAD_ARGUMENT before anything is launched.
//   * The function reads and clears the CUDA runtime's last-error state before and after its launches:
//     a launch failure is returned here (RLK_NOALLOC_CUDA_ERROR) and not left for the host's next call.
//   * The function never calls cudaMalloc / cudaFree or any allocating library routine.
//   * All calls on a device share the one scratch array, and it keeps the previous call's contents.
//     The kernels overwrite every scratch element they later read, so nothing needs clearing, but two
//     calls that overlap on the GPU (different streams, no dependency) race on it: serialise them.
//   * x, dy, dx are [rows, dim] with row pitch `ld` elements, of type `x_dtype`; weight and dweight are
//     [dim] of type `w_dtype`; rstd is float32 [rows] as saved by the forward.  dtype codes:
//     0 = float32, 1 = bfloat16, 2 = float16.  All pointers are device pointers on the current device.
#pragma once

#include <cuda_runtime.h>

#define RLK_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define RLK_NOALLOC_MAX_ROW_BYTES (227 * 1024)

#define RLK_NOALLOC_OK 0
#define RLK_NOALLOC_TOO_LARGE 1
#define RLK_NOALLOC_BAD_ARGUMENT 2
#define RLK_NOALLOC_CUDA_ERROR 3

#ifdef __cplusplus
extern "C" {
#endif

// Returns one of the RLK_NOALLOC_* codes.  On RLK_NOALLOC_CUDA_ERROR, `rlk_noalloc_last_error` describes it.
int rlk_rmsnorm_backward_noalloc(const void* x, const void* weight, const void* dy, const float* rstd, void* dx,
                                 void* dweight, long long rows, int dim, long long ld, int x_dtype, int w_dtype,
                                 cudaStream_t stream);

// Scratch floats a problem of this size needs (to compare against RLK_NOALLOC_SCRATCH_FLOATS).
long long rlk_rmsnorm_backward_noalloc_scratch_floats(long long rows, int dim);

const char* rlk_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
