// Host-side construction of TMA tensor maps without linking libcuda: the driver entry point is
// resolved through the runtime (cudaGetDriverEntryPoint), so the extension also loads on machines
// without a driver (CPU-only test boxes).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

namespace rlk {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Driver-API calls need the primary context bound to the calling thread.  Threads that have only been
// handed a device index (e.g. autograd worker threads) may not have it yet; a runtime call binds it.
inline void bind_primary_context() {
  thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

inline EncodeTiledFn encode_tiled_fn() {
  bind_primary_context();
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
      throw std::runtime_error("rl_engine: cuTensorMapEncodeTiled is not available from this driver");
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 2-D row-major bf16 tensor [rows, cols] with leading dimension `ld` (elements); the box is
// [box_rows, box_cols] with box_cols * 2 bytes <= 128 when the 128-byte swizzle is used.
inline CUtensorMap make_tmap_2d_bf16(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                                     uint32_t box_cols, bool swizzle128 = true) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) throw std::invalid_argument("TMA base must be 16-byte aligned");
  if ((ld * 2) % 16 != 0) throw std::invalid_argument("TMA row pitch must be a multiple of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_tiled_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    throw std::runtime_error("rl_engine: cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  }
  return m;
}

// 2-D row-major tensor of 8-bit elements [rows, cols] (pitch `ld` bytes); box_cols <= 128 with the 128-byte swizzle.
inline CUtensorMap make_tmap_2d_u8(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                                   uint32_t box_cols) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) throw std::invalid_argument("TMA base must be 16-byte aligned");
  if (ld % 16 != 0) throw std::invalid_argument("TMA row pitch must be a multiple of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_tiled_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    throw std::runtime_error("rl_engine: cuTensorMapEncodeTiled(u8) failed with code " + std::to_string(int(r)));
  }
  return m;
}

// 3-D variant: [batch, rows, cols] with explicit row and batch pitches (elements).
inline CUtensorMap make_tmap_3d_bf16(const void* base, uint64_t batch, uint64_t rows, uint64_t cols, uint64_t row_ld,
                                     uint64_t batch_ld, uint32_t box_rows, uint32_t box_cols) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) throw std::invalid_argument("TMA base must be 16-byte aligned");
  if ((row_ld * 2) % 16 != 0 || (batch_ld * 2) % 16 != 0)
    throw std::invalid_argument("TMA pitches must be multiples of 16 bytes");
  CUtensorMap m;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {row_ld * 2, batch_ld * 2};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode_tiled_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    throw std::runtime_error("rl_engine: cuTensorMapEncodeTiled(3d) failed with code " + std::to_string(int(r)));
  }
  return m;
}

}  // namespace rlk
