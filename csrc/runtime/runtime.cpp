#include "runtime.h"

#include <cuda_runtime.h>
#include <stdint.h>

namespace rlk {

// Debug-bounds builds (-DRLK_DEBUG_BOUNDS=1): checked index accesses in kernels that have no error-word parameter of
// their own report to the word registered here for the device that is current at launch time.
namespace {
uint32_t* g_debug_words[64] = {};
}

void bind_debug_error_word(int device, uint32_t* word) {
  if (device >= 0 && device < 64) g_debug_words[device] = word;
}

uint32_t* debug_error_word() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
  return g_debug_words[device];
}

void bind_runtime(pybind11::module_& m) {
  bind_symmetric_heap(m);
  bind_comm(m);
}
}  // namespace rlk
