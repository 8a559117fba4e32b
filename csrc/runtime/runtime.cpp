#include "runtime.h"

namespace rlk {
void bind_runtime(pybind11::module_& m) {
  bind_symmetric_heap(m);
  bind_comm(m);
}
}  // namespace rlk
