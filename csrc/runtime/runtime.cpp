#include "runtime.h"

namespace rlk {
void bind_runtime(pybind11::module_& m) { (void)m; }
}  // namespace rlk
