// C++ runtime pieces exposed to Python next to the kernels (symmetric heap, peer signals).
#pragma once

#include <pybind11/pybind11.h>

namespace rlk {
void bind_runtime(pybind11::module_& m);
void bind_symmetric_heap(pybind11::module_& m);
void bind_comm(pybind11::module_& m);
// Adds to the process-wide count of native kernel launches reported by `launch_count()`.
void count_launch(int n);
}  // namespace rlk
