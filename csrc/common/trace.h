// NVTX ranges around the native launchers.  Off unless RLK_NVTX=1 is set when the process starts, so the
// default cost is one predictable branch per call.  NVTX v3 is header-only: nothing is linked; the range
// calls are no-ops until a tool (Nsight Systems / Compute) injects itself.
// The reference has no tracing hooks (its profiler times with CUDA events only: benchmarks/profiler.py:187-214).
#pragma once

#include <nvtx3/nvToolsExt.h>

#include <cstdlib>
#include <utility>

namespace rlk {

inline bool trace_enabled() {
  static const bool on = [] {
    const char* env = std::getenv("RLK_NVTX");
    return env != nullptr && env[0] != '\0' && env[0] != '0';
  }();
  return on;
}

class TraceRange {
 public:
  explicit TraceRange(const char* name) : active_(trace_enabled()) {
    if (active_) nvtxRangePushA(name);
  }
  ~TraceRange() {
    if (active_) nvtxRangePop();
  }
  TraceRange(const TraceRange&) = delete;
  TraceRange& operator=(const TraceRange&) = delete;

 private:
  bool active_;
};

// Wrap a free function so that every call runs inside a range named after the binding.
template <typename R, typename... Args>
auto traced(const char* name, R (*fn)(Args...)) {
  return [name, fn](Args... args) -> R {
    TraceRange range(name);
    return fn(std::forward<Args>(args)...);
  };
}

}  // namespace rlk
