// Device-side time stamps: one thread writes %globaltimer (nanoseconds, the same clock domain on all GPUs
// of a node within NTP-like skew) into a slot of a device array, in stream order.  Lets a step be timed on
// the device ("max over ranks") without host synchronisation inside the timed region.
// The reference times with host-synchronised CUDA events only (benchmarks/profiler.py:187-214).
#include "../common/ptx.cuh"
#include "kernels.h"

namespace rlk {

namespace {
__global__ void device_stamp_kernel(unsigned long long* out, int slot) { out[slot] = global_timer_ns(); }
}  // namespace

void device_stamp(unsigned long long* out, int slot, cudaStream_t stream) {
  device_stamp_kernel<<<1, 1, 0, stream>>>(out, slot);
}

}  // namespace rlk
