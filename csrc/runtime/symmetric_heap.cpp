// Symmetric heap: one CUDA virtual-memory allocation per rank, exported as a POSIX file descriptor
// and mapped by every peer of the node, so kernels can load/store any rank's segment over
// NVLink / NVSwitch with ordinary pointers (no NCCL, no NVSHMEM).
//
// The driver API is resolved at run time through the CUDA runtime, so the extension has no link-time
// dependency on libcuda.  File descriptors travel between processes over a unix socket (SCM_RIGHTS);
// that part lives in Python (rl_engine/parallel/symmetric.py).
//
// The reference reaches the same driver calls through ctypes for its weight bridge
// (rl_engine/executors/bridge.py:985-1332); this is the native equivalent and also serves the
// fused compute+communication kernels.
#include <cuda.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "runtime.h"

namespace rlk {

namespace {

template <class Fn>
Fn driver_fn(const char* name) {
  cudaFree(nullptr);  // make sure the primary context exists and is current
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
    throw std::runtime_error(std::string("rl_engine: CUDA driver entry point not found: ") + name);
  return reinterpret_cast<Fn>(p);
}

void check(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) throw std::runtime_error(std::string("rl_engine: ") + what + " failed with CUresult " + std::to_string(int(r)));
}

struct Driver {
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*memRelease)(CUmemGenericAllocationHandle);
  CUresult (*memGetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*memAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*memAddressFree)(CUdeviceptr, size_t);
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*memUnmap)(CUdeviceptr, size_t);
  CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*memExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*memImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);

  static const Driver& get() {
    static Driver d = [] {
      Driver x;
      x.memCreate = driver_fn<decltype(x.memCreate)>("cuMemCreate");
      x.memRelease = driver_fn<decltype(x.memRelease)>("cuMemRelease");
      x.memGetGranularity = driver_fn<decltype(x.memGetGranularity)>("cuMemGetAllocationGranularity");
      x.memAddressReserve = driver_fn<decltype(x.memAddressReserve)>("cuMemAddressReserve");
      x.memAddressFree = driver_fn<decltype(x.memAddressFree)>("cuMemAddressFree");
      x.memMap = driver_fn<decltype(x.memMap)>("cuMemMap");
      x.memUnmap = driver_fn<decltype(x.memUnmap)>("cuMemUnmap");
      x.memSetAccess = driver_fn<decltype(x.memSetAccess)>("cuMemSetAccess");
      x.memExport = driver_fn<decltype(x.memExport)>("cuMemExportToShareableHandle");
      x.memImport = driver_fn<decltype(x.memImport)>("cuMemImportFromShareableHandle");
      return x;
    }();
    return d;
  }
};

class SymmetricHeap {
 public:
  SymmetricHeap(int device, size_t bytes, int rank, int world)
      : device_(device), rank_(rank), world_(world), handles_(world, 0), bases_(world, 0), mapped_(world, false) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world) throw std::invalid_argument("SymmetricHeap: bad rank/world");
    cudaSetDevice(device);
    const Driver& d = Driver::get();
    CUmemAllocationProp prop = {};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gran = 0;
    check(d.memGetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
    size_ = (bytes + gran - 1) / gran * gran;
    check(d.memCreate(&handles_[rank], size_, &prop, 0), "cuMemCreate");
    map(rank);
    cudaMemset(reinterpret_cast<void*>(bases_[rank]), 0, size_);
    cudaDeviceSynchronize();
  }

  ~SymmetricHeap() { close(); }

  int export_fd() {
    int fd = -1;
    check(Driver::get().memExport(&fd, handles_[rank_], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
          "cuMemExportToShareableHandle");
    return fd;
  }

  void import_peer(int peer, int fd) {
    if (peer < 0 || peer >= world_ || peer == rank_) throw std::invalid_argument("SymmetricHeap: bad peer rank");
    if (mapped_[peer]) throw std::runtime_error("SymmetricHeap: peer already imported");
    cudaSetDevice(device_);
    check(Driver::get().memImport(&handles_[peer], reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
          "cuMemImportFromShareableHandle");
    map(peer);
  }

  uint64_t ptr(int r) const {
    if (r < 0 || r >= world_ || !mapped_[r]) throw std::invalid_argument("SymmetricHeap: rank not mapped");
    return static_cast<uint64_t>(bases_[r]);
  }
  std::vector<uint64_t> ptrs() const {
    std::vector<uint64_t> out;
    for (int r = 0; r < world_; ++r) out.push_back(mapped_[r] ? static_cast<uint64_t>(bases_[r]) : 0);
    return out;
  }
  size_t size() const { return size_; }
  int rank() const { return rank_; }
  int world() const { return world_; }

  // A tensor aliasing [offset, offset + numel * itemsize) of rank r's segment.  The heap must outlive it.
  torch::Tensor tensor(int r, size_t offset, std::vector<int64_t> shape, torch::ScalarType dtype) const {
    if (r != rank_) throw std::invalid_argument("SymmetricHeap.tensor: only the local segment can be viewed; use read_peer");
    int64_t numel = 1;
    for (auto s : shape) numel *= s;
    const size_t bytes = static_cast<size_t>(numel) * c10::elementSize(dtype);
    if (offset + bytes > size_) throw std::out_of_range("SymmetricHeap: tensor exceeds the segment");
    void* p = reinterpret_cast<void*>(ptr(r) + offset);
    return torch::from_blob(p, shape, torch::TensorOptions().dtype(dtype).device(torch::kCUDA, device_));
  }

  // A local copy of a window of rank r's segment (debugging / tests; kernels use the raw pointers).
  torch::Tensor read_peer(int r, size_t offset, std::vector<int64_t> shape, torch::ScalarType dtype) const {
    torch::Tensor out = torch::empty(shape, torch::TensorOptions().dtype(dtype).device(torch::kCUDA, device_));
    const size_t bytes = static_cast<size_t>(out.numel()) * c10::elementSize(dtype);
    if (offset + bytes > size_) throw std::out_of_range("SymmetricHeap: window exceeds the segment");
    cudaSetDevice(device_);
    cudaError_t e = cudaMemcpy(out.data_ptr(), reinterpret_cast<const void*>(ptr(r) + offset), bytes, cudaMemcpyDefault);
    if (e != cudaSuccess) throw std::runtime_error(std::string("SymmetricHeap: peer copy failed: ") + cudaGetErrorString(e));
    return out;
  }

  void close() {
    const Driver& d = Driver::get();
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
    for (int r = 0; r < world_; ++r) {
      if (mapped_[r]) {
        d.memUnmap(bases_[r], size_);
        d.memAddressFree(bases_[r], size_);
        mapped_[r] = false;
      }
      if (handles_[r]) {
        d.memRelease(handles_[r]);
        handles_[r] = 0;
      }
    }
  }

 private:
  void map(int r) {
    const Driver& d = Driver::get();
    check(d.memAddressReserve(&bases_[r], size_, 0, 0, 0), "cuMemAddressReserve");
    check(d.memMap(bases_[r], size_, 0, handles_[r], 0), "cuMemMap");
    CUmemAccessDesc access = {};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = device_;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    check(d.memSetAccess(bases_[r], size_, &access, 1), "cuMemSetAccess");
    mapped_[r] = true;
  }

  int device_, rank_, world_;
  size_t size_ = 0;
  std::vector<CUmemGenericAllocationHandle> handles_;
  std::vector<CUdeviceptr> bases_;
  std::vector<bool> mapped_;
};

// One CUDA VMM allocation that can be handed to another process on the same node as a POSIX file
// descriptor: the publisher side of the weight bridge creates it, a consumer opens the descriptor and
// maps the same physical memory (zero copy).  Reference analogue: rl_engine/executors/bridge.py:
// 1207-1332 (ctypes calls into libcuda).
class VmmSegment {
 public:
  // fd < 0: create a fresh allocation of >= bytes; fd >= 0: map the allocation behind the descriptor.
  VmmSegment(int device, size_t bytes, int fd) : device_(device) {
    cudaSetDevice(device);
    const Driver& d = Driver::get();
    CUmemAllocationProp prop = {};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gran = 0;
    check(d.memGetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
    size_ = (bytes + gran - 1) / gran * gran;
    if (size_ == 0) size_ = gran;
    if (fd < 0) {
      check(d.memCreate(&handle_, size_, &prop, 0), "cuMemCreate");
    } else {
      check(d.memImport(&handle_, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
            "cuMemImportFromShareableHandle");
    }
    check(d.memAddressReserve(&base_, size_, 0, 0, 0), "cuMemAddressReserve");
    check(d.memMap(base_, size_, 0, handle_, 0), "cuMemMap");
    CUmemAccessDesc access = {};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = device;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    check(d.memSetAccess(base_, size_, &access, 1), "cuMemSetAccess");
    open_ = true;
  }
  ~VmmSegment() { close(); }

  int export_fd() {
    int fd = -1;
    check(Driver::get().memExport(&fd, handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
    return fd;
  }
  uint64_t ptr() const { return static_cast<uint64_t>(base_); }
  size_t size() const { return size_; }
  torch::Tensor tensor(size_t offset, std::vector<int64_t> shape, std::vector<int64_t> strides, torch::ScalarType dtype) const {
    if (!open_) throw std::runtime_error("VmmSegment: closed");
    void* p = reinterpret_cast<void*>(base_ + offset);
    auto opts = torch::TensorOptions().dtype(dtype).device(torch::kCUDA, device_);
    return strides.empty() ? torch::from_blob(p, shape, opts) : torch::from_blob(p, shape, strides, opts);
  }
  void close() {
    if (!open_) return;
    const Driver& d = Driver::get();
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
    d.memUnmap(base_, size_);
    d.memAddressFree(base_, size_);
    d.memRelease(handle_);
    open_ = false;
  }

 private:
  int device_;
  size_t size_ = 0;
  CUmemGenericAllocationHandle handle_ = 0;
  CUdeviceptr base_ = 0;
  bool open_ = false;
};

}  // namespace

void bind_symmetric_heap(pybind11::module_& m) {
  namespace py = pybind11;
  py::class_<VmmSegment>(m, "VmmSegment")
      .def(py::init<int, size_t, int>(), py::arg("device"), py::arg("bytes"), py::arg("fd") = -1)
      .def("export_fd", &VmmSegment::export_fd)
      .def("ptr", &VmmSegment::ptr)
      .def("size", &VmmSegment::size)
      .def("tensor", &VmmSegment::tensor, py::arg("offset"), py::arg("shape"), py::arg("strides") = std::vector<int64_t>{},
           py::arg("dtype"))
      .def("close", &VmmSegment::close);
  py::class_<SymmetricHeap>(m, "SymmetricHeap")
      .def(py::init<int, size_t, int, int>(), py::arg("device"), py::arg("bytes"), py::arg("rank"), py::arg("world"))
      .def("export_fd", &SymmetricHeap::export_fd)
      .def("import_peer", &SymmetricHeap::import_peer)
      .def("ptr", &SymmetricHeap::ptr)
      .def("ptrs", &SymmetricHeap::ptrs)
      .def("size", &SymmetricHeap::size)
      .def("rank", &SymmetricHeap::rank)
      .def("world", &SymmetricHeap::world)
      .def("tensor", &SymmetricHeap::tensor)
      .def("read_peer", &SymmetricHeap::read_peer)
      .def("close", &SymmetricHeap::close);
}

}  // namespace rlk
