#include "runtime/symm_heap.h"

#include <cuda_runtime.h>
#include <pybind11/stl.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace py = pybind11;

namespace {

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

class SymmHeap {
 public:
  SymmHeap(size_t bytes, int rank, int world, int device) : bytes_(bytes), rank_(rank), world_(world), device_(device) {
    check(cudaSetDevice(device_), "cudaSetDevice");
    check(cudaMalloc(&local_, bytes_), "cudaMalloc(symmetric heap)");
    check(cudaMemset(local_, 0, bytes_), "cudaMemset(symmetric heap)");
    check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    bases_.assign(world_, 0);
    bases_[rank_] = reinterpret_cast<unsigned long long>(local_);
    opened_.assign(world_, nullptr);
    check(cudaMalloc(&bases_dev_, sizeof(unsigned long long) * world_), "cudaMalloc(base table)");
    upload();
  }
  ~SymmHeap() { close(); }

  py::bytes handle() {
    cudaIpcMemHandle_t h;
    check(cudaIpcGetMemHandle(&h, local_), "cudaIpcGetMemHandle");
    return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
  }

  // handles[r] = IPC handle bytes of rank r's heap (entry of this rank is ignored).
  void map_peers(const std::vector<py::bytes>& handles) {
    if ((int)handles.size() != world_) throw std::runtime_error("map_peers: need one handle per rank");
    check(cudaSetDevice(device_), "cudaSetDevice");
    for (int r = 0; r < world_; ++r) {
      if (r == rank_) continue;
      std::string s = handles[r];
      if (s.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("map_peers: bad handle size");
      cudaIpcMemHandle_t h;
      std::memcpy(&h, s.data(), sizeof(h));
      void* p = nullptr;
      check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
      opened_[r] = p;
      bases_[r] = reinterpret_cast<unsigned long long>(p);
    }
    upload();
  }

  // Single-process emulation of several ranks on one GPU: take the peers' raw base addresses.
  void map_local(const std::vector<unsigned long long>& bases) {
    if ((int)bases.size() != world_) throw std::runtime_error("map_local: need one base per rank");
    for (int r = 0; r < world_; ++r)
      if (r != rank_) bases_[r] = bases[r];
    upload();
  }

  void close() {
    for (auto& p : opened_) {
      if (p != nullptr) { cudaIpcCloseMemHandle(p); p = nullptr; }
    }
    if (bases_dev_ != nullptr) { cudaFree(bases_dev_); bases_dev_ = nullptr; }
    if (local_ != nullptr) { cudaFree(local_); local_ = nullptr; }
  }

  unsigned long long base(int r) const { return bases_.at(r); }
  unsigned long long local_base() const { return reinterpret_cast<unsigned long long>(local_); }
  unsigned long long bases_device_ptr() const { return reinterpret_cast<unsigned long long>(bases_dev_); }
  size_t size() const { return bytes_; }
  int rank() const { return rank_; }
  int world() const { return world_; }

 private:
  void upload() {
    check(cudaMemcpy(bases_dev_, bases_.data(), sizeof(unsigned long long) * world_, cudaMemcpyHostToDevice),
          "cudaMemcpy(base table)");
  }
  size_t bytes_;
  int rank_, world_, device_;
  void* local_ = nullptr;
  unsigned long long* bases_dev_ = nullptr;
  std::vector<unsigned long long> bases_;
  std::vector<void*> opened_;
};

// Host-mapped int32[8] that kernels write error codes to; the host reads it without a sync of
// its own (after the stream has been synchronised by the caller).
class StatusWord {
 public:
  StatusWord() {
    check(cudaHostAlloc(reinterpret_cast<void**>(&host_), sizeof(int) * 8, cudaHostAllocMapped), "cudaHostAlloc");
    std::memset(host_, 0, sizeof(int) * 8);
    check(cudaHostGetDevicePointer(reinterpret_cast<void**>(&dev_), host_, 0), "cudaHostGetDevicePointer");
  }
  ~StatusWord() {
    if (host_ != nullptr) cudaFreeHost(host_);
  }
  unsigned long long device_ptr() const { return reinterpret_cast<unsigned long long>(dev_); }
  std::vector<int> read() const { return std::vector<int>(host_, host_ + 8); }
  void clear() { std::memset(host_, 0, sizeof(int) * 8); }

 private:
  int* host_ = nullptr;
  int* dev_ = nullptr;
};

}  // namespace

void bind_symm_heap(py::module_& m) {
  py::class_<SymmHeap>(m, "SymmHeap")
      .def(py::init<size_t, int, int, int>(), py::arg("bytes"), py::arg("rank"), py::arg("world"), py::arg("device"))
      .def("handle", &SymmHeap::handle)
      .def("map_peers", &SymmHeap::map_peers)
      .def("map_local", &SymmHeap::map_local)
      .def("close", &SymmHeap::close)
      .def("base", &SymmHeap::base)
      .def("local_base", &SymmHeap::local_base)
      .def("bases_device_ptr", &SymmHeap::bases_device_ptr)
      .def("size", &SymmHeap::size)
      .def_property_readonly("rank", &SymmHeap::rank)
      .def_property_readonly("world", &SymmHeap::world);
  py::class_<StatusWord>(m, "StatusWord")
      .def(py::init<>())
      .def("device_ptr", &StatusWord::device_ptr)
      .def("read", &StatusWord::read)
      .def("clear", &StatusWord::clear);
}
