// C++ extension point: user-defined all-to-all algorithms.
//
// Subclass AbstractComm, then register a factory under a name:
//
//     struct MyComm : planmoe::AbstractComm {
//       using AbstractComm::AbstractComm;
//       void all_to_all(const void* in, void* out, size_t bytes, cudaStream_t s) override { ... }
//     };
//     static planmoe::CommRegistrar reg("mine", [](const planmoe::CommContext& c) {
//       return std::unique_ptr<planmoe::AbstractComm>(new MyComm(c)); });
//
// Build that into a shared object linked against planmoe_b200/_C.so and load it (ctypes.CDLL or
// torch.ops.load_library) before constructing the layer with comm_name="mine".  The reference offers
// the same hook by editing its factory (PlanMoE/custom/comm/abstract.h:10-24,
// PlanMoE/custom/custom_kernel.cpp:209-224, README.md:57-71); here registration replaces the edit, and
// the constructor receives the symmetric-heap view instead of NCCL communicators and streams.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace planmoe {

// What a comm object knows about the job.  heap_bases: device array [world_size] of peer-mapped
// heap base addresses (null in a one-rank world), rank r's copy of the heap starts at heap_bases[r];
// local_base: this rank's own base as a host-visible number; scratch_off / scratch_bytes: a zero-initialised
// block of the heap reserved for this comm object, at the same offset on every rank, to lay out as it likes
// (staging buffers, u64 flags, message tables); status: host-mapped int32[8] that bounded waits report to;
// budget_ns: how long a device-side wait may last.
struct CommContext {
  const unsigned long long* heap_bases = nullptr;
  unsigned long long local_base = 0;
  unsigned long long scratch_off = 0, scratch_bytes = 0;
  int world_size = 1, world_rank = 0, local_size = 1, local_rank = 0;
  int* status = nullptr;
  unsigned long long budget_ns = 20000000000ull;
};

class AbstractComm {
 public:
  explicit AbstractComm(const CommContext& ctx) : ctx_(ctx) {}
  virtual ~AbstractComm() = default;
  // Heap bytes an object of this class wants reserved for payloads of `payload_bytes` per call (asked on a
  // throw-away instance before the real one is built with a block of that size).
  virtual size_t scratch_bytes_for(size_t payload_bytes) const { return 2 * payload_bytes + (64u << 10); }
  // `in` holds world_size equal parts of bytes / world_size, part j for rank j; `out` receives the
  // parts of all source ranks in rank order.  Enqueue on `stream`; do not synchronise.
  virtual void all_to_all(const void* in, void* out, size_t bytes, cudaStream_t stream) = 0;
  // Optional hook that runs on the data before compression (the reference's pre_comm).
  virtual void pre_comm(void* /*data*/, size_t /*bytes*/, cudaStream_t /*stream*/) {}
  const CommContext& context() const { return ctx_; }

 protected:
  CommContext ctx_;
};

using CommFactory = std::function<std::unique_ptr<AbstractComm>(const CommContext&)>;

// Registry (lives in _C.so).  Later registrations under the same name win.
void register_comm(const std::string& name, CommFactory factory);
bool has_comm(const std::string& name);
std::unique_ptr<AbstractComm> make_comm(const std::string& name, const CommContext& ctx);
std::vector<std::string> comm_names();

struct CommRegistrar {
  CommRegistrar(const std::string& name, CommFactory f) { register_comm(name, std::move(f)); }
};

}  // namespace planmoe
