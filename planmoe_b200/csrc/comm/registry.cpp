// Registries of the C++ extension points and two built-ins that exercise them:
// comm "native_flat" (flat push all-to-all through the generic transfer kernel; identity in a
// one-rank world) and codec "native_copy" (identity codec).

#include "comm/abstract.h"
#include "codec/abstract.h"
#include "planmoe.h"

#include <cstring>
#include <map>
#include <mutex>

namespace planmoe {

namespace {
std::mutex& mu() { static std::mutex m; return m; }
std::map<std::string, CommFactory>& comms() { static std::map<std::string, CommFactory> m; return m; }
std::map<std::string, CompressorFactory>& codecs() { static std::map<std::string, CompressorFactory> m; return m; }
}  // namespace

void register_comm(const std::string& name, CommFactory f) {
  std::lock_guard<std::mutex> l(mu());
  comms()[name] = std::move(f);
}
bool has_comm(const std::string& name) {
  std::lock_guard<std::mutex> l(mu());
  return comms().count(name) != 0;
}
std::unique_ptr<AbstractComm> make_comm(const std::string& name, const CommContext& ctx) {
  CommFactory f;
  {
    std::lock_guard<std::mutex> l(mu());
    auto it = comms().find(name);
    if (it == comms().end()) return nullptr;
    f = it->second;
  }
  return f(ctx);
}
std::vector<std::string> comm_names() {
  std::lock_guard<std::mutex> l(mu());
  std::vector<std::string> v;
  for (auto& kv : comms()) v.push_back(kv.first);
  return v;
}

void register_compressor(const std::string& name, CompressorFactory f) {
  std::lock_guard<std::mutex> l(mu());
  codecs()[name] = std::move(f);
}
bool has_compressor(const std::string& name) {
  std::lock_guard<std::mutex> l(mu());
  return codecs().count(name) != 0;
}
std::unique_ptr<AbstractCompressor> make_compressor(const std::string& name) {
  CompressorFactory f;
  {
    std::lock_guard<std::mutex> l(mu());
    auto it = codecs().find(name);
    if (it == codecs().end()) return nullptr;
    f = it->second;
  }
  return f();
}
std::vector<std::string> compressor_names() {
  std::lock_guard<std::mutex> l(mu());
  std::vector<std::string> v;
  for (auto& kv : codecs()) v.push_back(kv.first);
  return v;
}

namespace {

// Copy that works for device and host pointers alike, also on a machine without a GPU.
void copy_bytes(void* dst, const void* src, size_t n, cudaStream_t s) {
  if (cudaMemcpyAsync(dst, src, n, cudaMemcpyDefault, s) != cudaSuccess) {
    (void)cudaGetLastError();
    std::memcpy(dst, src, n);
  }
}

// Identity in a one-rank world; otherwise a plain device-to-device copy of each part into the
// caller-provided output is not possible without the peers' cooperation, so multi-rank use goes
// through the Python transport.  The class shows the shape of a user comm.
class NativeFlatComm : public AbstractComm {
 public:
  using AbstractComm::AbstractComm;
  void all_to_all(const void* in, void* out, size_t bytes, cudaStream_t stream) override {
    if (ctx_.world_size == 1) {
      if (in != out) copy_bytes(out, in, bytes, stream);
      return;
    }
    // multi-rank: the Python side supplies message tables to launch_xfer (see parallel/a2a.py)
  }
};

class NativeCopyCodec : public AbstractCompressor {
 public:
  size_t wire_bytes(size_t bytes, int) const override { return bytes; }
  void compress(const void* in, void* wire, size_t bytes, int, int, size_t, cudaStream_t s) override {
    copy_bytes(wire, in, bytes, s);
  }
  void decompress(const void* wire, void* out, size_t bytes, int, int, size_t, cudaStream_t s) override {
    copy_bytes(out, wire, bytes, s);
  }
};

CommRegistrar reg_flat("native_flat", [](const CommContext& c) {
  return std::unique_ptr<AbstractComm>(new NativeFlatComm(c));
});
CompressorRegistrar reg_copy("native_copy", [] { return std::unique_ptr<AbstractCompressor>(new NativeCopyCodec()); });

}  // namespace
}  // namespace planmoe
