// An all-to-all algorithm written OUTSIDE the library against its C++ extension point
// (planmoe_b200/csrc/comm/abstract.h): a flat exchange that serves the farthest peer first.  It uses nothing
// but the CommContext it is given and the exported transfer kernel launcher planmoe::launch_xfer:
// staging buffers and flags live in the scratch block of the symmetric heap, two parities deep.
// tests/test_user_comm.py compiles this file, loads it next to _C.so and runs a MoE layer with
// comm_name="user_reverse".
#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>
#include <vector>

#include "comm/abstract.h"
#include "planmoe.h"

namespace {

class ReverseFlatComm : public planmoe::AbstractComm {
 public:
  using planmoe::AbstractComm::AbstractComm;
  ~ReverseFlatComm() override {
    if (tables_ != nullptr) cudaFree(tables_);
  }
  size_t scratch_bytes_for(size_t payload) const override { return 4096 + 2 * payload; }

  void all_to_all(const void* in, void* out, size_t bytes, cudaStream_t stream) override {
    const int W = ctx_.world_size, me = ctx_.world_rank;
    if (W == 1) {
      if (in != out && cudaMemcpyAsync(out, in, bytes, cudaMemcpyDefault, stream) != cudaSuccess) {
        (void)cudaGetLastError();
        std::memcpy(out, in, bytes);
      }
      return;
    }
    const size_t n = bytes / W;
    if (bytes % ((size_t)W * 16) || 4096 + 2 * bytes > ctx_.scratch_bytes) throw std::runtime_error("user comm: bad payload size");
    const int parity = (int)(calls_++ & 1);
    if (n != n_) build(n, stream);
    arrived_[parity] += 1;                                         // one CTA per message
    const unsigned long long flag_off = ctx_.scratch_off + (unsigned long long)parity * W * 8;
    const long long* push = tables_ + (size_t)parity * W * 6;
    const long long* copy_out = tables_ + (size_t)2 * W * 6;
    const int* widx = reinterpret_cast<const int*>(tables_ + (size_t)3 * W * 6);
    planmoe::launch_xfer(in, push, W, 1, ctx_.heap_bases, flag_off, nullptr, nullptr, 0, 0, ctx_.budget_ns, ctx_.status,
                         nullptr, stream);
    const unsigned char* staging = reinterpret_cast<const unsigned char*>(ctx_.local_base + staging_off(parity, n));
    planmoe::launch_xfer(staging, copy_out, W, 1, ctx_.heap_bases, 0,
                         reinterpret_cast<const unsigned long long*>(ctx_.local_base + flag_off), widx, W, arrived_[parity],
                         ctx_.budget_ns, ctx_.status, out, stream);
    (void)me;
  }

 private:
  unsigned long long staging_off(int parity, size_t n) const {
    return ctx_.scratch_off + 4096 + (unsigned long long)parity * ctx_.world_size * n;
  }
  void build(size_t n, cudaStream_t stream) {
    const int W = ctx_.world_size, me = ctx_.world_rank;
    std::vector<long long> h((size_t)3 * W * 6 + W);               // 2 push tables, 1 copy-out table, W ints (packed)
    for (int parity = 0; parity < 2; ++parity)
      for (int i = 0; i < W; ++i) {
        const int d = (me + W - 1 - i + W) % W;                    // farthest peer first, myself last
        const long long m[6] = {d, me, (long long)(d * n), (long long)(staging_off(parity, n) + me * n), (long long)n, -1};
        std::memcpy(&h[((size_t)parity * W + i) * 6], m, sizeof(m));
      }
    for (int s = 0; s < W; ++s) {
      const long long m[6] = {-1, -1, (long long)(s * n), (long long)(s * n), (long long)n, s};
      std::memcpy(&h[((size_t)2 * W + s) * 6], m, sizeof(m));
    }
    int* widx = reinterpret_cast<int*>(&h[(size_t)3 * W * 6]);
    for (int s = 0; s < W; ++s) widx[s] = s;
    cudaStreamSynchronize(stream);
    if (tables_ == nullptr) cudaMalloc(reinterpret_cast<void**>(&tables_), h.size() * sizeof(long long));
    cudaMemcpy(tables_, h.data(), h.size() * sizeof(long long), cudaMemcpyHostToDevice);
    n_ = n;
  }
  long long* tables_ = nullptr;
  size_t n_ = 0;
  unsigned long long calls_ = 0, arrived_[2] = {0, 0};
};

planmoe::CommRegistrar reg("user_reverse", [](const planmoe::CommContext& c) {
  return std::unique_ptr<planmoe::AbstractComm>(new ReverseFlatComm(c));
});

}  // namespace
