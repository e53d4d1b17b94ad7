// Registries of the C++ extension points and built-ins written against them: comms "native_flat" (flat push
// all-to-all) and "native_pipe" (Pipe-A2A), both on the generic transfer kernel, and codec "native_copy"
// (identity codec).

#include "comm/abstract.h"
#include "codec/abstract.h"
#include "planmoe.h"

#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>

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

// Flat all-to-all written against the extension interface alone: a message table for the generic transfer
// kernel (planmoe::launch_xfer), staging buffers and flags laid out in the object's scratch block.
//
// Scratch layout (every rank the same):  [0, 1 KiB) u64 flags [2 parities][W]  |  [1 KiB, 1 KiB + table area)
// message tables and the wait index list  |  staging buffers [2 parities][W][n] for n bytes per pair.
// Call k uses parity k & 1.  A rank can only be two calls ahead of a peer when that peer has finished reading the
// older staging buffer (an all-to-all completes nowhere before every rank has entered it), so two parities
// suffice; flags are cumulative arrival counters and never reset.
class NativeFlatComm : public AbstractComm {
 public:
  using AbstractComm::AbstractComm;
  ~NativeFlatComm() override {
    for (auto& s : side_) if (s) cudaStreamDestroy(s);
    for (auto& e : ev_) if (e) cudaEventDestroy(e);
  }
  size_t scratch_bytes_for(size_t payload_bytes) const override {
    return kFlagArea + table_area() + 2 * ((payload_bytes + 1023) / 1024 * 1024);
  }
  void all_to_all(const void* in, void* out, size_t bytes, cudaStream_t stream) override {
    const int W = ctx_.world_size;
    if (W == 1) {
      if (in != out) copy_bytes(out, in, bytes, stream);
      return;
    }
    if (bytes % ((size_t)W * 16) != 0) throw std::runtime_error("native comm: per-pair payload must be a multiple of 16 bytes");
    const size_t n = bytes / W;
    if (kFlagArea + table_area() + 2 * bytes > ctx_.scratch_bytes)
      throw std::runtime_error("native comm: scratch block too small for this payload");
    const int parity = (int)(calls_ & 1);
    ++calls_;
    if (n != table_n_) build_tables(n, stream);
    const int ctas = ctas_for(n);
    arrived_[parity] += (unsigned long long)ctas;                 // one message per source, `ctas` CTAs each
    const unsigned long long flag_off = ctx_.scratch_off + (unsigned long long)parity * W * 8;
    const unsigned long long* local_flags =
        reinterpret_cast<const unsigned long long*>(ctx_.local_base + flag_off);
    push(in, parity, ctas, flag_off, stream);
    // copy-out: the slice from source s waits for flag s only
    const unsigned char* staging = reinterpret_cast<const unsigned char*>(ctx_.local_base + staging_off(parity, n));
    launch_xfer(staging, table(kOut), W, ctas, ctx_.heap_bases, 0, local_flags, wait_idx(), W, arrived_[parity],
                ctx_.budget_ns, ctx_.status, out, stream);
  }

 protected:
  enum { kPushAll = 0, kPushIntra = 2, kPushInter = 4, kOut = 6 };    // table slots (push tables exist per parity)
  static constexpr size_t kFlagArea = 1024;
  size_t table_area() const { return (size_t)8 * ctx_.world_size * 48 + 4096; }
  unsigned long long staging_off(int parity, size_t n) const {
    return ctx_.scratch_off + kFlagArea + table_area() + (unsigned long long)parity * ctx_.world_size * n;
  }
  const long long* table(int slot) const {
    return reinterpret_cast<const long long*>(ctx_.local_base + ctx_.scratch_off + kFlagArea + (size_t)slot * ctx_.world_size * 48);
  }
  const int* wait_idx() const {
    return reinterpret_cast<const int*>(ctx_.local_base + ctx_.scratch_off + kFlagArea + (size_t)8 * ctx_.world_size * 48);
  }
  int ctas_for(size_t n) const {
    long long c = (long long)(n >> 16);
    const long long cap = 592 / ctx_.world_size;
    if (c > cap) c = cap;
    return c < 1 ? 1 : (int)c;
  }
  int n_intra_ = 0, n_inter_ = 0;

  // Message = (dest rank or -1, flag index to signal or -1, src_off, dst_off, bytes, wait_one or -1).
  void build_tables(size_t n, cudaStream_t stream) {
    const int W = ctx_.world_size, L = ctx_.local_size > 0 ? ctx_.local_size : W, me = ctx_.world_rank;
    host_.assign((size_t)8 * W * 6, 0);
    n_intra_ = n_inter_ = 0;
    for (int parity = 0; parity < 2; ++parity) {
      int ia = 0, ib = 0;
      for (int d = 0; d < W; ++d) {
        const long long m[6] = {d, me, (long long)(d * n), (long long)(staging_off(parity, n) + me * n), (long long)n, -1};
        std::memcpy(&host_[((size_t)(kPushAll + parity) * W + d) * 6], m, sizeof(m));
        const bool intra = (d / L) == (me / L);
        long long* dst = intra ? &host_[((size_t)(kPushIntra + parity) * W + ia++) * 6]
                               : &host_[((size_t)(kPushInter + parity) * W + ib++) * 6];
        std::memcpy(dst, m, sizeof(m));
      }
      n_intra_ = ia; n_inter_ = ib;
    }
    for (int s = 0; s < W; ++s) {
      const long long m[6] = {-1, -1, (long long)(s * n), (long long)(s * n), (long long)n, s};
      std::memcpy(&host_[((size_t)kOut * W + s) * 6], m, sizeof(m));
    }
    widx_.resize(W);
    for (int s = 0; s < W; ++s) widx_[s] = s;
    void* tab = reinterpret_cast<void*>(ctx_.local_base + ctx_.scratch_off + kFlagArea);
    // tables of an earlier payload size may still be read by launches in flight: order the upload behind them
    cudaStreamSynchronize(stream);
    cudaMemcpyAsync(tab, host_.data(), host_.size() * sizeof(long long), cudaMemcpyHostToDevice, stream);
    cudaMemcpyAsync(const_cast<int*>(wait_idx()), widx_.data(), widx_.size() * sizeof(int), cudaMemcpyHostToDevice, stream);
    cudaStreamSynchronize(stream);
    table_n_ = n;
  }
  virtual void push(const void* in, int parity, int ctas, unsigned long long flag_off, cudaStream_t stream) {
    launch_xfer(in, table(kPushAll + parity), ctx_.world_size, ctas, ctx_.heap_bases, flag_off, nullptr, nullptr, 0, 0,
                ctx_.budget_ns, ctx_.status, nullptr, stream);
  }
  void ensure_side() {
    if (side_[0] != nullptr) return;
    for (auto& s : side_) cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    for (auto& e : ev_) cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
  }
  cudaStream_t side_[2] = {nullptr, nullptr};
  cudaEvent_t ev_[3] = {nullptr, nullptr, nullptr};

 private:
  unsigned long long calls_ = 0, arrived_[2] = {0, 0};
  size_t table_n_ = 0;
  std::vector<long long> host_;
  std::vector<int> widx_;
};

// Pipe-A2A on the same interface: the messages for peers inside my group (LOCAL_SIZE consecutive ranks) and for
// peers outside it leave as two launches on two streams, so the two classes of traffic progress independently
// (reference: PlanMoE/custom/comm/pipe.cpp:12-31, which uses two NCCL communicators and streams).
class NativePipeComm : public NativeFlatComm {
 public:
  using NativeFlatComm::NativeFlatComm;

 protected:
  void push(const void* in, int parity, int ctas, unsigned long long flag_off, cudaStream_t stream) override {
    if (n_inter_ == 0 || n_intra_ == 0) { NativeFlatComm::push(in, parity, ctas, flag_off, stream); return; }
    ensure_side();
    cudaEventRecord(ev_[0], stream);
    const int counts[2] = {n_intra_, n_inter_};
    const int slots[2] = {kPushIntra + parity, kPushInter + parity};
    for (int i = 0; i < 2; ++i) {
      cudaStreamWaitEvent(side_[i], ev_[0], 0);
      launch_xfer(in, table(slots[i]), counts[i], ctas, ctx_.heap_bases, flag_off, nullptr, nullptr, 0, 0, ctx_.budget_ns,
                  ctx_.status, nullptr, side_[i]);
      cudaEventRecord(ev_[1 + i], side_[i]);
      cudaStreamWaitEvent(stream, ev_[1 + i], 0);
    }
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
CommRegistrar reg_pipe("native_pipe", [](const CommContext& c) {
  return std::unique_ptr<AbstractComm>(new NativePipeComm(c));
});
CompressorRegistrar reg_copy("native_copy", [] { return std::unique_ptr<AbstractCompressor>(new NativeCopyCodec()); });

}  // namespace
}  // namespace planmoe
