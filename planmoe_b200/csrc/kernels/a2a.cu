// Generic "wait, copy to peers, signal" kernel: the building block of every stand-alone
// all-to-all algorithm (flat, Pipe-A2A, HeTu-hierarchical, 2DH) of the symmetric-heap transport.
//
// One launch executes a table of messages.  CTA (i, m) first acquire-waits (bounded) on the local flags
// message m depends on, then moves slice i of message m through the bulk-copy engine (cp.async.bulk
// global -> shared -> global, four 16 KiB units in flight, no thread touches the data) from local memory to
//   heap_bases[dest] + dst_off     (a peer's or this rank's heap), or
//   local_dst + dst_off            (dest < 0: plain local output tensor),
// and finally, if the message carries a flag index, issues a system-scope fence and a release-add
// on that flag in the destination rank's heap.  Messages may be self-describing (`len_off >= 0`): the
// u32 at byte `len_off` of the message's source holds its payload size, and only `len_base` + that many
// bytes (rounded up to 16) are moved.  That is how the variable-length slices of the LZ codec travel
// without the host ever reading a size: the header goes with the data, hop by hop.  Layout transforms of the hierarchical algorithms
// are folded into the (src_off, dst_off) pairs, so no staging transpose kernels exist
// (reference: PlanMoE/custom/comm/layout_transform.cu:3-83 and the memStrideCopy kernels of
// PlanMoE/custom/jit.h:301-312).  The ncclSend/ncclRecv groups of custom/comm/{naive,pipe,hetu}.cpp
// and custom/dd_comm.cpp become tables for this kernel.

#include "planmoe.h"
#include "kernels/common.cuh"

namespace planmoe {

constexpr int kXferSlots = 4;                  // bulk-copy slots per CTA, one per lane of the single warp
constexpr unsigned kXferSlotBytes = 16384;

// msgs: int64 [n_msgs][6] = (dest rank or -1, flag index to signal or -1, src_off, dst_off, bytes,
// index into wait_flags this message alone depends on, or -1: every listed flag).
__global__ void __launch_bounds__(32)
xfer_kernel(const unsigned char* __restrict__ src_base, const long long* __restrict__ msgs, int n_msgs,
            const unsigned long long* __restrict__ heap_bases, unsigned long long flag_off,
            const unsigned long long* __restrict__ wait_flags, const int* __restrict__ wait_idx, int n_wait,
            unsigned long long want, unsigned long long budget_ns, int* status, unsigned char* local_dst,
            long long len_off, unsigned long long len_base) {
  extern __shared__ __align__(128) unsigned char xs[];
  __shared__ unsigned long long bars[kXferSlots];
  const int lane = threadIdx.x;
  const int m = blockIdx.y;
  if (m >= n_msgs) return;
  const long long dest = msgs[m * 6 + 0];
  const long long flag_idx = msgs[m * 6 + 1];
  const unsigned long long src_off = (unsigned long long)msgs[m * 6 + 2];
  const unsigned long long dst_off = (unsigned long long)msgs[m * 6 + 3];
  unsigned long long bytes = (unsigned long long)msgs[m * 6 + 4];
  const long long wait_one = msgs[m * 6 + 5];

  // ---- what this message reads must have arrived (bounded) --------------------------------------
  bool ok = true;
  if (n_wait > 0) {
    if (wait_one >= 0) {
      if (lane == 0) ok = wait_flag_ge(wait_flags + wait_one, want, budget_ns, status, (int)wait_one);
    } else {
      for (int f = lane; f < n_wait; f += 32)
        if (!wait_flag_ge(wait_flags + wait_idx[f], want, budget_ns, status, wait_idx[f])) ok = false;
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return;
    fence_proxy_async();                           // what peers wrote -> this CTA's bulk loads
  }
  if (lane < kXferSlots) mbar_init(smem_u32(&bars[lane]), 1);
  fence_barrier_init();
  __syncwarp();
  if (len_off >= 0) {                              // self-describing message: move the valid prefix only
    const unsigned v = *reinterpret_cast<const volatile unsigned*>(src_base + src_off + len_off);
    const unsigned long long valid = (len_base + (unsigned long long)v + 15ull) & ~15ull;
    if (valid < bytes) bytes = valid;
  }

  // ---- my slice of the message, in 16 KiB units, through the bulk-copy engine --------------------
  // Lane l owns slot l: load a unit into it, wait for the bytes, store it to the destination, and reuse
  // the slot once the store has read it.  Four units are in flight per CTA and no thread touches data.
  const unsigned long long units = (bytes + kXferSlotBytes - 1) / kXferSlotBytes;
  const unsigned long long per = (units + gridDim.x - 1) / gridDim.x;
  const unsigned long long u0 = (unsigned long long)blockIdx.x * per;
  const unsigned long long u1 = u0 + per < units ? u0 + per : units;
  const unsigned char* src = src_base + src_off;
  unsigned char* dst = (dest >= 0 ? reinterpret_cast<unsigned char*>(heap_bases[dest]) : local_dst) + dst_off;
  if (lane < kXferSlots) {
    const unsigned slot_s = smem_u32(xs + lane * kXferSlotBytes);
    const unsigned bar = smem_u32(&bars[lane]);
    unsigned phase = 0;
    for (unsigned long long u = u0 + lane; u < u1 && ok; u += kXferSlots) {
      const unsigned long long off = u * kXferSlotBytes;
      const unsigned n = (unsigned)(bytes - off < kXferSlotBytes ? bytes - off : kXferSlotBytes);
      bulk_wait_read_all();
      mbar_expect_tx(bar, n);
      bulk_load(slot_s, src + off, n, bar);
      ok = mbar_wait_bounded(bar, phase, budget_ns, status, 4, lane);
      phase ^= 1u;
      if (ok) {
        bulk_store(dst + off, slot_s, n);
        bulk_commit();
      }
    }
    bulk_wait_all();                               // my stores have been performed
  }
  ok = __all_sync(0xffffffffu, ok);

  if (ok && flag_idx >= 0 && dest >= 0) {
    // every lane's bulk stores have completed (wait_group above, then the warp vote): the data is in place, so
    // the flag update needs no release or fence of its own
    if (lane == 0) {
      unsigned long long* flags = reinterpret_cast<unsigned long long*>(
          reinterpret_cast<unsigned char*>(heap_bases[dest]) + flag_off);
      red_relaxed_sys_add(flags + flag_idx, 1ull);
    }
  }
}

void launch_xfer(const void* src_base, const long long* msgs, int n_msgs, int ctas_per_msg,
                 const unsigned long long* heap_bases, unsigned long long flag_off,
                 const unsigned long long* wait_flags, const int* wait_idx, int n_wait, unsigned long long want,
                 unsigned long long budget_ns, int* status, void* local_dst, cudaStream_t stream, long long len_off,
                 unsigned long long len_base) {
  if (n_msgs <= 0) return;
  if (ctas_per_msg < 1) ctas_per_msg = 1;
  constexpr int smem = kXferSlots * kXferSlotBytes;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(xfer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured = true;
  }
  dim3 grid(ctas_per_msg, n_msgs);
  xfer_kernel<<<grid, 32, smem, stream>>>(reinterpret_cast<const unsigned char*>(src_base), msgs, n_msgs, heap_bases,
                                        flag_off, wait_flags, wait_idx, n_wait, want, budget_ns, status,
                                        reinterpret_cast<unsigned char*>(local_dst), len_off, len_base);
}

// A kernel that only waits (used by tests of the bounded-wait path and by host code that needs a
// stream-ordered "data has arrived" point).
__global__ void wait_flags_kernel(const unsigned long long* flags, int n, unsigned long long want,
                                  unsigned long long budget_ns, int* status) {
  for (int f = threadIdx.x; f < n; f += blockDim.x) wait_flag_ge(flags + f, want, budget_ns, status, f);
}

void launch_wait_flags(const unsigned long long* flags, int n, unsigned long long want, unsigned long long budget_ns,
                       int* status, cudaStream_t stream) {
  if (n <= 0) return;
  wait_flags_kernel<<<1, 128, 0, stream>>>(flags, n, want, budget_ns, status);
}

// Occupies the stream for `ns` nanoseconds (at most 200 ms) without touching memory.  Host code that wants to
// time a burst of launches on the device enqueues this first, so that the burst is fully queued before its
// first kernel starts and runs without launch gaps.
__global__ void delay_kernel(unsigned long long ns) {
  const unsigned long long t0 = global_timer_ns();
  while (global_timer_ns() - t0 < ns) __nanosleep(1000);
}

void launch_delay(unsigned long long ns, cudaStream_t stream) {
  if (ns > 200000000ull) ns = 200000000ull;
  delay_kernel<<<1, 1, 0, stream>>>(ns);
}

}  // namespace planmoe
