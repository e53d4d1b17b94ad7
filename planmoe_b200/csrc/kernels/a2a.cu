// Generic "wait, copy to peers, signal" kernel: the building block of every stand-alone
// all-to-all algorithm (flat, Pipe-A2A, HeTu-hierarchical, 2DH) of the symmetric-heap transport.
//
// One launch executes a table of messages.  CTA (i, m) first acquire-waits (bounded) on the listed
// local flags, then copies slice i of message m with 16-byte loads/stores from local memory to
//   heap_bases[dest] + dst_off     (a peer's or this rank's heap), or
//   local_dst + dst_off            (dest < 0: plain local output tensor),
// and finally, if the message carries a flag index, issues a system-scope fence and a release-add
// on that flag in the destination rank's heap.  Layout transforms of the hierarchical algorithms
// are folded into the (src_off, dst_off) pairs, so no staging transpose kernels exist
// (reference: PlanMoE/custom/comm/layout_transform.cu:3-83 and the memStrideCopy kernels of
// PlanMoE/custom/jit.h:301-312).  The ncclSend/ncclRecv groups of custom/comm/{naive,pipe,hetu}.cpp
// and custom/dd_comm.cpp become tables for this kernel.

#include "planmoe.h"
#include "kernels/common.cuh"

namespace planmoe {

__global__ void __launch_bounds__(256)
xfer_kernel(const unsigned char* __restrict__ src_base, const long long* __restrict__ msgs, int n_msgs,
            const unsigned long long* __restrict__ heap_bases, unsigned long long flag_off,
            const unsigned long long* __restrict__ wait_flags, const int* __restrict__ wait_idx, int n_wait,
            unsigned long long want, unsigned long long budget_ns, int* status, unsigned char* local_dst) {
  __shared__ int ok_s;
  if (n_wait > 0) {
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    for (int f = threadIdx.x; f < n_wait; f += blockDim.x) {
      if (!wait_flag_ge(wait_flags + wait_idx[f], want, budget_ns, status, wait_idx[f])) ok_s = 0;
    }
    __syncthreads();
    if (!ok_s) return;
  }
  const int m = blockIdx.y;
  if (m >= n_msgs) return;
  const long long dest = msgs[m * 5 + 0];
  const long long flag_idx = msgs[m * 5 + 1];
  const unsigned long long src_off = (unsigned long long)msgs[m * 5 + 2];
  const unsigned long long dst_off = (unsigned long long)msgs[m * 5 + 3];
  const unsigned long long bytes = (unsigned long long)msgs[m * 5 + 4];

  const uint4* src = reinterpret_cast<const uint4*>(src_base + src_off);
  unsigned char* dbase = dest >= 0 ? reinterpret_cast<unsigned char*>(heap_bases[dest]) : local_dst;
  uint4* dst = reinterpret_cast<uint4*>(dbase + dst_off);
  const unsigned long long nvec = bytes >> 4;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  // 4 independent 16-byte transfers in flight per thread
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
  }
  for (; i < nvec; i += stride) dst[i] = src[i];

  if (flag_idx >= 0 && dest >= 0) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      unsigned long long* flags = reinterpret_cast<unsigned long long*>(
          reinterpret_cast<unsigned char*>(heap_bases[dest]) + flag_off);
      red_release_sys_add(flags + flag_idx, 1ull);
    }
  }
}

void launch_xfer(const void* src_base, const long long* msgs, int n_msgs, int ctas_per_msg,
                 const unsigned long long* heap_bases, unsigned long long flag_off,
                 const unsigned long long* wait_flags, const int* wait_idx, int n_wait, unsigned long long want,
                 unsigned long long budget_ns, int* status, void* local_dst, cudaStream_t stream) {
  if (n_msgs <= 0) return;
  if (ctas_per_msg < 1) ctas_per_msg = 1;
  dim3 grid(ctas_per_msg, n_msgs);
  xfer_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const unsigned char*>(src_base), msgs, n_msgs, heap_bases,
                                      flag_off, wait_flags, wait_idx, n_wait, want, budget_ns, status,
                                      reinterpret_cast<unsigned char*>(local_dst));
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

}  // namespace planmoe
