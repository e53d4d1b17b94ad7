// Device-side helpers shared by the kernels: 16-byte vector access, dtype conversion, warp
// reductions, system-scope flag access with bounded waits, mbarrier and bulk-copy wrappers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace planmoe {

// Element counts per 16-byte vector.
template <class T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <class T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <class T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// A 16-byte packet of N elements of T, loadable/storable with one instruction.
template <class T>
struct alignas(16) Pack {
  T v[Vec16<T>::N];
};

template <class T>
__device__ __forceinline__ Pack<T> ld16(const T* p) {
  Pack<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <class T>
__device__ __forceinline__ void st16(T* p, const Pack<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- system-scope signalling between GPUs (flags live in peer-mapped symmetric memory) ----

__device__ __forceinline__ void red_release_sys_add(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Flag update without release semantics: for a sender whose data writes have already COMPLETED (bulk async
// stores after cp.async.bulk.wait_group), so that nothing is left for a release to order.  A release or fence
// at system scope at this point would wait for every store the SM still has in flight to other GPUs, which
// serialises a streaming sender on the link's round-trip time.
__device__ __forceinline__ void red_relaxed_sys_add(unsigned long long* p, unsigned long long v) {
  asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Error codes written to the status word (host-mapped int32[8]):
//   [0] code  [1] detail a  [2] detail b  [3] detail c
enum StatusCode : int {
  kStatusOk = 0,
  kStatusFlagTimeout = 1,      // a = flag index, b = expected low word, c = seen low word
  kStatusMbarTimeout = 2,      // a = role, b = stage / tile
  kStatusBadArgument = 3,
};

__device__ __forceinline__ void report_status(int* status, int code, int a, int b, int c) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = a; status[2] = b; status[3] = c;
    __threadfence_system();
  }
}

// Spin until *flag >= want or until budget_ns elapsed.  Returns false on timeout (and records
// it in the status word); never traps and never spins without a bound.
__device__ __forceinline__ bool wait_flag_ge(const unsigned long long* flag, unsigned long long want,
                                             unsigned long long budget_ns, int* status, int tag) {
  if (ld_acquire_sys(flag) >= want) return true;
  const unsigned long long t0 = global_timer_ns();
  unsigned ns = 32;
  while (true) {
    unsigned long long v = ld_acquire_sys(flag);
    if (v >= want) return true;
    if (global_timer_ns() - t0 > budget_ns) {
      report_status(status, kStatusFlagTimeout, tag, (int)want, (int)v);
      return false;
    }
    __nanosleep(ns);
    if (ns < 1024) ns <<= 1;
  }
}

// ---- shared-memory barriers and the bulk-copy engine (cp.async.bulk, no tensor map) ----
// Bulk copies move 16-byte-aligned byte ranges between global and shared memory without occupying
// threads: a load completes on an mbarrier (complete_tx), stores are tracked in per-thread bulk groups.
// None of these uses cluster multicast.

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }


// Bounded wait on an mbarrier phase: false once budget_ns have passed (the status word records it).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, unsigned long long budget_ns,
                                                  int* status, int role, int detail) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0u && global_timer_ns() - t0 > budget_ns) {
      report_status(status, kStatusMbarTimeout, role, detail, (int)parity);
      return false;
    }
  }
  return true;
}

}  // namespace planmoe
