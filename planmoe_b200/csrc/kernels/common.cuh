// Device-side helpers shared by the SIMT kernels: 16-byte vector access, dtype conversion,
// warp reductions, system-scope flag access with bounded waits.
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

}  // namespace planmoe
