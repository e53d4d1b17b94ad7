// Stand-alone int8 row-affine codec kernels (sm_100a).
//
//   encode: per row r of [R, M]: lo = min, range = max - lo, q = round((x - lo) * 255 / range)
//   decode: x = q * range / 255 + lo
//
// One warp per row, 16-byte accesses, a single pass after the min/max reduction (the row is
// re-read from L1/L2).  Replaces the reference's chains of 8 + 5 ATen launches
// (PlanMoE/custom/compressor/int8.cpp:10-24, :47-59); unlike those, a constant row (range 0)
// is guarded and quantisation rounds to nearest.  The same arithmetic is fused into the
// dispatch send kernel (kernels/dispatch.cu, QUANT = true).

#include "planmoe.h"
#include "kernels/common.cuh"

namespace planmoe {

template <class T>
__global__ void __launch_bounds__(256)
int8_encode_kernel(const T* __restrict__ x, unsigned char* __restrict__ q, float* __restrict__ scale,
                   float* __restrict__ bias, int R, int M) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int V = Vec16<T>::N;
  for (int r = blockIdx.x * 8 + warp; r < R; r += gridDim.x * 8) {
    const T* src = x + (size_t)r * M;
    float lo = INFINITY, hi = -INFINITY;
    if (M % 16 == 0) {
      for (int v = lane; v < M / V; v += 32) {
        Pack<T> p = ld16(src + v * V);
#pragma unroll
        for (int i = 0; i < V; ++i) { float f = to_f32(p.v[i]); lo = fminf(lo, f); hi = fmaxf(hi, f); }
      }
    } else {
      for (int j = lane; j < M; j += 32) { float f = to_f32(src[j]); lo = fminf(lo, f); hi = fmaxf(hi, f); }
    }
    lo = warp_min(lo); hi = warp_max(hi);
    const float range = hi - lo;
    const float inv = range > 0.f ? 255.f / range : 0.f;
    unsigned char* dst = q + (size_t)r * M;
    if (M % 16 == 0) {
      for (int v = lane; v < M / 16; v += 32) {
        alignas(16) unsigned char o[16];
#pragma unroll
        for (int h = 0; h < 16 / V; ++h) {
          Pack<T> p = ld16(src + (size_t)v * 16 + h * V);
#pragma unroll
          for (int i = 0; i < V; ++i)
            o[h * V + i] = (unsigned char)fminf(fmaxf(rintf((to_f32(p.v[i]) - lo) * inv), 0.f), 255.f);
        }
        reinterpret_cast<uint4*>(dst)[v] = *reinterpret_cast<uint4*>(o);
      }
    } else {
      for (int j = lane; j < M; j += 32)
        dst[j] = (unsigned char)fminf(fmaxf(rintf((to_f32(src[j]) - lo) * inv), 0.f), 255.f);
    }
    if (lane == 0) { scale[r] = range; bias[r] = lo; }
  }
}

template <class T>
__global__ void __launch_bounds__(256)
int8_decode_kernel(const unsigned char* __restrict__ q, const float* __restrict__ scale,
                   const float* __restrict__ bias, T* __restrict__ out, int R, int M) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int V = Vec16<T>::N;
  for (int r = blockIdx.x * 8 + warp; r < R; r += gridDim.x * 8) {
    const float s = scale[r] * (1.f / 255.f), b = bias[r];
    const unsigned char* src = q + (size_t)r * M;
    T* dst = out + (size_t)r * M;
    if (M % 16 == 0) {
      for (int v = lane; v < M / 16; v += 32) {
        uint4 raw = reinterpret_cast<const uint4*>(src)[v];
        const unsigned char* qq = reinterpret_cast<const unsigned char*>(&raw);
#pragma unroll
        for (int h = 0; h < 16 / V; ++h) {
          Pack<T> o;
#pragma unroll
          for (int i = 0; i < V; ++i) o.v[i] = from_f32<T>((float)qq[h * V + i] * s + b);
          st16(dst + (size_t)v * 16 + h * V, o);
        }
      }
    } else {
      for (int j = lane; j < M; j += 32) dst[j] = from_f32<T>((float)src[j] * s + b);
    }
  }
}

// Wire rows of the fused MoE send: row r of [R, M] becomes M bytes of uint8 followed by the 16-byte trailer
// {(max - min) / 255, min, 0, 0}, i.e. rows of M + 16 bytes that travel as one piece and de-quantise as
// q * trailer[0] + trailer[1].  M must be a multiple of 16.
template <class T>
__global__ void __launch_bounds__(256)
int8_rows_encode_kernel(const T* __restrict__ x, unsigned char* __restrict__ out, int R, int M) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int V = Vec16<T>::N;
  const size_t out_stride = (size_t)M + 16;
  for (int r = blockIdx.x * 8 + warp; r < R; r += gridDim.x * 8) {
    const T* src = x + (size_t)r * M;
    float lo = INFINITY, hi = -INFINITY;
    for (int v = lane; v < M / V; v += 32) {
      Pack<T> p = ld16(src + v * V);
#pragma unroll
      for (int i = 0; i < V; ++i) { float f = to_f32(p.v[i]); lo = fminf(lo, f); hi = fmaxf(hi, f); }
    }
    lo = warp_min(lo); hi = warp_max(hi);
    const float range = hi - lo;
    const float inv = range > 0.f ? 255.f / range : 0.f;
    unsigned char* dst = out + (size_t)r * out_stride;
    for (int v = lane; v < M / 16; v += 32) {
      alignas(16) unsigned char o[16];
#pragma unroll
      for (int h = 0; h < 16 / V; ++h) {
        Pack<T> p = ld16(src + (size_t)v * 16 + h * V);
#pragma unroll
        for (int i = 0; i < V; ++i)
          o[h * V + i] = (unsigned char)fminf(fmaxf(rintf((to_f32(p.v[i]) - lo) * inv), 0.f), 255.f);
      }
      reinterpret_cast<uint4*>(dst)[v] = *reinterpret_cast<uint4*>(o);
    }
    if (lane == 0) *reinterpret_cast<float4*>(dst + M) = make_float4(range * (1.f / 255.f), lo, 0.f, 0.f);
  }
}

template <class T>
void launch_int8_rows_encode(const T* x, unsigned char* out, int R, int M, cudaStream_t stream) {
  int ctas = (R + 7) / 8;
  if (ctas > 148 * 8) ctas = 148 * 8;
  if (ctas < 1) return;
  int8_rows_encode_kernel<T><<<ctas, 256, 0, stream>>>(x, out, R, M);
}

template <class T>
void launch_int8_encode(const T* x, unsigned char* q, float* scale, float* bias, int R, int M,
                        cudaStream_t stream) {
  int ctas = (R + 7) / 8;
  if (ctas > 148 * 8) ctas = 148 * 8;
  if (ctas < 1) return;
  int8_encode_kernel<T><<<ctas, 256, 0, stream>>>(x, q, scale, bias, R, M);
}
template <class T>
void launch_int8_decode(const unsigned char* q, const float* scale, const float* bias, T* out, int R,
                        int M, cudaStream_t stream) {
  int ctas = (R + 7) / 8;
  if (ctas > 148 * 8) ctas = 148 * 8;
  if (ctas < 1) return;
  int8_decode_kernel<T><<<ctas, 256, 0, stream>>>(q, scale, bias, out, R, M);
}

#define INSTANTIATE(T)                                                                          \
  template void launch_int8_encode<T>(const T*, unsigned char*, float*, float*, int, int,        \
                                      cudaStream_t);                                            \
  template void launch_int8_decode<T>(const unsigned char*, const float*, const float*, T*, int, \
                                      int, cudaStream_t);                                       \
  template void launch_int8_rows_encode<T>(const T*, unsigned char*, int, int, cudaStream_t);
INSTANTIATE(float)
INSTANTIATE(__nv_bfloat16)
INSTANTIATE(__half)

}  // namespace planmoe
