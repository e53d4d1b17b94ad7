// CPU C++ reference loops for the three sparse dispatch primitives (fp32 / fp64).
//
// They are the oracle for the CUDA kernels and the CPU execution path of the MoE layer
// (the reference's counterpart is invoke_cpu<T>, PlanMoE/custom/custom_kernel.cpp:57-112).
// Layout: x[S][M], disp[E*C][M], idx/loc[K][S], gates[K][S] (may be null = weight 1).
// A (token, choice) with idx < 0 or loc outside [0, C) is dropped.

#include "planmoe.h"

#include <cstring>

namespace planmoe {

template <class T>
void cpu_scatter(const T* x, const int* idx, const int* loc, const T* gates, T* disp,
                 int K, int S, int M, int E, int C) {
  std::memset(disp, 0, sizeof(T) * (size_t)E * C * M);
  for (int k = 0; k < K; ++k) {
    for (int t = 0; t < S; ++t) {
      const int e = idx[(size_t)k * S + t], l = loc[(size_t)k * S + t];
      if (e < 0 || e >= E || l < 0 || l >= C) continue;
      const T g = gates ? gates[(size_t)k * S + t] : T(1);
      T* dst = disp + ((size_t)e * C + l) * M;
      const T* src = x + (size_t)t * M;
      for (int j = 0; j < M; ++j) dst[j] += g * src[j];
    }
  }
}

template <class T>
void cpu_gather(const T* disp, const int* idx, const int* loc, const T* gates, T* out,
                int K, int S, int M, int C) {
  std::memset(out, 0, sizeof(T) * (size_t)S * M);
  for (int k = 0; k < K; ++k) {
    for (int t = 0; t < S; ++t) {
      const int e = idx[(size_t)k * S + t], l = loc[(size_t)k * S + t];
      if (e < 0 || l < 0 || l >= C) continue;
      const T g = gates ? gates[(size_t)k * S + t] : T(1);
      const T* src = disp + ((size_t)e * C + l) * M;
      T* dst = out + (size_t)t * M;
      for (int j = 0; j < M; ++j) dst[j] += g * src[j];
    }
  }
}

template <class T>
void cpu_gate_grad(const T* disp, const T* dy, const int* idx, const int* loc, T* dgates,
                   int K, int S, int M, int C) {
  for (int k = 0; k < K; ++k) {
    for (int t = 0; t < S; ++t) {
      const int e = idx[(size_t)k * S + t], l = loc[(size_t)k * S + t];
      T acc = T(0);
      if (!(e < 0 || l < 0 || l >= C)) {
        const T* a = disp + ((size_t)e * C + l) * M;
        const T* b = dy + (size_t)t * M;
        for (int j = 0; j < M; ++j) acc += a[j] * b[j];
      }
      dgates[(size_t)k * S + t] = acc;
    }
  }
}

#define INSTANTIATE(T)                                                                         \
  template void cpu_scatter<T>(const T*, const int*, const int*, const T*, T*, int, int, int,  \
                               int, int);                                                      \
  template void cpu_gather<T>(const T*, const int*, const int*, const T*, T*, int, int, int,   \
                              int);                                                            \
  template void cpu_gate_grad<T>(const T*, const T*, const int*, const int*, T*, int, int,     \
                                 int, int);
INSTANTIATE(float)
INSTANTIATE(double)

}  // namespace planmoe
