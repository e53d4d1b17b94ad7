// Column sums of a bf16 [groups][rows][N] tensor with library-owned scratch (see the header for
// who this is for and what the limits are).  Two-stage reduction in a fixed order: slabs of 256
// rows, then the slab partials in slab order, so results are reproducible run to run.

#include "kernels/colsum_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

namespace {

constexpr int kSlab = 256;          // rows reduced by one CTA
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is a handle for cudaGetSymbolAddress, not a pointer.
static __device__ __align__(256) float g_scratch[PLANMOE_COLSUM_NOALLOC_MAX_FLOATS];

std::mutex g_mu;
float* g_scratch_addr[kMaxDevices] = {};     // per-device address of g_scratch, filled on first use
thread_local int t_last_cuda_error = 0;

__global__ void __launch_bounds__(256)
noalloc_partial_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ partial, long long rows, int N,
                       long long row_stride, long long group_stride, int slabs) {
  const int col = (blockIdx.x * 256 + threadIdx.x) * 2;
  if (col >= N) return;
  const int slab = blockIdx.y, g = blockIdx.z;
  const long long r0 = (long long)slab * kSlab;
  const long long r1 = r0 + kSlab < rows ? r0 + kSlab : rows;
  const __nv_bfloat16* base = x + (long long)g * group_stride + col;
  float a0 = 0.f, a1 = 0.f;
  for (long long r = r0; r < r1; ++r) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(base + r * row_stride));
    a0 += f.x; a1 += f.y;
  }
  float* dst = partial + ((long long)g * slabs + slab) * N + col;
  dst[0] = a0; dst[1] = a1;
}

__global__ void noalloc_final_kernel(const float* __restrict__ partial, float* __restrict__ out, int N, int slabs) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  const int g = blockIdx.y;
  if (col >= N) return;
  float acc = 0.f;
  for (int s = 0; s < slabs; ++s) acc += partial[((long long)g * slabs + s) * N + col];
  out[(long long)g * N + col] = acc;
}

// Device address of the scratch array on the current device; resolved once per device.
cudaError_t scratch_for_current_device(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[dev] = p;
  }
  *ptr = g_scratch_addr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int planmoe_colsum_bf16_noalloc(const void* x, float* out, int groups, long long rows, int N,
                                           long long row_stride, long long group_stride, void* stream) {
  if (x == nullptr || out == nullptr || groups <= 0 || rows <= 0 || N <= 0 || (N & 1) ||
      (reinterpret_cast<uintptr_t>(x) & 3) || (row_stride & 1) || (group_stride & 1))
    return PLANMOE_NOALLOC_BAD_ARGUMENT;
  const long long slabs = (rows + kSlab - 1) / kSlab;
  const long long need = (long long)groups * slabs * N;
  if (need > (long long)PLANMOE_COLSUM_NOALLOC_MAX_FLOATS || slabs > 65535 || groups > 65535)
    return PLANMOE_NOALLOC_TOO_LARGE;

  // An error left behind by earlier work of this thread is the caller's to handle: report it as such instead of
  // launching and then mistaking it for a failure of this call.
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) { t_last_cuda_error = (int)e; return PLANMOE_NOALLOC_PENDING_ERROR; }

  float* scratch = nullptr;
  e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) { t_last_cuda_error = (int)e; return PLANMOE_NOALLOC_CUDA_ERROR; }

  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  dim3 g1((N / 2 + 255) / 256, (unsigned)slabs, (unsigned)groups);
  noalloc_partial_kernel<<<g1, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), scratch, rows, N, row_stride,
                                          group_stride, (int)slabs);
  dim3 g2((N + 255) / 256, (unsigned)groups);
  noalloc_final_kernel<<<g2, 256, 0, s>>>(scratch, out, N, (int)slabs);
  e = cudaGetLastError();
  if (e != cudaSuccess) { t_last_cuda_error = (int)e; return PLANMOE_NOALLOC_CUDA_ERROR; }
  return PLANMOE_NOALLOC_OK;
}

extern "C" int planmoe_colsum_noalloc_last_cuda_error(void) { return t_last_cuda_error; }
