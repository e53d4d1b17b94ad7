// Allocation-free column-sum entry point.  This entry point has no counterpart in the reference.
//
// Who needs it: code that runs where device allocation is forbidden or impossible — a region
// being captured into a CUDA graph, a real-time serving loop that must not touch the allocator
// (cudaMalloc synchronises the device and can fail under memory pressure), or a host program
// written in C that links this library without libtorch and therefore has no caching allocator to
// borrow scratch from.  The regular path (`colsum` in the Python module) takes its scratch from
// torch's allocator on every call; this one keeps the scratch inside the library image.
//
//   out[g][n] = sum over r of x[g][r][n]      x: bf16, out: fp32 [groups][N]
//
// Scratch: one file-scope device array of PLANMOE_COLSUM_NOALLOC_MAX_FLOATS floats (4 MiB).  Every
// GPU that loads the library holds that array until the process exits.  A call needs
// groups * ceil(rows / 256) * N scratch floats; larger problems are rejected with
// PLANMOE_NOALLOC_TOO_LARGE and nothing is launched.
//
// Set-up: the first call on each device resolves the array's device address (the array's name
// is only a host-side handle; it is not an address a kernel can use) and caches it for that device.
// That first call must therefore be made with the target device current and should be made
// before any stream capture begins.
//
// Sharing: all calls on one device use the same scratch.  Calls must not overlap on the GPU —
// issue them on one stream, or order them with events.  The scratch is fully rewritten by every
// call before it is read, so nothing needs clearing between calls.
//
// The function calls no cudaMalloc / cudaFree and no allocating library routine.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PLANMOE_COLSUM_NOALLOC_MAX_FLOATS (1u << 20)

enum {
  PLANMOE_NOALLOC_OK = 0,
  PLANMOE_NOALLOC_BAD_ARGUMENT = 1,   // null pointer, non-positive extent, odd N, misaligned x
  PLANMOE_NOALLOC_TOO_LARGE = 2,      // needs more scratch than the built-in array holds
  PLANMOE_NOALLOC_CUDA_ERROR = 3,     // symbol lookup or launch failed (see planmoe_colsum_noalloc_last_cuda_error)
  PLANMOE_NOALLOC_PENDING_ERROR = 4,  // an earlier CUDA error of this thread was still pending: nothing was launched
};

// x: device pointer to bf16, element strides `row_stride` / `group_stride`; out: device pointer to
// groups * N floats; stream: a cudaStream_t (0 = default stream).  Returns one of the codes above.
int planmoe_colsum_bf16_noalloc(const void* x, float* out, int groups, long long rows, int N,
                                long long row_stride, long long group_stride, void* stream);

// cudaError_t value of the most recent PLANMOE_NOALLOC_CUDA_ERROR on this thread (0 if none).
int planmoe_colsum_noalloc_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
