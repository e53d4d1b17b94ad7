// ZFP fixed-rate 2-D and LZ codec kernels (sm_100a) plus their CPU twins.
//
// ZFP: one thread per 4x4 block; a thread reads four 4-element row segments (neighbouring threads
// read neighbouring segments, so rows are read coalesced) and writes its 2*rate-byte code word with
// 16-byte stores.  LZ: one thread per 2 KiB block for both directions, then a per-slice scan and a
// compaction copy pack the blocks back to back.  Both reuse the host/device block coders of
// codec_core.h, so the CUDA streams are bit-identical to the CPU oracle.
//
// Counterparts in the reference: libzfp calls of PlanMoE/custom/compressor/zfpc.cpp:31-51,66-85 and
// the GPULZ kernels + CUB scans of PlanMoE/custom/compressor/gpulz.cu:16-313,418-536.

#include "codec/codecs.h"
#include "codec/codec_core.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>
#include <vector>

namespace planmoe {

using namespace codec;

namespace {

__host__ __device__ inline float load_elem(const void* base, int elem, long long i) {
  if (elem == 0) return reinterpret_cast<const float*>(base)[i];
#if defined(__CUDA_ARCH__)
  if (elem == 1) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
  return __half2float(reinterpret_cast<const __half*>(base)[i]);
#else
  const uint16_t h = reinterpret_cast<const uint16_t*>(base)[i];
  if (elem == 1) {
    union { uint32_t u; float f; } v;
    v.u = (uint32_t)h << 16;
    return v.f;
  }
  return __half2float(*reinterpret_cast<const __half*>(&h));
#endif
}
__host__ __device__ inline void store_elem(void* base, int elem, long long i, float f) {
  if (elem == 0) { reinterpret_cast<float*>(base)[i] = f; return; }
  if (elem == 1) { reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(f); return; }
  reinterpret_cast<__half*>(base)[i] = __float2half_rn(f);
}

__host__ __device__ inline void zfp_block_io(bool encode, const void* x_in, void* x_out, int elem, uint8_t* stream,
                                             long long b, long long rows, long long M, int rate) {
  const long long bx = M / 4, by = (rows + 3) / 4;
  const long long per_slice = bx * by;
  const long long slice = b / per_slice, bb = b - slice * per_slice;
  const long long yb = bb / bx, xb = bb - yb * bx;
  const int words_n = rate / 2;                         // 16 * rate / 32
  uint32_t words[kZfpMaxWords];
  float f[16];
  uint32_t* dst = reinterpret_cast<uint32_t*>(stream + b * (long long)(2 * rate));
  if (encode) {
    for (int r = 0; r < 4; ++r) {
      const long long row = yb * 4 + r;
      for (int c = 0; c < 4; ++c)
        f[r * 4 + c] = row < rows ? load_elem(x_in, elem, (slice * rows + row) * M + xb * 4 + c) : 0.f;
    }
    for (int i = 0; i < words_n; ++i) words[i] = 0;
    zfp_encode_block(f, words, 16 * rate);
    for (int i = 0; i < words_n; ++i) dst[i] = words[i];
  } else {
    for (int i = 0; i < words_n; ++i) words[i] = dst[i];
    zfp_decode_block(words, f, 16 * rate);
    for (int r = 0; r < 4; ++r) {
      const long long row = yb * 4 + r;
      if (row >= rows) break;
      for (int c = 0; c < 4; ++c) store_elem(x_out, elem, (slice * rows + row) * M + xb * 4 + c, f[r * 4 + c]);
    }
  }
}

__global__ void __launch_bounds__(128)
zfp_kernel(bool encode, const void* x_in, void* x_out, int elem, uint8_t* stream, long long nblocks, long long rows,
           long long M, int rate) {
  const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b < nblocks) zfp_block_io(encode, x_in, x_out, elem, stream, b, rows, M, rate);
}

}  // namespace

size_t zfp_stream_bytes(long long rows, long long M, int rate) {
  return (size_t)(((rows + 3) / 4) * (M / 4) * 2 * rate);
}

void zfp_encode_cpu(const void* x, int elem, uint8_t* stream, long long lead, long long rows, long long M, int rate) {
  const long long n = lead * ((rows + 3) / 4) * (M / 4);
  for (long long b = 0; b < n; ++b) zfp_block_io(true, x, nullptr, elem, stream, b, rows, M, rate);
}
void zfp_decode_cpu(const uint8_t* stream, void* x, int elem, long long lead, long long rows, long long M, int rate) {
  const long long n = lead * ((rows + 3) / 4) * (M / 4);
  for (long long b = 0; b < n; ++b)
    zfp_block_io(false, nullptr, x, elem, const_cast<uint8_t*>(stream), b, rows, M, rate);
}
void launch_zfp_encode(const void* x, int elem, uint8_t* stream, long long lead, long long rows, long long M, int rate,
                       cudaStream_t s) {
  const long long n = lead * ((rows + 3) / 4) * (M / 4);
  if (n <= 0) return;
  zfp_kernel<<<(unsigned)((n + 127) / 128), 128, 0, s>>>(true, x, nullptr, elem, stream, n, rows, M, rate);
}
void launch_zfp_decode(const uint8_t* stream, void* x, int elem, long long lead, long long rows, long long M, int rate,
                       cudaStream_t s) {
  const long long n = lead * ((rows + 3) / 4) * (M / 4);
  if (n <= 0) return;
  zfp_kernel<<<(unsigned)((n + 127) / 128), 128, 0, s>>>(false, nullptr, x, elem, const_cast<uint8_t*>(stream), n, rows, M,
                                                        rate);
}

// ------------------------------------------------------------------------------------------------
// LZ
// ------------------------------------------------------------------------------------------------
namespace {

__host__ __device__ inline long long lz_blocks(long long raw_bytes) { return (raw_bytes + kLzBlockBytes - 1) / kLzBlockBytes; }
__host__ __device__ inline long long lz_header_bytes(long long nb) { return ((4 + 4 * (nb + 1)) + 15) / 16 * 16; }

__host__ __device__ inline int lz_encode_one(const uint8_t* raw, long long raw_bytes, long long blk, int sym, uint8_t* slot) {
  const long long off = blk * kLzBlockBytes;
  const int bytes = (int)(raw_bytes - off < kLzBlockBytes ? raw_bytes - off : kLzBlockBytes);
  if (sym == 2) return lz_encode_block<uint16_t>(reinterpret_cast<const uint16_t*>(raw + off), bytes / 2, slot);
  return lz_encode_block<uint32_t>(reinterpret_cast<const uint32_t*>(raw + off), bytes / 4, slot);
}
__host__ __device__ inline void lz_decode_one(const uint8_t* packed, uint8_t* raw, long long raw_bytes, long long blk, int sym) {
  const long long off = blk * kLzBlockBytes;
  const int bytes = (int)(raw_bytes - off < kLzBlockBytes ? raw_bytes - off : kLzBlockBytes);
  if (sym == 2) lz_decode_block<uint16_t>(packed, reinterpret_cast<uint16_t*>(raw + off), bytes / 2);
  else lz_decode_block<uint32_t>(packed, reinterpret_cast<uint32_t*>(raw + off), bytes / 4);
}

// scratch layout: [slices][nb] slots of kLzSlotBytes, then int sizes [slices][nb]
__global__ void __launch_bounds__(64)
lz_encode_blocks_kernel(const uint8_t* raw, uint8_t* slots, int* blk_sizes, long long slices, long long raw_bytes, int sym) {
  const long long nb = lz_blocks(raw_bytes);
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= slices * nb) return;
  const long long s = i / nb, b = i - s * nb;
  blk_sizes[i] = lz_encode_one(raw + s * raw_bytes, raw_bytes, b, sym, slots + i * kLzSlotBytes);
}

// one CTA per slice: exclusive scan of the block sizes -> header of the slice payload
__global__ void __launch_bounds__(256)
lz_scan_kernel(const int* blk_sizes, uint8_t* payload, int* sizes, long long raw_bytes, long long payload_stride) {
  __shared__ unsigned carry;
  __shared__ unsigned warp_tot[8];
  const long long nb = lz_blocks(raw_bytes);
  const long long s = blockIdx.x;
  uint32_t* hdr = reinterpret_cast<uint32_t*>(payload + s * payload_stride);
  if (threadIdx.x == 0) { carry = 0; hdr[0] = (uint32_t)nb; }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (long long base = 0; base < nb; base += 256) {
    const long long i = base + threadIdx.x;
    unsigned v = i < nb ? (unsigned)blk_sizes[s * nb + i] : 0u;
    unsigned incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    unsigned before = carry;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    if (i < nb) hdr[1 + i] = before + incl - v;
    __syncthreads();
    if (threadIdx.x == 255) carry = before + incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    hdr[1 + nb] = carry;
    for (long long w = 2 + nb; w < lz_header_bytes(nb) / 4; ++w) hdr[w] = 0;   // header padding
    sizes[s] = (int)(lz_header_bytes(nb) + carry);
  }
}

__global__ void __launch_bounds__(128)
lz_compact_kernel(const uint8_t* slots, const int* blk_sizes, uint8_t* payload, long long raw_bytes, long long payload_stride) {
  // one warp per block: byte copy of the block's code into its packed position
  const long long nb = lz_blocks(raw_bytes);
  const long long i = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const long long s = blockIdx.y;
  if (i >= nb) return;
  const uint32_t* hdr = reinterpret_cast<const uint32_t*>(payload + s * payload_stride);
  uint8_t* dst = payload + s * payload_stride + lz_header_bytes(nb) + hdr[1 + i];
  const uint8_t* src = slots + (s * nb + i) * kLzSlotBytes;
  const int n = blk_sizes[s * nb + i];
  for (int k = threadIdx.x & 31; k < n; k += 32) dst[k] = src[k];
}

__global__ void __launch_bounds__(64)
lz_decode_blocks_kernel(const uint8_t* payload, uint8_t* raw, long long slices, long long raw_bytes, long long payload_stride,
                        int sym) {
  const long long nb = lz_blocks(raw_bytes);
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= slices * nb) return;
  const long long s = i / nb, b = i - s * nb;
  const uint8_t* base = payload + s * payload_stride;
  const uint32_t* hdr = reinterpret_cast<const uint32_t*>(base);
  lz_decode_one(base + lz_header_bytes(nb) + hdr[1 + b], raw + s * raw_bytes, raw_bytes, b, sym);
}

}  // namespace

size_t lz_payload_capacity(long long raw_bytes) {
  const long long nb = lz_blocks(raw_bytes);
  return (size_t)((lz_header_bytes(nb) + nb * kLzSlotBytes + 15) / 16 * 16);
}
size_t lz_scratch_bytes(long long slices, long long raw_bytes) {
  const long long nb = lz_blocks(raw_bytes);
  return (size_t)(slices * nb * (kLzSlotBytes + 4) + 16);
}

void lz_encode_cpu(const uint8_t* raw, uint8_t* payload, int* sizes, long long slices, long long raw_bytes,
                   long long payload_stride, int sym) {
  const long long nb = lz_blocks(raw_bytes);
  std::vector<uint8_t> slot(kLzSlotBytes);
  for (long long s = 0; s < slices; ++s) {
    uint8_t* base = payload + s * payload_stride;
    uint32_t* hdr = reinterpret_cast<uint32_t*>(base);
    hdr[0] = (uint32_t)nb;
    uint32_t off = 0;
    for (long long b = 0; b < nb; ++b) {
      const int n = lz_encode_one(raw + s * raw_bytes, raw_bytes, b, sym, slot.data());
      hdr[1 + b] = off;
      std::memcpy(base + lz_header_bytes(nb) + off, slot.data(), n);
      off += (uint32_t)n;
    }
    hdr[1 + nb] = off;
    for (long long w = 2 + nb; w < lz_header_bytes(nb) / 4; ++w) hdr[w] = 0;   // header padding
    sizes[s] = (int)(lz_header_bytes(nb) + off);
  }
}
void lz_decode_cpu(const uint8_t* payload, uint8_t* raw, long long slices, long long raw_bytes, long long payload_stride,
                   int sym) {
  const long long nb = lz_blocks(raw_bytes);
  for (long long s = 0; s < slices; ++s) {
    const uint8_t* base = payload + s * payload_stride;
    const uint32_t* hdr = reinterpret_cast<const uint32_t*>(base);
    for (long long b = 0; b < nb; ++b)
      lz_decode_one(base + lz_header_bytes(nb) + hdr[1 + b], raw + s * raw_bytes, raw_bytes, b, sym);
  }
}

void launch_lz_encode(const uint8_t* raw, uint8_t* payload, int* sizes, uint8_t* scratch, long long slices,
                      long long raw_bytes, long long payload_stride, int sym, cudaStream_t stream) {
  const long long nb = lz_blocks(raw_bytes);
  const long long total = slices * nb;
  if (total <= 0) return;
  uint8_t* slots = scratch;
  int* blk_sizes = reinterpret_cast<int*>(scratch + (total * kLzSlotBytes + 15) / 16 * 16);
  lz_encode_blocks_kernel<<<(unsigned)((total + 63) / 64), 64, 0, stream>>>(raw, slots, blk_sizes, slices, raw_bytes, sym);
  lz_scan_kernel<<<(unsigned)slices, 256, 0, stream>>>(blk_sizes, payload, sizes, raw_bytes, payload_stride);
  dim3 grid((unsigned)((nb + 3) / 4), (unsigned)slices);
  lz_compact_kernel<<<grid, 128, 0, stream>>>(slots, blk_sizes, payload, raw_bytes, payload_stride);
}
void launch_lz_decode(const uint8_t* payload, uint8_t* raw, long long slices, long long raw_bytes,
                      long long payload_stride, int sym, cudaStream_t stream) {
  const long long total = slices * lz_blocks(raw_bytes);
  if (total <= 0) return;
  lz_decode_blocks_kernel<<<(unsigned)((total + 63) / 64), 64, 0, stream>>>(payload, raw, slices, raw_bytes, payload_stride, sym);
}

}  // namespace planmoe
