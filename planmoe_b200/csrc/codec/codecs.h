// Launchers of the ZFP and LZ codecs (CUDA kernels and CPU loops over the same block coders).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace planmoe {

// elem: 0 = fp32, 1 = bf16, 2 = fp16.  x: [lead][rows][M]; stream: [lead][blocks * 2 * rate] bytes,
// blocks = ceil(rows / 4) * (M / 4).  rate in {4, 8, 16} bits per value.
size_t zfp_stream_bytes(long long rows, long long M, int rate);
void zfp_encode_cpu(const void* x, int elem, uint8_t* stream, long long lead, long long rows, long long M, int rate);
void zfp_decode_cpu(const uint8_t* stream, void* x, int elem, long long lead, long long rows, long long M, int rate);
void launch_zfp_encode(const void* x, int elem, uint8_t* stream, long long lead, long long rows, long long M, int rate,
                       cudaStream_t stream_);
void launch_zfp_decode(const uint8_t* stream, void* x, int elem, long long lead, long long rows, long long M, int rate,
                       cudaStream_t stream_);

// LZ: raw [slices][raw_bytes] (raw_bytes a multiple of sym); payload [slices][payload_stride];
// per slice: u32 n_blocks, u32 offsets[n_blocks + 1], then the packed blocks.  sizes[slice] = bytes used.
size_t lz_payload_capacity(long long raw_bytes);
size_t lz_scratch_bytes(long long slices, long long raw_bytes);
// Where a slice says how long it is: the u32 at byte *len_off holds the bytes of packed code that follow the
// *header_bytes of header, so a slice occupies header_bytes + that value.
void lz_slice_layout(long long raw_bytes, long long* len_off, long long* header_bytes);
void lz_encode_cpu(const uint8_t* raw, uint8_t* payload, int* sizes, long long slices, long long raw_bytes,
                   long long payload_stride, int sym);
void lz_decode_cpu(const uint8_t* payload, uint8_t* raw, long long slices, long long raw_bytes,
                   long long payload_stride, int sym);
void launch_lz_encode(const uint8_t* raw, uint8_t* payload, int* sizes, uint8_t* scratch, long long slices,
                      long long raw_bytes, long long payload_stride, int sym, cudaStream_t stream);
void launch_lz_decode(const uint8_t* payload, uint8_t* raw, long long slices, long long raw_bytes,
                      long long payload_stride, int sym, cudaStream_t stream);

}  // namespace planmoe
