// ZFP fixed-rate 2-D and LZ codec kernels (sm_100a) plus their CPU twins.
//
// ZFP: one thread per 4x4 block; a thread reads four 4-element row segments (neighbouring threads
// read neighbouring segments, so rows are read coalesced) and writes its 2*rate-byte code word with
// 16-byte stores.  LZ: one warp per 2 KiB block for both directions, then a per-slice scan and a
// compaction copy pack the blocks back to back.  Both reuse the host/device block coders of
// codec_core.h, so the CUDA streams are bit-identical to the CPU oracle.
//
// Counterparts in the reference: libzfp calls of PlanMoE/custom/compressor/zfpc.cpp:31-51,66-85 and
// the GPULZ kernels + CUB scans of PlanMoE/custom/compressor/gpulz.cu:16-313,418-536.

#include "codec/codecs.h"
#include "codec/codec_core.h"
#include <cstddef>

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
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const long long row = yb * 4 + r;
#if defined(__CUDA_ARCH__)
      if (elem == 1 && row < rows) {              // bf16: the block's four values of this row in one 8-byte load
        const uint2 raw = *reinterpret_cast<const uint2*>(
            reinterpret_cast<const __nv_bfloat16*>(x_in) + (slice * rows + row) * M + xb * 4);
        f[r * 4 + 0] = __uint_as_float(raw.x << 16);
        f[r * 4 + 1] = __uint_as_float(raw.x & 0xffff0000u);
        f[r * 4 + 2] = __uint_as_float(raw.y << 16);
        f[r * 4 + 3] = __uint_as_float(raw.y & 0xffff0000u);
        continue;
      }
#endif
      for (int c = 0; c < 4; ++c)
        f[r * 4 + c] = row < rows ? load_elem(x_in, elem, (slice * rows + row) * M + xb * 4 + c) : 0.f;
    }
    for (int i = 0; i < words_n; ++i) words[i] = 0;
    zfp_encode_block(f, words, 16 * rate);
    for (int i = 0; i < words_n; ++i) dst[i] = words[i];
  } else {
    for (int i = 0; i < words_n; ++i) words[i] = dst[i];
    zfp_decode_block(words, f, 16 * rate);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const long long row = yb * 4 + r;
      if (row >= rows) break;
#if defined(__CUDA_ARCH__)
      if (elem == 1) {                            // bf16: one 8-byte store per row of the block
        const __nv_bfloat162 lo = __floats2bfloat162_rn(f[r * 4 + 0], f[r * 4 + 1]);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(f[r * 4 + 2], f[r * 4 + 3]);
        uint2 raw;
        raw.x = *reinterpret_cast<const uint32_t*>(&lo);
        raw.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(x_out) + (slice * rows + row) * M + xb * 4) = raw;
        continue;
      }
#endif
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
//
// Warp-parallel block coder.  One warp codes one 2 KiB block and produces exactly the bytes of the
// serial coder lz_encode_block (the CPU twin, which the tests compare against):
//   1. every lane finds, for its positions p = lane, lane + 32, ..., the longest match in the 32-symbol
//      window (first candidate of maximal length), as the serial coder would if a token started at p, from
//      per-position candidate bit masks;
//   2. the token starts are the positions reachable from 0 by next(p) = p + (match ? length : 1): each lane
//      owns a segment of 32 positions, computes where a walk from each of them leaves the segment, the exits
//      are chained from position 0 to give every segment its entry, and each lane walks its own segment;
//   3. token ordinals and data offsets come from a warp scan over the per-segment counts of that walk;
//   4. a second walk assembles flags and data in shared memory, which are then copied to the block's slot.
constexpr int kLzWarps = 4;                       // blocks coded per CTA
constexpr int kLzMaxSym = kLzBlockBytes / 2;      // symbols per block with 16-bit symbols

constexpr int kLzInfoWords = 32 * 33;             // position p lives at word (p % 32) * 33 + p / 32 (see lz_tp)

template <class Sym>
struct LzEncSmem {
  Sym in[kLzBlockBytes / sizeof(Sym)];
  // One word per position, written at the end of step 1: bits 0-10 next(p) = p + (match ? length : 1), bit 31
  // match; a match has its length in bits 11-16 and its distance in bits 17-22, a 16-bit literal its symbol in
  // bits 11-26.
  uint32_t info[kLzInfoWords];
  uint32_t flagw[kLzMaxSym / 32];                 // one bit per token: 1 = match
  // step 1: candidate masks eq[1024]; afterwards: exit positions (u16 [kLzInfoWords]) and the token payload
  uint32_t scratch[(kLzInfoWords * 2 + kLzBlockBytes + 3) / 4];
  __device__ uint32_t* eq() { return scratch; }
  __device__ uint16_t* exits() { return reinterpret_cast<uint16_t*>(scratch); }
  __device__ uint8_t* data() { return reinterpret_cast<uint8_t*>(scratch) + kLzInfoWords * 2; }
};
static_assert(kLzWindow == 32 && kLzMaxMatch <= 32 && kLzMaxSym <= 1024, "lz encoder: masks, info fields and segments");
static_assert(sizeof(LzEncSmem<uint16_t>::scratch) >= kLzMaxSym * 4, "eq() needs one word per position");

// Positions are handed to lanes in two ways: strided (p = k * 32 + lane, steps 1) and in segments of 32 consecutive
// positions per lane (steps 2-4).  This index keeps both conflict-free or nearly so: strided writes hit 32 banks,
// and lanes walking their segments in lock-step (same offset) do too.
__device__ __forceinline__ int lz_tp(int p) { return (p & 31) * 33 + (p >> 5); }

template <class Sym>
__device__ __forceinline__ void lz_encode_block_warp(const Sym* __restrict__ g_in, int nsym, uint8_t* __restrict__ out,
                                                     int* __restrict__ out_size, LzEncSmem<Sym>& sm, int lane) {
  constexpr int min_match = sizeof(Sym) == 2 ? 2 : 1;
  for (int i = lane; i < nsym; i += 32) sm.in[i] = g_in[i];
  for (int i = lane; i < kLzMaxSym / 32; i += 32) sm.flagw[i] = 0u;
  __syncwarp();

  // 1. longest match per position.  eq[q] has bit d-1 set when in[q - d] == in[q] (d = 1 .. 32): a candidate at
  // distance d matches L symbols from p exactly when eq[p] & eq[p + 1] & ... & eq[p + L - 1] keeps bit d-1, so the
  // longest match is found by and-ing masks until nothing survives, and the first candidate of maximal length
  // (the serial coder's choice) is the largest surviving distance.
  uint32_t* eq = sm.eq();
  for (int p = lane; p < nsym; p += 32) {
    const Sym v = sm.in[p];
    uint32_t m = 0u;
    const int dmax = p < kLzWindow ? p : kLzWindow;
#pragma unroll 8
    for (int d = 1; d <= dmax; ++d) m |= (sm.in[p - d] == v ? 1u : 0u) << (d - 1);
    eq[p] = m;
  }
  __syncwarp();
  uint32_t info_r[kLzMaxSym / 32];                  // eq shares its memory with later steps: results wait in registers
#pragma unroll
  for (int k = 0; k < kLzMaxSym / 32; ++k) {
    const int p = k * 32 + lane;
    uint32_t w = 0u;
    if (p < nsym) {
      const int lim = nsym - p < kLzMaxMatch ? nsym - p : kLzMaxMatch;
      uint32_t m = eq[p];
      int best = 0;
      if (m != 0u) {
        best = 1;
        while (best < lim) {
          const uint32_t m2 = m & eq[p + best];
          if (m2 == 0u) break;
          m = m2;
          ++best;
        }
      }
      if (best >= min_match && best > 0) {
        w = 0x80000000u | (uint32_t)(p + best) | ((uint32_t)best << 11) | ((uint32_t)(32 - __clz(m)) << 17);
      } else {
        w = (uint32_t)(p + 1);
        if (sizeof(Sym) == 2) w |= (uint32_t)sm.in[p] << 11;
      }
    }
    info_r[k] = w;
  }
  __syncwarp();                                   // every lane is done reading eq
#pragma unroll
  for (int k = 0; k < kLzMaxSym / 32; ++k) {
    const int p = k * 32 + lane;
    if (p < nsym) sm.info[lz_tp(p)] = info_r[k];
  }
  __syncwarp();

  // 2. token starts = positions reachable from 0 by next().  Lane l owns the segment [32 l, 32 l + 32).  (a) Going
  // backwards through its segment every lane finds, for each position, where a walk from there leaves the
  // segment; (b) following these exits from position 0, segment by segment, gives every segment its entry
  // point (a jump is at most 32 long, so a walk enters each segment it does not end in); (c) each lane then
  // walks its segment from its entry.
  const int p0 = lane * 32, p1 = p0 + 32 < nsym ? p0 + 32 : nsym;
  uint16_t* exits = sm.exits();
  for (int o = p1 - p0 - 1; o >= 0; --o) {
    const int nx = (int)(sm.info[o * 33 + lane] & 0x7ffu);
    exits[o * 33 + lane] = (uint16_t)(nx >= p1 ? nx : exits[(nx & 31) * 33 + lane]);
  }
  __syncwarp();
  int entry = -1;
  {
    int e = 0;
    for (int l = 0; l < 32 && e < nsym; ++l) {
      const int end = (l + 1) * 32 < nsym ? (l + 1) * 32 : nsym;
      if (e < end) {
        if (l == lane) entry = e;
        e = exits[(e & 31) * 33 + l];
      }
    }
  }

  // 3. ordinals and data offsets from a first walk
  int ntok_l = 0, bytes_l = 0;
  for (int p = entry; p >= 0 && p < p1;) {
    const uint32_t w = sm.info[(p & 31) * 33 + lane];
    ++ntok_l;
    bytes_l += (w >> 31) ? 2 : (int)sizeof(Sym);
    p = (int)(w & 0x7ffu);
  }
  int tok_incl = ntok_l, byt_incl = bytes_l;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, tok_incl, o);
    const int b = __shfl_up_sync(0xffffffffu, byt_incl, o);
    if (lane >= o) { tok_incl += t; byt_incl += b; }
  }
  const int ntok = __shfl_sync(0xffffffffu, tok_incl, 31);
  const int dbytes = __shfl_sync(0xffffffffu, byt_incl, 31);
  int t = tok_incl - ntok_l, dpos = byt_incl - bytes_l;

  // 4. flags + data from a second walk
  uint8_t* data = sm.data();
  for (int p = entry; p >= 0 && p < p1; ++t) {
    const uint32_t w = sm.info[(p & 31) * 33 + lane];
    if (w >> 31) {
      atomicOr(&sm.flagw[t >> 5], 1u << (t & 31));
      data[dpos++] = (uint8_t)((w >> 11) & 63u);
      data[dpos++] = (uint8_t)((w >> 17) & 63u);
    } else {
      const uint32_t v = sizeof(Sym) == 2 ? ((w >> 11) & 0xffffu) : (uint32_t)sm.in[p];
#pragma unroll
      for (unsigned b = 0; b < sizeof(Sym); ++b) data[dpos++] = (uint8_t)(v >> (8 * b));
    }
    p = (int)(w & 0x7ffu);
  }
  __syncwarp();
  const int flag_bytes = (ntok + 7) >> 3;
  if (lane == 0) {
    out[0] = (uint8_t)(ntok & 0xff);
    out[1] = (uint8_t)(ntok >> 8);
    *out_size = 2 + flag_bytes + dbytes;
  }
  const uint8_t* fb = reinterpret_cast<const uint8_t*>(sm.flagw);
  for (int i = lane; i < flag_bytes; i += 32) out[2 + i] = fb[i];
  uint8_t* od = out + 2 + flag_bytes;
  for (int i = lane; i < dbytes; i += 32) od[i] = data[i];
  __syncwarp();
}

template <class Sym>
__global__ void __launch_bounds__(kLzWarps * 32)
lz_encode_blocks_kernel(const uint8_t* raw, uint8_t* slots, int* blk_sizes, long long slices, long long raw_bytes) {
  extern __shared__ __align__(16) uint8_t lz_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  LzEncSmem<Sym>& sm = reinterpret_cast<LzEncSmem<Sym>*>(lz_smem)[warp];
  const long long nb = lz_blocks(raw_bytes);
  const long long i = (long long)blockIdx.x * kLzWarps + warp;
  if (i >= slices * nb) return;
  const long long s = i / nb, b = i - s * nb;
  const long long off = b * kLzBlockBytes;
  const int bytes = (int)(raw_bytes - off < kLzBlockBytes ? raw_bytes - off : kLzBlockBytes);
  lz_encode_block_warp<Sym>(reinterpret_cast<const Sym*>(raw + s * raw_bytes + off), bytes / (int)sizeof(Sym),
                            slots + i * kLzSlotBytes, blk_sizes + i, sm, lane);
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

// Warp-parallel block decoder (same output as lz_decode_block).  Tokens are expanded to a source map
// (a literal is its own source; symbol i of a match sources position p - distance) from a warp scan of
// token lengths; sources are resolved to literals with ten rounds of pointer doubling, because a match
// may copy symbols that an earlier (or the same, overlapping) match produced.
template <class Sym>
struct LzDecSmem {
  uint8_t code[kLzSlotBytes + 2];                 // the block's code bytes
  Sym val[kLzBlockBytes / sizeof(Sym)];           // literal value at p (defined where src[p] == p)
  uint16_t src[2][kLzMaxSym];
};

template <class Sym>
__device__ __forceinline__ void lz_decode_block_warp(const uint8_t* __restrict__ g_code, int code_bytes,
                                                     Sym* __restrict__ g_out, int nsym, LzDecSmem<Sym>& sm, int lane) {
  for (int i = lane; i < code_bytes; i += 32) sm.code[i] = g_code[i];
  for (int q = lane; q < nsym; q += 32) { sm.src[0][q] = (uint16_t)q; sm.val[q] = (Sym)0; }   // defined even for a short code
  __syncwarp();
  const int ntok = (int)sm.code[0] | ((int)sm.code[1] << 8);
  const uint8_t* flags = sm.code + 2;
  const uint8_t* data = flags + ((ntok + 7) >> 3);

  // lane owns tokens [t0, t1): first their data bytes, then (needs the lengths) their output symbols
  const int seg = (ntok + 31) / 32;
  const int t0 = lane * seg < ntok ? lane * seg : ntok, t1 = t0 + seg < ntok ? t0 + seg : ntok;
  int byt_l = 0;
  for (int t = t0; t < t1; ++t) byt_l += ((flags[t >> 3] >> (t & 7)) & 1u) ? 2 : (int)sizeof(Sym);
  int byt_incl = byt_l;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int b = __shfl_up_sync(0xffffffffu, byt_incl, o);
    if (lane >= o) byt_incl += b;
  }
  int dpos = byt_incl - byt_l;
  int sym_l = 0;
  {
    int d = dpos;
    for (int t = t0; t < t1; ++t) {
      if ((flags[t >> 3] >> (t & 7)) & 1u) { sym_l += data[d]; d += 2; }
      else { sym_l += 1; d += (int)sizeof(Sym); }
    }
  }
  int sym_incl = sym_l;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int b = __shfl_up_sync(0xffffffffu, sym_incl, o);
    if (lane >= o) sym_incl += b;
  }
  int p = sym_incl - sym_l;
  for (int t = t0; t < t1; ++t) {
    if ((flags[t >> 3] >> (t & 7)) & 1u) {
      const int len = data[dpos], dist = data[dpos + 1];
      dpos += 2;
      for (int i = 0; i < len && p < nsym; ++i, ++p) sm.src[0][p] = (uint16_t)(p - dist > 0 ? p - dist : 0);
    } else {
      uint32_t v = 0;
#pragma unroll
      for (unsigned b = 0; b < sizeof(Sym); ++b) v |= (uint32_t)data[dpos++] << (8 * b);
      if (p < nsym) { sm.val[p] = (Sym)v; sm.src[0][p] = (uint16_t)p; }
      ++p;
    }
  }
  __syncwarp();
  int cur = 0;
  for (int hop = 1; hop < nsym; hop <<= 1) {
    for (int q = lane; q < nsym; q += 32) sm.src[cur ^ 1][q] = sm.src[cur][sm.src[cur][q]];
    __syncwarp();
    cur ^= 1;
  }
  for (int q = lane; q < nsym; q += 32) g_out[q] = sm.val[sm.src[cur][q]];
  __syncwarp();
}

template <class Sym>
__global__ void __launch_bounds__(kLzWarps * 32)
lz_decode_blocks_kernel(const uint8_t* payload, uint8_t* raw, long long slices, long long raw_bytes, long long payload_stride) {
  extern __shared__ __align__(16) uint8_t lz_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  LzDecSmem<Sym>& sm = reinterpret_cast<LzDecSmem<Sym>*>(lz_smem)[warp];
  const long long nb = lz_blocks(raw_bytes);
  const long long i = (long long)blockIdx.x * kLzWarps + warp;
  if (i >= slices * nb) return;
  const long long s = i / nb, b = i - s * nb;
  const uint8_t* base = payload + s * payload_stride;
  const uint32_t* hdr = reinterpret_cast<const uint32_t*>(base);
  const long long off = b * kLzBlockBytes;
  const int bytes = (int)(raw_bytes - off < kLzBlockBytes ? raw_bytes - off : kLzBlockBytes);
  const int code_bytes = (int)(hdr[2 + b] - hdr[1 + b]);
  if (code_bytes < 2 || code_bytes > kLzSlotBytes) return;       // corrupt header: leave the block untouched
  lz_decode_block_warp<Sym>(base + lz_header_bytes(nb) + hdr[1 + b], code_bytes,
                            reinterpret_cast<Sym*>(raw + s * raw_bytes + off), bytes / (int)sizeof(Sym), sm, lane);
}

}  // namespace

size_t lz_payload_capacity(long long raw_bytes) {
  const long long nb = lz_blocks(raw_bytes);
  return (size_t)((lz_header_bytes(nb) + nb * kLzSlotBytes + 15) / 16 * 16);
}
void lz_slice_layout(long long raw_bytes, long long* len_off, long long* header_bytes) {
  const long long nb = lz_blocks(raw_bytes);
  *len_off = 4 * (1 + nb);
  *header_bytes = lz_header_bytes(nb);
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
  const unsigned ctas = (unsigned)((total + kLzWarps - 1) / kLzWarps);
  if (sym == 2) {
    constexpr int smem = kLzWarps * (int)sizeof(LzEncSmem<uint16_t>);
    static bool once = false;
    if (!once) { cudaFuncSetAttribute(lz_encode_blocks_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); once = true; }
    lz_encode_blocks_kernel<uint16_t><<<ctas, kLzWarps * 32, smem, stream>>>(raw, slots, blk_sizes, slices, raw_bytes);
  } else {
    constexpr int smem = kLzWarps * (int)sizeof(LzEncSmem<uint32_t>);
    static bool once = false;
    if (!once) { cudaFuncSetAttribute(lz_encode_blocks_kernel<uint32_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); once = true; }
    lz_encode_blocks_kernel<uint32_t><<<ctas, kLzWarps * 32, smem, stream>>>(raw, slots, blk_sizes, slices, raw_bytes);
  }
  lz_scan_kernel<<<(unsigned)slices, 256, 0, stream>>>(blk_sizes, payload, sizes, raw_bytes, payload_stride);
  dim3 grid((unsigned)((nb + 3) / 4), (unsigned)slices);
  lz_compact_kernel<<<grid, 128, 0, stream>>>(slots, blk_sizes, payload, raw_bytes, payload_stride);
}
void launch_lz_decode(const uint8_t* payload, uint8_t* raw, long long slices, long long raw_bytes,
                      long long payload_stride, int sym, cudaStream_t stream) {
  const long long total = slices * lz_blocks(raw_bytes);
  if (total <= 0) return;
  const unsigned ctas = (unsigned)((total + kLzWarps - 1) / kLzWarps);
  if (sym == 2) {
    constexpr int smem = kLzWarps * (int)sizeof(LzDecSmem<uint16_t>);
    static bool once = false;
    if (!once) { cudaFuncSetAttribute(lz_decode_blocks_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); once = true; }
    lz_decode_blocks_kernel<uint16_t><<<ctas, kLzWarps * 32, smem, stream>>>(payload, raw, slices, raw_bytes, payload_stride);
  } else {
    constexpr int smem = kLzWarps * (int)sizeof(LzDecSmem<uint32_t>);
    static bool once = false;
    if (!once) { cudaFuncSetAttribute(lz_decode_blocks_kernel<uint32_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); once = true; }
    lz_decode_blocks_kernel<uint32_t><<<ctas, kLzWarps * 32, smem, stream>>>(payload, raw, slices, raw_bytes, payload_stride);
  }
}

}  // namespace planmoe
