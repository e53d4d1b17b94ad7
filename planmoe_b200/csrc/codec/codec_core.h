// Block-level ZFP (fixed-rate 2-D) and LZ coders, written once as host+device functions so that the
// CPU oracle and the CUDA kernels run literally the same arithmetic (bit-identical streams).
//
// ZFP block (4x4 floats -> 16*rate bits): common exponent, block-floating-point cast to int32,
// decorrelating lifting transform on rows then columns, sequency reordering, negabinary mapping,
// embedded bit-plane coding with group testing under a fixed bit budget, zero padding.  The
// reference delegates this to a privately patched libzfp (PlanMoE/custom/compressor/zfpc.cpp:31-51,
// 66-85) that is not part of its repository; the stream layout here is block-major with a fixed
// block size, so an even split of the stream is an even split of the tensor's leading dimension.
//
// LZ block (2 KiB of 16- or 32-bit symbols): greedy longest-match search in a sliding window of 32
// symbols, token stream of literals (raw symbol) and matches ({length, distance} bytes), one flag
// bit per token (LSB first).  Same coding scheme as the reference's GPULZ kernels
// (PlanMoE/custom/compressor/gpulz.cu:16-313) but symbols are compared by raw bits (so -0.0 and NaN
// payloads round-trip), 16-bit symbols are supported, and blocks are packed back to back.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define PM_HD __host__ __device__ __forceinline__
#else
#define PM_HD inline
#endif

namespace planmoe {
namespace codec {

// ------------------------------------------------------------------------------------------------
// bit stream over a small word array (LSB first)
// ------------------------------------------------------------------------------------------------
// Bits are collected in a 64-bit register and leave for the word array 32 at a time, so the array is touched
// once per word, not once per bit.
struct BitWriter {
  uint32_t* w;      // cleared by the caller
  int widx;         // next word to write
  uint64_t acc;     // pending bits, LSB first
  int nacc;         // number of pending bits (< 32 between calls)
  PM_HD void spill() {
    if (nacc >= 32) {
      w[widx++] = (uint32_t)acc;
      acc >>= 32;
      nacc -= 32;
    }
  }
  PM_HD void put(uint32_t bit) {
    acc |= (uint64_t)(bit & 1u) << nacc;
    ++nacc;
    spill();
  }
  // writes the low n bits of x (n <= 16), returns x >> n
  PM_HD uint32_t put_bits(uint32_t x, int n) {
    acc |= (uint64_t)(x & ((1u << n) - 1u)) << nacc;
    nacc += n;
    spill();
    return x >> n;
  }
  PM_HD void flush() {
    if (nacc > 0) w[widx] = (uint32_t)acc;
  }
};
struct BitReader {
  const uint32_t* w;
  int widx;         // next word to fetch
  int nwords;       // words available
  uint64_t acc;     // fetched bits not yet consumed, LSB first
  int nacc;
  PM_HD void fill(int need) {
    if (nacc < need) {
      const uint32_t next = widx < nwords ? w[widx] : 0u;
      ++widx;
      acc |= (uint64_t)next << nacc;
      nacc += 32;
    }
  }
  PM_HD uint32_t get() {
    fill(1);
    const uint32_t b = (uint32_t)acc & 1u;
    acc >>= 1;
    --nacc;
    return b;
  }
  PM_HD uint32_t get_bits(int n) {          // n <= 16
    if (n == 0) return 0u;
    fill(n);
    const uint32_t x = (uint32_t)acc & ((1u << n) - 1u);
    acc >>= n;
    nacc -= n;
    return x;
  }
};

// ------------------------------------------------------------------------------------------------
// ZFP 2-D block coder
// ------------------------------------------------------------------------------------------------
constexpr int kZfpMaxWords = 8;     // up to rate 16 (256 bits per block)

PM_HD void zfp_fwd_lift(int32_t* p, int s) {
  int32_t x = p[0], y = p[s], z = p[2 * s], w = p[3 * s];
  x += w; x >>= 1; w -= x;
  z += y; z >>= 1; y -= z;
  x += z; x >>= 1; z -= x;
  w += y; w >>= 1; y -= w;
  w += y >> 1; y -= w >> 1;
  p[0] = x; p[s] = y; p[2 * s] = z; p[3 * s] = w;
}
PM_HD void zfp_inv_lift(int32_t* p, int s) {
  int32_t x = p[0], y = p[s], z = p[2 * s], w = p[3 * s];
  y += w >> 1; w -= y >> 1;
  y += w; w <<= 1; w -= y;
  z += x; x <<= 1; x -= z;
  y += z; z <<= 1; z -= y;
  w += x; x <<= 1; x -= w;
  p[0] = x; p[s] = y; p[2 * s] = z; p[3 * s] = w;
}

PM_HD int zfp_perm(int i) {
  // coefficients ordered by total sequency
  switch (i) {
    case 0: return 0;  case 1: return 1;  case 2: return 4;  case 3: return 5;
    case 4: return 2;  case 5: return 8;  case 6: return 6;  case 7: return 9;
    case 8: return 3;  case 9: return 12; case 10: return 10; case 11: return 7;
    case 12: return 13; case 13: return 11; case 14: return 14; default: return 15;
  }
}

// exponent e with |x| < 2^e (frexp convention); x != 0
PM_HD int zfp_exponent(float x) {
  union { float f; uint32_t u; } v;
  v.f = x;
  int e = (int)((v.u >> 23) & 0xff);
  if (e == 0) {                      // subnormal: normalise
    uint32_t m = v.u & 0x7fffffu;
    if (m == 0) return -127;
    e = 1;
    while (!(m & 0x800000u)) { m <<= 1; --e; }
  }
  return e - 126;
}
PM_HD float zfp_ldexp(float x, int e) {
  // multiply by 2^e with two exact steps to stay inside the finite range
  union { float f; uint32_t u; } a, b;
  const int e1 = e / 2, e2 = e - e1;
  a.u = (uint32_t)(e1 + 127) << 23;
  b.u = (uint32_t)(e2 + 127) << 23;
  return x * a.f * b.f;
}

// Encode 16 floats (row-major 4x4) into `words` (cleared by the caller), maxbits = 16 * rate.
PM_HD void zfp_encode_block(const float* f, uint32_t* words, int maxbits) {
  BitWriter bw{words, 0, 0ull, 0};
  float amax = 0.f;
  for (int i = 0; i < 16; ++i) { const float a = f[i] < 0 ? -f[i] : f[i]; if (a > amax) amax = a; }
  if (!(amax > 0.f) || !(amax < 3.0e38f)) { return; }          // all-zero (or non-finite) block: bit 0 = 0
  const int emax = zfp_exponent(amax);
  const uint32_t ebiased = (uint32_t)(emax + 127);
  bw.put_bits(2u * ebiased + 1u, 9);
  int32_t q[16];
  for (int i = 0; i < 16; ++i) q[i] = (int32_t)zfp_ldexp(f[i], 30 - emax);
  for (int y = 0; y < 4; ++y) zfp_fwd_lift(q + 4 * y, 1);
  for (int x = 0; x < 4; ++x) zfp_fwd_lift(q + x, 4);
  uint32_t u[16];
  for (int i = 0; i < 16; ++i) u[i] = ((uint32_t)q[zfp_perm(i)] + 0xaaaaaaaau) ^ 0xaaaaaaaau;
  int bits = maxbits - 9;
  int n = 0;
  for (int k = 32; bits && k-- > 0;) {
    uint32_t x = 0;
    for (int i = 0; i < 16; ++i) x += ((u[i] >> k) & 1u) << i;
    const int m = n < bits ? n : bits;
    bits -= m;
    x = bw.put_bits(x, m);
    for (; n < 16 && bits && (bits--, bw.put(!!x), !!x); x >>= 1, n++)
      for (; n < 15 && bits && (bits--, bw.put(x & 1u), !(x & 1u)); x >>= 1, n++) {}
  }
  bw.flush();
}

PM_HD void zfp_decode_block(const uint32_t* words, float* f, int maxbits) {
  BitReader br{words, 0, maxbits / 32, 0ull, 0};
  if (!br.get()) {
    for (int i = 0; i < 16; ++i) f[i] = 0.f;
    return;
  }
  const int emax = (int)br.get_bits(8) - 127;
  uint32_t u[16];
  for (int i = 0; i < 16; ++i) u[i] = 0;
  int bits = maxbits - 9;
  int n = 0;
  for (int k = 32; bits && k-- > 0;) {
    const int m = n < bits ? n : bits;
    bits -= m;
    uint32_t x = br.get_bits(m);
    for (; n < 16 && bits && (bits--, br.get()); x += 1u << n++)
      for (; n < 15 && bits && (bits--, !br.get()); n++) {}
    for (int i = 0; x; ++i, x >>= 1) u[i] += (x & 1u) << k;
  }
  int32_t q[16];
  for (int i = 0; i < 16; ++i) q[zfp_perm(i)] = (int32_t)((u[i] ^ 0xaaaaaaaau) - 0xaaaaaaaau);
  for (int x = 0; x < 4; ++x) zfp_inv_lift(q + x, 4);
  for (int y = 0; y < 4; ++y) zfp_inv_lift(q + 4 * y, 1);
  for (int i = 0; i < 16; ++i) f[i] = zfp_ldexp((float)q[i], emax - 30);
}

// ------------------------------------------------------------------------------------------------
// LZ block coder
// ------------------------------------------------------------------------------------------------
constexpr int kLzBlockBytes = 2048;
constexpr int kLzWindow = 32;
constexpr int kLzMaxMatch = 32;
// worst case: 2-byte header + flag bytes for 1024 tokens + every symbol a literal
constexpr int kLzSlotBytes = 2 + 128 + kLzBlockBytes;

template <class Sym>
PM_HD int lz_encode_block(const Sym* in, int nsym, uint8_t* out) {
  // out: [u16 n_tokens][flag bytes ceil(n_tokens / 8)][data]; returns bytes written.
  // The flag area is placed after a first pass that only counts tokens, so the data can be
  // emitted in one more pass without scratch.
  const int min_match = sizeof(Sym) == 2 ? 2 : 1;
  // pass 1: count tokens
  int ntok = 0;
  for (int p = 0; p < nsym;) {
    int best = 0;
    const int w0 = p - kLzWindow < 0 ? 0 : p - kLzWindow;
    for (int c = w0; c < p; ++c) {
      int len = 0;
      while (len < kLzMaxMatch && p + len < nsym && in[c + len] == in[p + len]) ++len;
      if (len > best) best = len;
    }
    p += (best >= min_match && best > 0) ? best : 1;
    ++ntok;
  }
  const int flag_bytes = (ntok + 7) >> 3;
  out[0] = (uint8_t)(ntok & 0xff);
  out[1] = (uint8_t)(ntok >> 8);
  uint8_t* flags = out + 2;
  for (int i = 0; i < flag_bytes; ++i) flags[i] = 0;
  uint8_t* data = flags + flag_bytes;
  int dpos = 0, t = 0;
  for (int p = 0; p < nsym; ++t) {
    int best = 0, bestc = 0;
    const int w0 = p - kLzWindow < 0 ? 0 : p - kLzWindow;
    for (int c = w0; c < p; ++c) {
      int len = 0;
      while (len < kLzMaxMatch && p + len < nsym && in[c + len] == in[p + len]) ++len;
      if (len > best) { best = len; bestc = c; }
    }
    if (best >= min_match && best > 0) {
      flags[t >> 3] |= (uint8_t)(1u << (t & 7));
      data[dpos++] = (uint8_t)best;
      data[dpos++] = (uint8_t)(p - bestc);
      p += best;
    } else {
      const Sym s = in[p];
      for (unsigned b = 0; b < sizeof(Sym); ++b) data[dpos++] = (uint8_t)((uint32_t)s >> (8 * b));
      p += 1;
    }
  }
  return 2 + flag_bytes + dpos;
}

template <class Sym>
PM_HD void lz_decode_block(const uint8_t* in, Sym* out, int nsym) {
  const int ntok = (int)in[0] | ((int)in[1] << 8);
  const uint8_t* flags = in + 2;
  const uint8_t* data = flags + ((ntok + 7) >> 3);
  int dpos = 0, p = 0;
  for (int t = 0; t < ntok && p < nsym; ++t) {
    if ((flags[t >> 3] >> (t & 7)) & 1u) {
      const int len = data[dpos], dist = data[dpos + 1];
      dpos += 2;
      for (int i = 0; i < len && p < nsym; ++i, ++p) out[p] = out[p - dist];
    } else {
      uint32_t s = 0;
      for (unsigned b = 0; b < sizeof(Sym); ++b) s |= (uint32_t)data[dpos++] << (8 * b);
      out[p++] = (Sym)s;
    }
  }
}

}  // namespace codec
}  // namespace planmoe
