// Token <-> expert-slot movement kernels (sm_100a), local or pushed straight into peer GPUs.
//
//   scatter_rows   slot-major gather of token rows (optionally gate-weighted, optionally int8
//                  row-quantised) written to the slot's home: a local [E*C, M] buffer, or the
//                  receive buffer of the rank that owns the expert, followed by a release-add on
//                  that rank's (chunk, source) flag.  One launch serves the forward dispatch and
//                  the backward of the combine.
//   gather_rows    token-major gate-weighted sum over the k picks, optionally after a bounded
//                  acquire-wait on the (chunk, source) flags of the buffer being read.  Serves the
//                  forward combine-decode and the backward of the dispatch.
//   gate_grad      dgate[k][t] = <disp[slot_k(t)], dy[t]>.
//   build_slot_map inverse of (idx, loc): slot -> token*K+k, or -1.
//
// Slot ownership is unique, so the scatter is a plain store: no atomics, bit-reproducible,
// and empty slots are written as zeros by the same pass (no separate memset of the buffer).
// These replace the reference's JIT kernels (PlanMoE/jit_kernels/sparse.py:21-134), its
// contiguous/permute copies (impls/communicate.py:604-623) and, in push mode, the ncclSend /
// ncclRecv pairs of custom/comm/naive.cpp:17-26.

#include "planmoe.h"
#include "kernels/common.cuh"

namespace planmoe {

constexpr int kRowThreads = 256;
constexpr int kRowWarps = kRowThreads / 32;

__global__ void fill_slot_map_kernel(const int* __restrict__ idx, const int* __restrict__ loc,
                                     int* __restrict__ slot_map, int K, int S, int E, int C) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= K * S) return;
  const int k = i / S, t = i - k * S;
  const int e = idx[i], l = loc[i];
  if (e >= 0 && e < E && l >= 0 && l < C) slot_map[(size_t)e * C + l] = t * K + k;
}

void launch_build_slot_map(const int* idx, const int* loc, int* slot_map, int K, int S, int E,
                           int C, cudaStream_t stream) {
  cudaMemsetAsync(slot_map, 0xFF, sizeof(int) * (size_t)E * C, stream);
  const int n = K * S;
  if (n > 0) fill_slot_map_kernel<<<(n + 255) / 256, 256, 0, stream>>>(idx, loc, slot_map, K, S, E, C);
}

// Destination row of global slot (e, c) in push mode.  The receive buffer of a rank is laid out
// [chunk][E_local][W_src][C/chunks][M] so that each chunk is a dense batched-GEMM operand.
struct PushGeom {
  const unsigned long long* heap_bases;  // [W] peer-mapped base of the symmetric heap, or null
  unsigned long long data_off;           // byte offset of the destination buffer in the heap
  unsigned long long flag_off;           // byte offset of the u64 flag array [chunks][W]
  unsigned long long scale_off;          // byte offset of the fp32 (scale,bias) rows (int8 mode)
  int W, my_rank, E_local, C, chunks;
  int chunk_begin, chunk_count;          // chunks served by this launch
};

template <class T, bool QUANT>
__global__ void __launch_bounds__(kRowThreads, 6)
scatter_rows_kernel(const T* __restrict__ x, const int* __restrict__ slot_map,
                    const float* __restrict__ gates, T* __restrict__ local_out, int K, int S,
                    int M, PushGeom g) {
  // 1-D persistent grid.  Chunks are served in order (chunk 0 leaves first for every destination),
  // destinations start at my right-hand neighbour so that ranks do not all hit the same peer at once.
  // After a chunk has been stored for all destinations the CTA fences once and adds one arrival to the
  // chunk's flag on every destination: a flag is complete when all gridDim.x CTAs have arrived.
  // The register bound keeps one such CTA co-resident with a GEMM CTA on the same SM.
  const int Cc = g.C / g.chunks;
  const int rows = g.E_local * Cc;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int V = Vec16<T>::N;
  const int nvec = M / V;

  for (int j = g.chunk_begin; j < g.chunk_begin + g.chunk_count; ++j) {
  for (int rr = 0; rr < g.W; ++rr) {
  const int r = g.heap_bases != nullptr ? (g.my_rank + 1 + rr) % g.W : rr;
  unsigned char* dst_base;
  if (g.heap_bases != nullptr) {
    dst_base = reinterpret_cast<unsigned char*>(g.heap_bases[r]) + g.data_off;
  } else {
    dst_base = reinterpret_cast<unsigned char*>(local_out);
  }

  for (int row = blockIdx.x * kRowWarps + warp; row < rows; row += gridDim.x * kRowWarps) {
    const int el = row / Cc, cc = row - el * Cc;
    const int e = r * g.E_local + el, c = j * Cc + cc;
    const int owner = slot_map[(size_t)e * g.C + c];
    // destination row index inside the receiving buffer
    size_t drow;
    if (g.heap_bases != nullptr) {
      drow = (((size_t)j * g.E_local + el) * g.W + g.my_rank) * Cc + cc;
    } else {
      drow = (size_t)e * g.C + c;
    }
    if constexpr (!QUANT) {
      T* dst = reinterpret_cast<T*>(dst_base) + drow * M;
      if (owner < 0) {
        Pack<T> z;
#pragma unroll
        for (int i = 0; i < V; ++i) z.v[i] = from_f32<T>(0.f);
        for (int v = lane; v < nvec; v += 32) st16(dst + v * V, z);
      } else {
        const int t = owner / K, k = owner - t * K;
        const T* src = x + (size_t)t * M;
        if (gates == nullptr) {
          for (int v = lane; v < nvec; v += 32) st16(dst + v * V, ld16(src + v * V));
        } else {
          const float gw = gates[(size_t)k * S + t];
          for (int v = lane; v < nvec; v += 32) {
            Pack<T> p = ld16(src + v * V);
#pragma unroll
            for (int i = 0; i < V; ++i) p.v[i] = from_f32<T>(gw * to_f32(p.v[i]));
            st16(dst + v * V, p);
          }
        }
      }
    } else {
      // int8 row-affine quantisation fused into the send: q = round((x - lo) * 255 / (hi - lo))
      unsigned char* dst = dst_base + drow * M;
      float* sb = reinterpret_cast<float*>(
          (g.heap_bases != nullptr ? reinterpret_cast<unsigned char*>(g.heap_bases[r]) + g.scale_off
                                   : reinterpret_cast<unsigned char*>(local_out) + g.scale_off)) + drow * 2;
      if (owner < 0) {
        for (int v = lane; v < M / 16; v += 32) reinterpret_cast<uint4*>(dst)[v] = make_uint4(0, 0, 0, 0);
        if (lane == 0) { sb[0] = 0.f; sb[1] = 0.f; }
      } else {
        const int t = owner / K, k = owner - t * K;
        const T* src = x + (size_t)t * M;
        const float gw = gates ? gates[(size_t)k * S + t] : 1.f;
        float lo = INFINITY, hi = -INFINITY;
        for (int v = lane; v < nvec; v += 32) {
          Pack<T> p = ld16(src + v * V);
#pragma unroll
          for (int i = 0; i < V; ++i) { float f = gw * to_f32(p.v[i]); lo = fminf(lo, f); hi = fmaxf(hi, f); }
        }
        lo = warp_min(lo); hi = warp_max(hi);
        const float range = hi - lo;
        const float inv = range > 0.f ? 255.f / range : 0.f;
        // 16 output bytes per lane-iteration = 16 elements = (16 / V) input vectors
        for (int v = lane; v < M / 16; v += 32) {
          alignas(16) unsigned char q[16];
#pragma unroll
          for (int h = 0; h < 16 / V; ++h) {
            Pack<T> p = ld16(src + (size_t)v * 16 + h * V);
#pragma unroll
            for (int i = 0; i < V; ++i) {
              float f = (gw * to_f32(p.v[i]) - lo) * inv;
              q[h * V + i] = (unsigned char)fminf(fmaxf(rintf(f), 0.f), 255.f);
            }
          }
          reinterpret_cast<uint4*>(dst)[v] = *reinterpret_cast<uint4*>(q);
        }
        if (lane == 0) { sb[0] = range; sb[1] = lo; }
      }
    }
  }

  }  // destinations

  if (g.heap_bases != nullptr && g.flag_off != ~0ull) {
    __syncthreads();
    if (threadIdx.x == 0) __threadfence_system();
    __syncthreads();
    if (threadIdx.x < g.W) {
      unsigned long long* flags = reinterpret_cast<unsigned long long*>(
          reinterpret_cast<unsigned char*>(g.heap_bases[threadIdx.x]) + g.flag_off);
      red_release_sys_add(flags + (size_t)j * g.W + g.my_rank, 1ull);
    }
  }
  }  // chunks
}

template <class T>
void launch_scatter_rows(const T* x, const int* slot_map, const float* gates, T* local_out, int K,
                         int S, int M, int E, int C, const PushArgs* push, bool quant,
                         cudaStream_t stream) {
  PushGeom g{};
  int ctas;
  if (push == nullptr) {
    g.heap_bases = nullptr; g.data_off = 0; g.flag_off = ~0ull; g.scale_off = 0;
    g.W = 1; g.my_rank = 0; g.E_local = E; g.C = C; g.chunks = 1; g.chunk_begin = 0; g.chunk_count = 1;
    ctas = (E * C + kRowWarps - 1) / kRowWarps;
    if (ctas > 148 * 6) ctas = 148 * 6;
  } else {
    g.heap_bases = push->heap_bases; g.data_off = push->data_off; g.flag_off = push->flag_off;
    g.scale_off = push->scale_off;
    g.W = push->W; g.my_rank = push->my_rank; g.E_local = E / push->W; g.C = C; g.chunks = push->chunks;
    g.chunk_begin = push->chunk_begin; g.chunk_count = push->chunk_count > 0 ? push->chunk_count : push->chunks;
    ctas = push->ctas_per_msg;       // total CTAs of the persistent grid (= arrivals per flag)
  }
  if (ctas < 1) ctas = 1;
  if (quant)
    scatter_rows_kernel<T, true><<<ctas, kRowThreads, 0, stream>>>(x, slot_map, gates, local_out, K, S, M, g);
  else
    scatter_rows_kernel<T, false><<<ctas, kRowThreads, 0, stream>>>(x, slot_map, gates, local_out, K, S, M, g);
}

// ------------------------------------------------------------------------------------------

struct WaitGeom {
  const unsigned long long* flags;  // local u64 flags [n_flags], or null (no wait)
  int n_flags;
  unsigned long long want;
  const unsigned long long* want_ptr;   // overrides `want` when set
  unsigned long long budget_ns;
  int* status;
};

// MAXK bounds the number of picks per token held in registers: 2 covers top-1 / top-2 gates and keeps
// the kernel at 32 registers, so that eight CTAs (all 64 warps) fit on an SM and the whole token range
// is resident in one wave; 8 is the general case.
template <class T, int DEQUANT, int MAXK>
__global__ void __launch_bounds__(kRowThreads, MAXK <= 2 ? 8 : 4)
gather_rows_kernel(const void* __restrict__ disp_, const float* __restrict__ scale_bias,
                   const int* __restrict__ idx, const int* __restrict__ loc,
                   const float* __restrict__ gates, T* __restrict__ out, int K, int S, int M,
                   int C, WaitGeom w, long long group_rows) {
  __shared__ int ok_s;
  if (w.flags != nullptr) {
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    const unsigned long long want = w.want_ptr != nullptr ? *w.want_ptr : w.want;
    for (int f = threadIdx.x; f < w.n_flags; f += blockDim.x) {
      if (!wait_flag_ge(w.flags + f, want, w.budget_ns, w.status, f)) ok_s = 0;
    }
    __syncthreads();
    if (!ok_s) return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int V = Vec16<T>::N;
  const int nvec = M / V;
  for (int t = blockIdx.x * kRowWarps + warp; t < S; t += gridDim.x * kRowWarps) {
    long long slot[MAXK];
    float gw[MAXK];
#pragma unroll
    for (int k = 0; k < MAXK; ++k) {
      slot[k] = -1; gw[k] = 0.f;
      if (k < K) {
        const int e = idx[(size_t)k * S + t], l = loc[(size_t)k * S + t];
        if (e >= 0 && l >= 0 && l < C) {
          slot[k] = (long long)e * C + l;
          gw[k] = gates ? gates[(size_t)k * S + t] : 1.f;
        }
      }
    }
    T* dst = out + (size_t)t * M;
    if constexpr (DEQUANT == 2) {
      // uint8 rows, one (scale, low) pair per 128 columns and row, pairs laid out [M / 128][group_rows]
      const unsigned char* disp = reinterpret_cast<const unsigned char*>(disp_);
      const float2* sc = reinterpret_cast<const float2*>(scale_bias);
      for (int v = lane; v < M / 16; v += 32) {
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
#pragma unroll
        for (int k = 0; k < MAXK; ++k) {
          if (k < K && slot[k] >= 0) {
            const float2 sl = sc[(size_t)(v >> 3) * group_rows + slot[k]];
            const float a = sl.x * gw[k], b = sl.y * gw[k];
            uint4 raw = *reinterpret_cast<const uint4*>(disp + slot[k] * M + (size_t)v * 16);
            const unsigned char* q = reinterpret_cast<const unsigned char*>(&raw);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] += fmaf(a, (float)q[i], b);
          }
        }
#pragma unroll
        for (int h = 0; h < 16 / V; ++h) {
          Pack<T> o;
#pragma unroll
          for (int i = 0; i < V; ++i) o.v[i] = from_f32<T>(acc[h * V + i]);
          st16(dst + (size_t)v * 16 + h * V, o);
        }
      }
    } else if constexpr (DEQUANT == 0) {
      const T* disp = reinterpret_cast<const T*>(disp_);
      for (int v = lane; v < nvec; v += 32) {
        float acc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = 0.f;
#pragma unroll
        for (int k = 0; k < MAXK; ++k) {
          if (k < K && slot[k] >= 0) {
            Pack<T> p = ld16(disp + slot[k] * M + v * V);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] += gw[k] * to_f32(p.v[i]);
          }
        }
        Pack<T> o;
#pragma unroll
        for (int i = 0; i < V; ++i) o.v[i] = from_f32<T>(acc[i]);
        st16(dst + v * V, o);
      }
    } else {
      const unsigned char* disp = reinterpret_cast<const unsigned char*>(disp_);
      float sc[MAXK], bi[MAXK];
#pragma unroll
      for (int k = 0; k < MAXK; ++k) {
        sc[k] = bi[k] = 0.f;
        if (k < K && slot[k] >= 0) {
          sc[k] = scale_bias[slot[k] * 2] * (1.f / 255.f) * gw[k];
          bi[k] = scale_bias[slot[k] * 2 + 1] * gw[k];
        }
      }
      for (int v = lane; v < M / 16; v += 32) {
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
#pragma unroll
        for (int k = 0; k < MAXK; ++k) {
          if (k < K && slot[k] >= 0) {
            uint4 raw = *reinterpret_cast<const uint4*>(disp + slot[k] * M + (size_t)v * 16);
            const unsigned char* q = reinterpret_cast<const unsigned char*>(&raw);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] += sc[k] * (float)q[i] + bi[k];
          }
        }
#pragma unroll
        for (int h = 0; h < 16 / V; ++h) {
          Pack<T> o;
#pragma unroll
          for (int i = 0; i < V; ++i) o.v[i] = from_f32<T>(acc[h * V + i]);
          st16(dst + (size_t)v * 16 + h * V, o);
        }
      }
    }
  }
}

template <class T>
void launch_gather_rows(const void* disp, const float* scale_bias, const int* idx, const int* loc,
                        const float* gates, T* out, int K, int S, int M, int C,
                        const WaitArgs* wait, cudaStream_t stream, long long group_rows) {
  WaitGeom w{};
  if (wait != nullptr) {
    w.flags = wait->flags; w.n_flags = wait->n_flags; w.want = wait->want; w.want_ptr = wait->want_ptr;
    w.budget_ns = wait->budget_ns; w.status = wait->status;
  }
  int ctas = (S + kRowWarps - 1) / kRowWarps;
  if (ctas > 148 * 8) ctas = 148 * 8;
  if (ctas < 1) ctas = 1;
  if (scale_bias != nullptr && group_rows > 0)
    gather_rows_kernel<T, 2, 8><<<ctas, kRowThreads, 0, stream>>>(disp, scale_bias, idx, loc, gates, out, K, S, M, C, w, group_rows);
  else if (scale_bias != nullptr)
    gather_rows_kernel<T, 1, 8><<<ctas, kRowThreads, 0, stream>>>(disp, scale_bias, idx, loc, gates, out, K, S, M, C, w, 0);
  else if (K <= 2)
    gather_rows_kernel<T, 0, 2><<<ctas, kRowThreads, 0, stream>>>(disp, scale_bias, idx, loc, gates, out, K, S, M, C, w, 0);
  else
    gather_rows_kernel<T, 0, 8><<<ctas, kRowThreads, 0, stream>>>(disp, scale_bias, idx, loc, gates, out, K, S, M, C, w, 0);
}

// dgates[k][t] = <disp[slot_k(t)], dy[t]>.  With `scaled` != null the same pass also writes the
// gate-weighted rows scaled[t * K + k] = gates[k][t] * dy[t] (row index = the owner code of the slot
// map), so that a following dispatch-style send can move them with plain bulk copies.
template <class T>
__global__ void __launch_bounds__(kRowThreads, 8)
gate_grad_kernel(const T* __restrict__ disp, const T* __restrict__ dy, const int* __restrict__ idx,
                 const int* __restrict__ loc, float* __restrict__ dgates, const float* __restrict__ gates,
                 T* __restrict__ scaled, int K, int S, int M, int C, const float* __restrict__ disp_scales,
                 long long group_rows, unsigned char* __restrict__ scaled_q) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int V = Vec16<T>::N;
  const int nvec = M / V;
  for (int t = blockIdx.x * kRowWarps + warp; t < S; t += gridDim.x * kRowWarps) {
    const T* b = dy + (size_t)t * M;
    // int8 wire rows of the gate-weighted dy: gates are non-negative, so gate * dy quantises to the same bytes as
    // dy itself with range and low scaled by the gate; the row's range is found once per token
    float qlo = 0.f, qinv = 0.f, qrange = 0.f;
    if (scaled_q != nullptr) {
      float lo = INFINITY, hi = -INFINITY;
      for (int v = lane; v < nvec; v += 32) {
        Pack<T> pb = ld16(b + v * V);
#pragma unroll
        for (int i = 0; i < V; ++i) { const float f = to_f32(pb.v[i]); lo = fminf(lo, f); hi = fmaxf(hi, f); }
      }
      lo = warp_min(lo); hi = warp_max(hi);
      qlo = lo; qrange = hi - lo; qinv = qrange > 0.f ? 255.f / qrange : 0.f;
    }
    for (int k = 0; k < K; ++k) {
      const int e = idx[(size_t)k * S + t], l = loc[(size_t)k * S + t];
      float acc = 0.f;
      if (e >= 0 && l >= 0 && l < C) {
        const T* a = disp + ((size_t)e * C + l) * M;
        if (disp_scales != nullptr) {
          // the expert outputs arrived as uint8 rows with a (scale, low) pair per 128 columns and row
          const size_t slot = (size_t)e * C + l;
          const unsigned char* aq = reinterpret_cast<const unsigned char*>(disp) + slot * M;
          const float2* sc = reinterpret_cast<const float2*>(disp_scales);
          const float gw = gates != nullptr ? gates[(size_t)k * S + t] : 1.f;
          T* o = scaled != nullptr ? scaled + ((size_t)t * K + k) * M : nullptr;
          unsigned char* oq = scaled_q != nullptr ? scaled_q + ((size_t)t * K + k) * ((size_t)M + 16) : nullptr;
          for (int v = lane; v < M / 16; v += 32) {
            const float2 sl = sc[(size_t)(v >> 3) * group_rows + slot];
            const uint4 raw = *reinterpret_cast<const uint4*>(aq + (size_t)v * 16);
            const unsigned char* q = reinterpret_cast<const unsigned char*>(&raw);
            alignas(16) unsigned char qo[16];
#pragma unroll
            for (int h = 0; h < 16 / V; ++h) {
              Pack<T> pb = ld16(b + (size_t)v * 16 + h * V), po;
#pragma unroll
              for (int i = 0; i < V; ++i) {
                const float fb = to_f32(pb.v[i]);
                acc += fmaf(sl.x, (float)q[h * V + i], sl.y) * fb;
                po.v[i] = from_f32<T>(gw * fb);
                qo[h * V + i] = (unsigned char)fminf(fmaxf(rintf((fb - qlo) * qinv), 0.f), 255.f);
              }
              if (o != nullptr) st16(o + (size_t)v * 16 + h * V, po);
            }
            if (oq != nullptr) reinterpret_cast<uint4*>(oq)[v] = *reinterpret_cast<uint4*>(qo);
          }
          if (oq != nullptr && lane == 0)
            *reinterpret_cast<float4*>(oq + M) = make_float4(gw * qrange * (1.f / 255.f), gw * qlo, 0.f, 0.f);
        } else if (scaled != nullptr) {
          const float gw = gates[(size_t)k * S + t];
          T* o = scaled + ((size_t)t * K + k) * M;
          for (int v = lane; v < nvec; v += 32) {
            Pack<T> pa = ld16(a + v * V), pb = ld16(b + v * V), po;
#pragma unroll
            for (int i = 0; i < V; ++i) {
              const float fb = to_f32(pb.v[i]);
              acc += to_f32(pa.v[i]) * fb;
              po.v[i] = from_f32<T>(gw * fb);
            }
            st16(o + v * V, po);
          }
        } else {
          for (int v = lane; v < nvec; v += 32) {
            Pack<T> pa = ld16(a + v * V), pb = ld16(b + v * V);
#pragma unroll
            for (int i = 0; i < V; ++i) acc += to_f32(pa.v[i]) * to_f32(pb.v[i]);
          }
        }
      }
      acc = warp_sum(acc);
      if (lane == 0) dgates[(size_t)k * S + t] = acc;
    }
  }
}

template <class T>
void launch_gate_grad(const T* disp, const T* dy, const int* idx, const int* loc, float* dgates,
                      const float* gates, T* scaled, int K, int S, int M, int C, cudaStream_t stream,
                      const float* disp_scales, long long group_rows, unsigned char* scaled_q) {
  int ctas = (S + kRowWarps - 1) / kRowWarps;
  if (ctas > 148 * 8) ctas = 148 * 8;
  if (ctas < 1) ctas = 1;
  gate_grad_kernel<T><<<ctas, kRowThreads, 0, stream>>>(disp, dy, idx, loc, dgates, gates, scaled, K, S, M, C,
                                                        disp_scales, group_rows, scaled_q);
}

#define INSTANTIATE(T)                                                                             \
  template void launch_scatter_rows<T>(const T*, const int*, const float*, T*, int, int, int, int, \
                                       int, const PushArgs*, bool, cudaStream_t);                  \
  template void launch_gather_rows<T>(const void*, const float*, const int*, const int*,           \
                                      const float*, T*, int, int, int, int, const WaitArgs*,       \
                                      cudaStream_t, long long);                                    \
  template void launch_gate_grad<T>(const T*, const T*, const int*, const int*, float*, const float*, \
                                    T*, int, int, int, int, cudaStream_t, const float*, long long, unsigned char*);
INSTANTIATE(float)
INSTANTIATE(__nv_bfloat16)
INSTANTIATE(__half)

}  // namespace planmoe
