// Fused gate kernels (sm_100a): softmax + top-k + slot-location scan + slot map + GShard loss.
//
// One pass over the logits replaces the reference's chain of ~20 ATen launches plus its
// Blelloch-scan kernel (PlanMoE/impls/fast_dispatch.py:143-190, impls/losses.py:12-19,
// custom/custom_kernel.cpp:338-383).  Slot ordering is the reference's: within an expert, every
// k-th pick ranks after all (k-1)-th picks, and picks of equal k rank by token index.
//
//   gate_stats   per token: softmax, top-k (ties -> lower expert id), raw gate scores; per block:
//                (k, expert) histograms, in-block ranks, per-expert score sums.
//   gate_assign  per block: base offsets from the histograms of preceding blocks / lower k,
//                locations, normalised gates, slot map; block 0 also reduces the loss.
//   gate_bwd     per token: d(logits) from d(gates) and d(l_aux) (softmax recomputed).
//   cumsum_sub_one  stand-alone column-wise inclusive cumsum minus one of an int32 [S, E] mask.
//
// Everything is reduced in a fixed order: results are bit-reproducible run to run.

#include "planmoe.h"
#include "kernels/common.cuh"

namespace planmoe {

constexpr int kGateThreads = 64;    // small blocks: 8192 tokens still fill most SMs
constexpr int kGateWarps = kGateThreads / 32;
constexpr int kMaxE = 64;   // experts handled by the fused gate (per-thread register row)
constexpr int kMaxK = 4;

template <class T, int ME>
__device__ __forceinline__ void load_row(const T* row, int E, float* v) {
#pragma unroll
  for (int e = 0; e < ME; ++e) v[e] = (e < E) ? to_f32(row[e]) : -INFINITY;
}

template <class T, int ME>
__global__ void __launch_bounds__(kGateThreads)
gate_stats_kernel(const T* __restrict__ logits, int S, int E, int K,
                  int* __restrict__ idx,          // [K][S]
                  float* __restrict__ raw_gate,   // [K][S] un-normalised softmax score of pick k
                  int* __restrict__ rank_in_blk,  // [K][S]
                  int* __restrict__ blk_count,    // [nblk][K][E]
                  float* __restrict__ blk_score)  // [nblk][E]  sum of softmax scores
{
  __shared__ int warp_cnt[kGateWarps][kMaxK][kMaxE];
  __shared__ float score_sum[kGateWarps][kMaxE];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t = blockIdx.x * kGateThreads + tid;
  const bool live = t < S;

  for (int i = tid; i < kGateWarps * kMaxK * kMaxE; i += kGateThreads) (&warp_cnt[0][0][0])[i] = 0;
  __syncthreads();

  float p[ME];
  int pick[kMaxK];
  if (live) {
    load_row<T, ME>(logits + (size_t)t * E, E, p);
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < ME; ++e) mx = fmaxf(mx, p[e]);
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < ME; ++e) { p[e] = (e < E) ? expf(p[e] - mx) : 0.f; sum += p[e]; }
    const float inv = 1.f / sum;
#pragma unroll
    for (int e = 0; e < ME; ++e) p[e] *= inv;
  } else {
#pragma unroll
    for (int e = 0; e < ME; ++e) p[e] = 0.f;
  }

  // per-expert score sums: warp shuffle reduce, fixed order
#pragma unroll
  for (int e = 0; e < ME; ++e) {
    if (e < E) {
      float s = warp_sum(p[e]);
      if (lane == 0) score_sum[warp][e] = s;
    }
  }

  unsigned long long taken = 0ull;
  for (int k = 0; k < K; ++k) {
    int best = -1;
    float bv = -1.f;
#pragma unroll
    for (int e = 0; e < ME; ++e) {
      if (e < E && !((taken >> e) & 1ull) && p[e] > bv) { bv = p[e]; best = e; }
    }
    pick[k] = live ? best : -1;
    taken |= (best >= 0) ? (1ull << best) : 0ull;
    if (live) {
      idx[(size_t)k * S + t] = best;
      raw_gate[(size_t)k * S + t] = bv;
    }
    // rank among the lanes of this warp that picked the same expert for this k
    const unsigned peers = __match_any_sync(0xffffffffu, pick[k]);
    const int r = __popc(peers & ((1u << lane) - 1u));
    if (live && r == 0) warp_cnt[warp][k][best] = __popc(peers);
    pick[k] = live ? (best | (r << 8)) : -1;    // stash the in-warp rank
  }
  __syncthreads();

  for (int k = 0; k < K; ++k) {
    if (!live) break;
    const int e = pick[k] & 0xff, r = pick[k] >> 8;
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_cnt[w][k][e];
    rank_in_blk[(size_t)k * S + t] = before + r;
  }
  for (int i = tid; i < K * E; i += kGateThreads) {
    const int k = i / E, e = i - k * E;
    int c = 0;
    for (int w = 0; w < kGateWarps; ++w) c += warp_cnt[w][k][e];
    blk_count[((size_t)blockIdx.x * K + k) * E + e] = c;
  }
  for (int e = tid; e < E; e += kGateThreads) {
    float s = 0.f;
    for (int w = 0; w < kGateWarps; ++w) s += score_sum[w][e];
    blk_score[(size_t)blockIdx.x * E + e] = s;
  }
}

__global__ void __launch_bounds__(kGateThreads)
gate_assign_kernel(int S, int E, int K, int C, int normalize, float eps,
                   const int* __restrict__ idx, const float* __restrict__ raw_gate,
                   const int* __restrict__ rank_in_blk, const int* __restrict__ blk_count,
                   const float* __restrict__ blk_score, int nblk,
                   int* __restrict__ loc, float* __restrict__ gates, int* __restrict__ slot_map,
                   int* __restrict__ top1_count,  // [E] tokens whose first pick is e
                   float* __restrict__ l_aux)     // [1]
{
  __shared__ int base[kMaxK][kMaxE];
  __shared__ float red[kMaxE];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x;
  // base[k][e] = picks of expert e that rank before this block's k-th picks: every block's picks of a lower k,
  // then the k-th picks of the blocks before this one.  One warp per (k, e), lanes strided over that list.
  for (int i = warp; i < K * E; i += kGateWarps) {
    const int k = i / E, e = i - k * E;
    const int n = k * nblk + b;
    int acc = 0;
    for (int j = lane; j < n; j += 32) {
      const int kk = j / nblk, bb = j - kk * nblk;
      acc += blk_count[((size_t)bb * K + kk) * E + e];
    }
    acc = __reduce_add_sync(0xffffffffu, acc);
    if (lane == 0) base[k][e] = acc;
  }
  __syncthreads();

  const int t = b * kGateThreads + tid;
  if (t < S) {
    float g[kMaxK];
    float denom = 0.f;
    for (int k = 0; k < K; ++k) { g[k] = raw_gate[(size_t)k * S + t]; denom += g[k]; }
    const float scale = (normalize && K > 1) ? 1.f / fmaxf(denom, eps) : 1.f;
    for (int k = 0; k < K; ++k) {
      const int e = idx[(size_t)k * S + t];
      const int l = base[k][e] + rank_in_blk[(size_t)k * S + t];
      loc[(size_t)k * S + t] = l;
      gates[(size_t)k * S + t] = g[k] * scale;
      if (l < C) slot_map[(size_t)e * C + l] = t * K + k;
    }
  }

  if (b == 0) {
    // l_aux = E / S^2 * sum_e (sum_t score[t][e]) * (#tokens with top-1 == e); one warp per expert, lanes strided
    // over the blocks, lane sums combined by a shuffle tree: a fixed order
    for (int e = warp; e < E; e += kGateWarps) {
      float s = 0.f;
      int c = 0;
      for (int bb = lane; bb < nblk; bb += 32) {
        s += blk_score[(size_t)bb * E + e];
        c += blk_count[((size_t)bb * K + 0) * E + e];
      }
      s = warp_sum(s);
      c = __reduce_add_sync(0xffffffffu, c);
      if (lane == 0) {
        top1_count[e] = c;
        red[e] = s * (float)c;
      }
    }
    __syncthreads();
    if (tid == 0) {
      float acc = 0.f;
      for (int e = 0; e < E; ++e) acc += red[e];
      l_aux[0] = acc * (float)E / ((float)S * (float)S);
    }
  }
}

template <class T, int ME>
__global__ void __launch_bounds__(kGateThreads)
gate_bwd_kernel(const T* __restrict__ logits, int S, int E, int K, int normalize, float eps,
                const int* __restrict__ idx, const float* __restrict__ dgates,   // [K][S] or null
                const float* __restrict__ dl_aux,                                 // [1] or null
                const int* __restrict__ top1_count, T* __restrict__ dlogits) {
  const int t = blockIdx.x * kGateThreads + threadIdx.x;
  if (t >= S) return;
  float p[ME];
  load_row<T, ME>(logits + (size_t)t * E, E, p);
  float mx = -INFINITY;
#pragma unroll
  for (int e = 0; e < ME; ++e) mx = fmaxf(mx, p[e]);
  float sum = 0.f;
#pragma unroll
  for (int e = 0; e < ME; ++e) { p[e] = (e < E) ? expf(p[e] - mx) : 0.f; sum += p[e]; }
  const float inv = 1.f / sum;
#pragma unroll
  for (int e = 0; e < ME; ++e) p[e] *= inv;

  // d(score): loss part for every expert, gate part for the picked ones
  const float lw = dl_aux ? dl_aux[0] * (float)E / ((float)S * (float)S) : 0.f;
  int pk[kMaxK];
  float ds_pick[kMaxK];
  float denom = 0.f, dot = 0.f;
  for (int k = 0; k < K; ++k) {
    pk[k] = idx[(size_t)k * S + t];
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < ME; ++e) s = (e == pk[k]) ? p[e] : s;
    ds_pick[k] = s;    // temporarily the score
    denom += s;
  }
  const bool norm = normalize && K > 1;
  for (int k = 0; k < K; ++k) {
    const float dg = dgates ? dgates[(size_t)k * S + t] : 0.f;
    dot += dg * ds_pick[k];
  }
  for (int k = 0; k < K; ++k) {
    const float dg = dgates ? dgates[(size_t)k * S + t] : 0.f;
    if (norm) {
      if (denom > eps) ds_pick[k] = dg / denom - dot / (denom * denom);
      else ds_pick[k] = dg / eps;
    } else {
      ds_pick[k] = dg;
    }
  }
  float ds[ME];
  float inner = 0.f;
#pragma unroll
  for (int e = 0; e < ME; ++e) {
    float d = 0.f;
    if (e < E) {
      d = lw * (float)top1_count[e];
      for (int k = 0; k < K; ++k) d += (pk[k] == e) ? ds_pick[k] : 0.f;
    }
    ds[e] = d;
    inner += d * p[e];
  }
  T* out = dlogits + (size_t)t * E;
#pragma unroll
  for (int e = 0; e < ME; ++e)
    if (e < E) out[e] = from_f32<T>(p[e] * (ds[e] - inner));
}

template <class T>
void launch_gate_forward(const T* logits, int S, int E, int K, int C, bool normalize, float eps,
                         int* idx, int* loc, float* gates, float* raw_gate, int* slot_map,
                         int* top1_count, float* l_aux, int* ws_rank, int* ws_blk_count,
                         float* ws_blk_score, cudaStream_t stream) {
  const int nblk = (S + kGateThreads - 1) / kGateThreads;
  cudaMemsetAsync(slot_map, 0xFF, sizeof(int) * (size_t)E * C, stream);
  if (E <= 8)
    gate_stats_kernel<T, 8><<<nblk, kGateThreads, 0, stream>>>(logits, S, E, K, idx, raw_gate, ws_rank, ws_blk_count, ws_blk_score);
  else if (E <= 16)
    gate_stats_kernel<T, 16><<<nblk, kGateThreads, 0, stream>>>(logits, S, E, K, idx, raw_gate, ws_rank, ws_blk_count, ws_blk_score);
  else if (E <= 32)
    gate_stats_kernel<T, 32><<<nblk, kGateThreads, 0, stream>>>(logits, S, E, K, idx, raw_gate, ws_rank, ws_blk_count, ws_blk_score);
  else
    gate_stats_kernel<T, 64><<<nblk, kGateThreads, 0, stream>>>(logits, S, E, K, idx, raw_gate, ws_rank, ws_blk_count, ws_blk_score);
  gate_assign_kernel<<<nblk, kGateThreads, 0, stream>>>(S, E, K, C, normalize ? 1 : 0, eps, idx,
                                                      raw_gate, ws_rank, ws_blk_count, ws_blk_score,
                                                      nblk, loc, gates, slot_map, top1_count, l_aux);
}

template <class T>
void launch_gate_backward(const T* logits, int S, int E, int K, bool normalize, float eps,
                          const int* idx, const float* dgates, const float* dl_aux,
                          const int* top1_count, T* dlogits, cudaStream_t stream) {
  const int nblk = (S + kGateThreads - 1) / kGateThreads;
  const int nz = normalize ? 1 : 0;
  if (E <= 8)
    gate_bwd_kernel<T, 8><<<nblk, kGateThreads, 0, stream>>>(logits, S, E, K, nz, eps, idx, dgates, dl_aux, top1_count, dlogits);
  else if (E <= 16)
    gate_bwd_kernel<T, 16><<<nblk, kGateThreads, 0, stream>>>(logits, S, E, K, nz, eps, idx, dgates, dl_aux, top1_count, dlogits);
  else if (E <= 32)
    gate_bwd_kernel<T, 32><<<nblk, kGateThreads, 0, stream>>>(logits, S, E, K, nz, eps, idx, dgates, dl_aux, top1_count, dlogits);
  else
    gate_bwd_kernel<T, 64><<<nblk, kGateThreads, 0, stream>>>(logits, S, E, K, nz, eps, idx, dgates, dl_aux, top1_count, dlogits);
}

int gate_workspace_blocks(int S) { return (S + kGateThreads - 1) / kGateThreads; }

// ---- batch-prioritised routing: the order in which tokens claim slots -------------------------------
// The reference sorts tokens by the score of their best expert, highest first (importance = -max softmax
// score, PlanMoE/impls/fast_dispatch.py:135-138,153-154), and scans locations in that order.  Here the order
// comes from a counting rank: key[t] = max_e softmax(logits[t])[e] = 1 / sum_e exp(l[t][e] - max_e l[t]);
// rank[t] = number of tokens that go before t (larger key, or the same key and a lower index), perm = rank^-1.
// S^2 comparisons on fp32 keys staged through shared memory: exact, stable and free of sort libraries.
template <class T>
__global__ void __launch_bounds__(256)
importance_key_kernel(const T* __restrict__ logits, int S, int E, float* __restrict__ key) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= S) return;
  const T* row = logits + (size_t)t * E;
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) mx = fmaxf(mx, to_f32(row[e]));
  float sum = 0.f;
  for (int e = 0; e < E; ++e) sum += expf(to_f32(row[e]) - mx);
  key[t] = 1.f / sum;
}

// 32 tokens per CTA, eight threads per token: each thread counts over an eighth of every key tile, the eight
// counts are added by shuffles.  S / 32 CTAs keep the whole machine busy for a few thousand tokens.
__global__ void __launch_bounds__(256)
importance_rank_kernel(const float* __restrict__ key, int S, int* __restrict__ rank, int* __restrict__ perm) {
  __shared__ float tile[1024];
  const int part = threadIdx.x & 7;
  const int t = blockIdx.x * 32 + (threadIdx.x >> 3);
  const float mine = t < S ? key[t] : 0.f;
  int before = 0;
  for (int base = 0; base < S; base += 1024) {
    __syncthreads();
    for (int i = threadIdx.x; i < 1024; i += blockDim.x) tile[i] = base + i < S ? key[base + i] : -INFINITY;
    __syncthreads();
    const int n = min(1024, S - base);
    for (int i = part; i < n; i += 8) {
      const float other = tile[i];
      before += (other > mine || (other == mine && base + i < t)) ? 1 : 0;
    }
  }
  before += __shfl_xor_sync(0xffffffffu, before, 1);
  before += __shfl_xor_sync(0xffffffffu, before, 2);
  before += __shfl_xor_sync(0xffffffffu, before, 4);
  if (part == 0 && t < S) { rank[t] = before; perm[before] = t; }
}

template <class T>
void launch_importance_order(const T* logits, int S, int E, float* key, int* rank, int* perm, cudaStream_t stream) {
  if (S <= 0) return;
  importance_key_kernel<T><<<(S + 255) / 256, 256, 0, stream>>>(logits, S, E, key);
  importance_rank_kernel<<<(S + 31) / 32, 256, 0, stream>>>(key, S, rank, perm);
}
template void launch_importance_order<float>(const float*, int, int, float*, int*, int*, cudaStream_t);
template void launch_importance_order<__nv_bfloat16>(const __nv_bfloat16*, int, int, float*, int*, int*, cudaStream_t);
template void launch_importance_order<__half>(const __half*, int, int, float*, int*, int*, cudaStream_t);

// slot map of a permuted token order back to token ids: owner = position * K + k -> perm[position] * K + k
__global__ void remap_slot_map_kernel(int* __restrict__ slot_map, long long n, const int* __restrict__ perm, int K) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int o = slot_map[i];
  if (o >= 0) slot_map[i] = perm[o / K] * K + o % K;
}
void launch_remap_slot_map(int* slot_map, long long n, const int* perm, int K, cudaStream_t stream) {
  if (n > 0) remap_slot_map_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(slot_map, n, perm, K);
}

#define INSTANTIATE(T)                                                                            \
  template void launch_gate_forward<T>(const T*, int, int, int, int, bool, float, int*, int*,     \
                                       float*, float*, int*, int*, float*, int*, int*, float*,    \
                                       cudaStream_t);                                             \
  template void launch_gate_backward<T>(const T*, int, int, int, bool, float, const int*,         \
                                        const float*, const float*, const int*, T*, cudaStream_t);
INSTANTIATE(float)
INSTANTIATE(__nv_bfloat16)
INSTANTIATE(__half)

// ---- stand-alone cumsum - 1 -----------------------------------------------------------------
// Two passes over [S, E] int32: per-tile column sums, then each tile scans with the carried base.
constexpr int kScanRows = 128;

__global__ void cumsum_tile_sums_kernel(const int* __restrict__ x, int S, int E, int* __restrict__ tile_sum) {
  const int e = blockIdx.y * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const int r0 = blockIdx.x * kScanRows;
  int acc = 0;
  for (int r = r0; r < min(r0 + kScanRows, S); ++r) acc += x[(size_t)r * E + e];
  tile_sum[(size_t)blockIdx.x * E + e] = acc;
}

__global__ void cumsum_apply_kernel(const int* __restrict__ x, int S, int E,
                                    const int* __restrict__ tile_sum, int* __restrict__ out) {
  const int e = blockIdx.y * blockDim.x + threadIdx.x;
  if (e >= E) return;
  int acc = -1;
  for (int b = 0; b < (int)blockIdx.x; ++b) acc += tile_sum[(size_t)b * E + e];
  const int r0 = blockIdx.x * kScanRows;
  for (int r = r0; r < min(r0 + kScanRows, S); ++r) {
    acc += x[(size_t)r * E + e];
    out[(size_t)r * E + e] = acc;
  }
}

void launch_cumsum_sub_one(const int* x, int* out, int* tile_sum, int S, int E, cudaStream_t stream) {
  const int tiles = (S + kScanRows - 1) / kScanRows;
  const int threads = E < 128 ? ((E + 31) / 32) * 32 : 128;
  dim3 grid(tiles, (E + threads - 1) / threads);
  cumsum_tile_sums_kernel<<<grid, threads, 0, stream>>>(x, S, E, tile_sum);
  cumsum_apply_kernel<<<grid, threads, 0, stream>>>(x, S, E, tile_sum, out);
}
int cumsum_tiles(int S) { return (S + kScanRows - 1) / kScanRows; }

}  // namespace planmoe
