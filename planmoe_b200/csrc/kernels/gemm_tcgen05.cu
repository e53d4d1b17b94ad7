// Grouped bf16 GEMM for the expert FFNs on 5th-generation tensor cores (sm_100a).
//
//   D[g] (M x N) = A[g] (M x K) . B[g] (K x N)          g = 0 .. groups-1, fp32 accumulate
//
// Hand-written tcgen05 pipeline, one persistent CTA per SM, 384 threads in five roles.  By default two
// CTAs form a cluster and compute one 256 x 256 tile with tcgen05.mma.cta_group::2 (each CTA stages
// its own 128 rows of A and 128 of the 256 B columns; the even CTA issues the MMAs for both);
// problems with at most 128 rows per group run the one-CTA variant (128 x 256 tiles).
//   warp 0      TMA producer: cp.async.bulk.tensor (4-D maps, 128-byte swizzle) into a 5-stage
//               shared-memory ring (3-stage in the one-CTA variant; one stage less in launches that
//               carry a dispatch send, whose copy slots take the room), completion on the mbarrier of
//               the MMA-issuing CTA.  When the A operand is a receive buffer that peer GPUs fill,
//               the producer first acquire-waits (bounded) on the flag of every source rank whose
//               rows the tile touches: the GEMM starts on a tile as soon as its rows have landed
//               ("flag-gated A").
//   warp 1      MMA issuer: one thread issues tcgen05.mma.kind::f16, (128 or 256) x 256 x 16 per
//               instruction, accumulating in TMEM (2 x 256 columns, double buffered so the
//               epilogue of tile i overlaps the main loop of tile i+1); tcgen05.commit releases
//               ring stages and publishes the accumulator in every CTA of the group.
//   warps 2..9  epilogue: tcgen05.ld 32x32b -> registers -> bias / activation (saving its
//               derivative) / multiply by a saved derivative -> bf16 -> swizzled shared-memory
//               staging -> full-line 16-byte stores, either to local memory or straight into the
//               combine buffer of the rank that owns the token ("push"), followed by a release-add
//               on that rank's flag.  The TMEM load of the second half of a warp's columns is
//               issued under the stores of the first half.
//   warp 10     dispatch send (optional): while the tensor cores work, this warp of every CTA moves
//               token rows into the receive buffers of the ranks that own the experts with the
//               bulk-copy engine: cp.async.bulk global -> shared (row picked by slot map), an
//               optional int8 row quantisation in shared memory, cp.async.bulk shared -> peer
//               global; 64 KiB of slots are in flight per CTA, one slot per lane.  Work items are 16
//               rows for one destination, ordered the way the receivers consume them; when the stores
//               of an item have completed, the flag of the 128-row block they belong to on the
//               destination gets a release-add of the row count.  The producers of the same launch on
//               every rank are the flag-gated consumers, so the all-to-all and the GEMM that follows
//               it are one kernel and overlap 128 rows at a time; the copy never waits on another CTA
//               or rank, so no circular wait can form.
//   warp 11     de-quantiser (int8 wire only): waits for the arrival flag of a 128-row block of int8
//               rows in this rank's landing buffer, expands 32 rows at a time to the bf16 A operand
//               and release-adds the block's "ready" flag, which is what the TMA producer waits for.
//
// Operands may be K-major or MN-major (weights are stored input-major, and the weight-gradient
// GEMMs contract over the token dimension), so all four FFN GEMM flavours — forward, dgrad,
// wgrad — run on this one kernel without transposed copies.  A split-K "chunk" dimension lets a
// weight-gradient GEMM contract over all pipeline chunks of a receive buffer in one launch.
//
// TMA loads here never use cluster multicast and never read another GPU's memory: peer memory is
// only written (epilogue stores, bulk stores of the dispatch send) and signalled (flag adds); what
// a GPU computes on has landed in its own memory first.  Every wait (mbarrier or flag) is bounded:
// on expiry the CTA records a code in the status word, drains, frees its TMEM and returns.
//
// Takes the place of the reference's torch.matmul -> cuBLAS calls and separate bias / activation
// kernels (PlanMoE/experts/ffn.py:76-78) and of the permute copies around them
// (PlanMoE/impls/communicate.py:604-623).

#include "planmoe.h"
#include <algorithm>
#include "kernels/common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstring>
#include <mutex>

namespace planmoe {

namespace {

constexpr int BM = 128, BN = 256, BK = 64;       // BM = accumulator rows per CTA (TMEM lanes)
constexpr int UMMA_K = 16;
constexpr int kAccStages = 2;
constexpr int kThreads = 384;                     // TMA, MMA, 8 epilogue warps, copy warp, de-quantiser warp
constexpr uint32_t kCopyBytes = 65536;            // bulk-copy slots of the dispatch send: 16 x 4 KiB, 8 x 8 KiB or 4 x 16 KiB
constexpr uint32_t kCopyMinSlot = 4096, kCopyMaxSlot = 16384;
constexpr int kCopyMaxLanes = (int)(kCopyBytes / kCopyMinSlot);
constexpr uint32_t kZeroBytes = 1024;             // zeros, the source of rows for empty expert slots
constexpr uint32_t kSmemCopy = kCopyBytes + kZeroBytes;
constexpr int kGateBlock = 128;                   // rows per arrival flag of a flag-gated A operand (mode 1)
constexpr int kDequantRows = 32;                  // rows a de-quantiser warp expands per work unit
constexpr int kEpiWarps = 8;
constexpr uint32_t kABytes = BM * BK * 2;          // 16 KiB
constexpr uint32_t kStagingPerWarp = 32 * 128;     // one 32-row x 128-byte tile
constexpr uint32_t kSmemStaging = kEpiWarps * kStagingPerWarp;
constexpr uint32_t kSmemBias = BN * 4;
constexpr uint32_t kSmemBars = 512;

// Per-CTA geometry by CTA-group size CG.  CG = 1: one CTA computes a 128 x 256 tile from a 16 KiB A
// block and a 32 KiB B block per 64-deep K step.  CG = 2: a cluster of two CTAs computes a 256 x 256
// tile with one tcgen05.mma.cta_group::2 stream issued by the even CTA; each CTA stages its own 128
// rows of A and its own 128 of the 256 B columns (16 KiB each), so a K step costs 32 KiB of shared
// memory traffic per CTA instead of 48 and the ring is 5 deep instead of 3.
template <int CG, bool COPY> struct Geo {
  static constexpr int kBRows = BN / CG;                        // B columns staged per CTA
  static constexpr uint32_t kBBytes = kBRows * BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (CG == 1 ? 3 : 5) - (COPY ? 1 : 0);
  static constexpr uint32_t kSmemRing = kStages * kStageBytes;
  static constexpr uint32_t kCopyArea = COPY ? kSmemCopy : 0;
  // per epilogue warp 32 (scale, low) pairs of the int8 push epilogue (launches without a dispatch send only)
  static constexpr uint32_t kScaleArea = COPY ? 0 : kEpiWarps * 256;
  // ring | epilogue staging | bulk-copy slots of the dispatch send | bias | int8 scales | barriers.
  // No alignment slack: the dynamic shared array is declared 1024-byte aligned.
  static constexpr uint32_t kSmemTotal = kSmemRing + kSmemStaging + kCopyArea + kSmemBias + kScaleArea + kSmemBars;
};
static_assert(Geo<2, true>::kSmemTotal <= 232448 && Geo<1, true>::kSmemTotal <= 232448, "shared memory budget");
constexpr int kMaxStages = 6;
constexpr uint32_t kTmemCols = 512;

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
// TMA load into this CTA's shared memory.  `bar` is a shared::cluster address: the CTA's own barrier,
// or (cta_group::2) the barrier of the even CTA of the pair, which collects the bytes of both CTAs.
// No cluster multicast is used anywhere: every CTA fetches its own tiles.
template <int CG>
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
  if constexpr (CG == 1) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
  }
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CG == 1) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else                   asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  if constexpr (CG == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
  else                   asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
template <int CG>
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  if constexpr (CG == 1) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}
// Arrive on `bar` (a shared::cluster address, possibly in the other CTA of the pair) once every
// tcgen05.mma issued so far by this thread has completed.
template <int CG>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  else
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// ---- thread-block cluster helpers (CG = 2) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void epi_bar_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, Blackwell descriptor version 1.
//   bits [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4,
//   [46,48) version = 1, [61,64) layout = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation:
//   [4,6) D format = 1 (f32), [7,10) A format = 1 (bf16), [10,13) B format = 1 (bf16),
//   [15] A MN-major, [16] B MN-major, [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(bool a_mn, bool b_mn, int m) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct KernelParams {
  int groups, M, N, K;           // K per chunk
  int a_chunks;                  // split-K chunks (A and B agree)
  int epilogue, activation;
  __nv_bfloat16* D; long long d_row_stride, d_group_stride;
  __nv_bfloat16* aux; long long aux_row_stride, aux_group_stride;
  const __nv_bfloat16* bias; long long bias_group_stride;
  const unsigned long long* gate_flags; int gate_rows; unsigned long long gate_want;
  const unsigned long long* gate_want_ptr;
  int gate_mode, gate_nblk, perm_w, perm_q, perm_local, send_local_first;
  const void* a_ptr; long long a_row_stride, a_group_stride;   // the A operand as plain memory (de-quantiser output)
  const unsigned long long* heap_bases; unsigned long long push_data_off, push_flag_off;
  int push_rows, push_C, push_c0, push_chunk, W, my_rank;
  int push_q8;                   // push epilogue writes uint8 rows + one (scale, low) pair per 128 columns and row
  unsigned long long push_scale_off;   // heap offset of the pairs, fp32 [N / 128][rows of the destination buffer][2]
  long long push_rows_total;     // rows of the destination buffer (W * experts * push_C)
  // chunk_groups > 0: groups are [chunk][expert] with chunk_groups experts; weights / bias are indexed
  // by the expert, flags and push offsets by the chunk.
  int chunk_groups;
  unsigned long long budget_ns; int* status;
  GemmArgs::CopyJob copy;        // copy.ctas > 0: the copy warp of every CTA runs the dispatch send
  GemmArgs::DequantJob dequant;  // dequant.q != null: the de-quantiser warp of every CTA expands int8 rows
  int tma_out;                   // epilogue writes its staging tiles with bulk tensor stores (OutMaps valid)
  unsigned long long* trace;     // optional [grid][8] ns timestamps / durations of the roles (see GemmArgs::trace)
  int copy_dbg;                  // experiment switches of the copy role (PLANMOE_COPY_DBG)
};

// Tensor maps of the outputs, for the bulk tensor stores of the epilogue (box = 64 columns x 32 rows,
// 128-byte swizzle: exactly one epilogue warp's staging tile).  Plain-store epilogues: m[0] = D,
// m[1] = aux (the saved derivative).  Push epilogue: m[s] = the combine buffer of rank s.
struct OutMaps {
  CUtensorMap m[8];
};

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src_smem, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(src_smem), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

struct Ctl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[kAccStages];
  uint64_t acc_empty[kAccStages];
  uint64_t copy_full[kCopyMaxLanes];   // a row has landed in bulk-copy slot i
  uint32_t tmem_base;
  int dq_next;                 // next de-quantiser unit of this CTA (claimed by whichever warp is free)
  volatile int abort;
  volatile int epi_abort[2];   // written by epilogue warps before a barrier, read after it
};

// Bounded mbarrier wait: false on timeout or when another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Ctl* ctl, unsigned long long budget_ns,
                                          int* status, int role, int detail) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (ctl->abort) return false;
      if (global_timer_ns() - t0 > budget_ns) {
        ctl->abort = 1;
        report_status(status, kStatusMbarTimeout, role, detail, (int)parity);
        return false;
      }
    }
  }
  return true;
}

constexpr int kTraceSlots = 32;                    // u64 words of role trace per CTA
constexpr int kTraceTiles = 12;                    // per-tile gate waits recorded in slots 8 .. 31

__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Gaussian CDF and PDF at x with one exp2 and one approximate reciprocal: erf by the Abramowitz-Stegun
// 7.1.26 rational approximation (|error| < 1.5e-7, far below bf16 resolution); exp(-x^2/2) serves both.
__device__ __forceinline__ void gauss_cdf_pdf(float x, float& cdf, float& pdf) {
  const float z = fabsf(x) * 0.70710678118654752f;
  const float e = ex2_approx(-1.4426950408889634f * z * z);
  const float t = rcp_approx(fmaf(0.3275911f, z, 1.f));
  float poly = fmaf(t, 1.061405429f, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float half_erf = 0.5f - 0.5f * poly * t * e;            // erf(|x| / sqrt 2) / 2
  cdf = 0.5f + copysignf(half_erf, x);
  pdf = 0.3989422804014327f * e;
}

// Activation value and derivative in one go (they share the transcendental work).  ACT is a
// compile-time constant in the epilogue's inner loops.
template <int ACT>
__device__ __forceinline__ void act_both(float x, float& out, float& deriv) {
  if constexpr (ACT == kActRelu) {
    out = fmaxf(x, 0.f); deriv = x > 0.f ? 1.f : 0.f;
  } else if constexpr (ACT == kActGelu) {
    float cdf, pdf;
    gauss_cdf_pdf(x, cdf, pdf);
    out = x * cdf;
    deriv = fmaf(x, pdf, cdf);
  } else if constexpr (ACT == kActSilu) {
    const float sg = rcp_approx(1.f + ex2_approx(-1.4426950408889634f * x));
    out = x * sg;
    deriv = sg * fmaf(x, 1.f - sg, 1.f);
  } else {
    out = x; deriv = 1.f;
  }
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// ---------------------------------------------------------------------------------------------
// Tile order.  A tile index is (m-tile ordinal) * nt_count + n-tile; the m-tile ordinal runs over (group,
// m-tile) in the order in which the A rows become available.  Plain launches: groups in order, m-tiles in
// order.  When the A operand is filled by the fused dispatch send and every source rank's segment of a group
// holds perm_q > 1 whole tiles:
//   perm_local == 0: within a group the m-tiles are visited segment-interleaved (tile 0 of every source, then
//                    tile 1 of every source, ...), the order in which the senders deliver rows;
//   perm_local == 1: within a pipeline chunk, first this rank's own segment of every group (those rows never
//                    cross a link and the senders deliver them first), then, group by group, the other
//                    sources segment-interleaved starting at the right-hand neighbour.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mtile_coord(const KernelParams& p, int ord, int mt_count, int& g, int& mt) {
  if (p.perm_q <= 1) {
    g = ord / mt_count;
    mt = ord - g * mt_count;
    return;
  }
  if (!p.perm_local) {
    g = ord / mt_count;
    const int l = ord - g * mt_count;
    mt = (l % p.perm_w) * p.perm_q + l / p.perm_w;
    return;
  }
  const int gpc = p.chunk_groups > 0 ? p.chunk_groups : p.groups;      // groups of one pipeline chunk
  const int per_chunk = gpc * mt_count;
  const int chunk = ord / per_chunk;
  int u = ord - chunk * per_chunk;
  int el;
  if (u < gpc * p.perm_q) {                                            // own segments
    el = u / p.perm_q;
    mt = p.my_rank * p.perm_q + (u - el * p.perm_q);
  } else {
    u -= gpc * p.perm_q;
    const int others = p.perm_w - 1, rem = others * p.perm_q;
    el = u / rem;
    const int l = u - el * rem;
    int src = p.my_rank + 1 + l % others;
    if (src >= p.perm_w) src -= p.perm_w;
    mt = src * p.perm_q + l / others;
  }
  g = chunk * gpc + el;
}

__device__ __forceinline__ void red_release_gpu_add(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Copy role (warp 10 of every CTA): the dispatch send, driven by the bulk-copy engine.
//
// The 64 KiB copy area is cut into slots of one row each (16 slots for rows of up to 4 KiB, 8 for 8 KiB,
// 4 for 16 KiB), one lane per slot, in two sets that alternate from item to item.  A work item is `half`
// consecutive rows of one (chunk, local expert) group for one destination rank, i.e. one contiguous range of
// the destination's receive buffer [chunk][E_local][W_src][C/chunks][row]; item ids are ordered (group, row
// range, destination), the order in which the destinations consume rows, and CTA b takes items b, b + grid, ...
//
// The loop is software-pipelined so that no step waits for something it has just started:
//   iteration k   (1) the rows of item k, whose bulk loads were started one iteration ago, have landed in set
//                     k & 1: start their bulk stores into the peer's buffer (an empty expert slot is stored as
//                     zeros from a zero region instead) and commit them;
//                 (2) the stores of item k-1 have read the other set: look up the rows of item k+1 in the slot
//                     map and start their bulk loads into it;
//                 (3) the stores of item k-1 have completed: lane 31, which never issues a copy, adds the
//                     item's row count to the flag of the 128-row block it lies in on its destination (a
//                     relaxed add: the data it publishes has already been performed).
// Rows are moved as they are: int8 rows are quantised by the caller beforehand.  Nothing here waits on another
// CTA or rank.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void bulk_wait_group_1() { asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); }

__device__ __forceinline__ void copy_role(const KernelParams& p, uint8_t* cring, Ctl* ctl) {
  const GemmArgs::CopyJob& c = p.copy;
  const int lane = threadIdx.x & 31;
  const int Cc = c.C / c.chunks;
  const uint32_t row_bytes = (uint32_t)c.row_bytes;              // the same at the source and at the destination
  uint32_t slot_bytes = kCopyMinSlot;
  while (slot_bytes < row_bytes) slot_bytes <<= 1;               // host guarantees row_bytes <= kCopyMaxSlot
  const int slots = (int)(kCopyBytes / slot_bytes);
  const int half = slots / 2;                                    // rows per item
  const int items_per_seg = (Cc + half - 1) / half;
  const long long n_items = (long long)c.chunks * c.E_local * items_per_seg * p.W;
  const uint8_t* x = reinterpret_cast<const uint8_t*>(c.x);
  const uint32_t my_slot_s = smem_u32(cring + (lane < slots ? lane : 0) * slot_bytes);
  const uint32_t zero_s = smem_u32(cring + kCopyBytes);
  const uint32_t my_bar = smem_u32(&ctl->copy_full[lane < slots ? lane : 0]);
  const int my_set = lane < slots ? lane / half : -1;
  const int li = lane < slots ? lane - my_set * half : 0;        // my row within an item of my set
  uint32_t phase = 0;                                            // parity of my slot's barrier
  bool ok = true;

  for (uint32_t i = lane; i < kZeroBytes / 16; i += 32)
    reinterpret_cast<uint4*>(cring + kCopyBytes)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async();                                           // zeros visible to the bulk-copy engine
  __syncwarp();

  // geometry of an item (uniform over the warp)
  struct Item { int r, g, j, el, row0, nrows; };
  // Item order.  send_local_first == 0: (group, row range, destination) with the destinations starting at my
  // right-hand neighbour.  send_local_first == 1: chunk by chunk, first the items that stay on this rank (every
  // group of the chunk), then the others as (group, row range, destination): the destinations' tile loops start
  // on their own rows, which reach them without crossing a link.
  const long long per_chunk_loc = (long long)c.E_local * items_per_seg;
  const long long per_chunk = per_chunk_loc * p.W;
  auto decode = [&](long long item) {
    Item it;
    int rr, sub;
    if (!p.send_local_first || p.W == 1) {
      rr = (int)(item % p.W);
      long long t = item / p.W;
      sub = (int)(t % items_per_seg);
      it.g = (int)(t / items_per_seg);                           // chunk * E_local + local expert
      it.j = it.g / c.E_local; it.el = it.g - it.j * c.E_local;
    } else {
      it.j = (int)(item / per_chunk);
      long long t = item - (long long)it.j * per_chunk;
      if (t < per_chunk_loc) {
        rr = p.W - 1;                                            // myself
      } else {
        t -= per_chunk_loc;
        rr = (int)(t % (p.W - 1));
        t /= (p.W - 1);
      }
      sub = (int)(t % items_per_seg);
      it.el = (int)(t / items_per_seg);
      it.g = it.j * c.E_local + it.el;
    }
    it.r = (p.my_rank + 1 + rr) % p.W;                           // rr == W - 1 is this rank
    it.row0 = sub * half;
    it.nrows = min(half, Cc - it.row0);
    return it;
  };
  // my row of the item in flight in my set: where it goes and whether a bulk load is bringing it
  uint8_t* dst = nullptr;
  bool have_row = false, loaded = false;
  auto start_row = [&](const Item& it) {        // called by the lanes of the item's set
    have_row = li < it.nrows;
    loaded = false;
    if (!have_row) return;
    const int cc = it.row0 + li;
    const int owner = c.slot_map[(size_t)(it.r * c.E_local + it.el) * c.C + it.j * Cc + cc];
    dst = reinterpret_cast<uint8_t*>(p.heap_bases[it.r]) + c.data_off +
          (((size_t)it.g * p.W + p.my_rank) * Cc + cc) * row_bytes;
    if (owner >= 0) {
      // source row = token of the pick (gate-weighted sources hold one row per (token, pick): K == 1 then)
      const int tok = owner / c.K;
      bulk_wait_read_all();                                      // the store that last used my slot has read it
      mbar_expect_tx(my_bar, row_bytes);
      bulk_load(my_slot_s, x + (size_t)tok * row_bytes, row_bytes, my_bar);
      loaded = true;
    }
  };

  // the two items whose stores may still be in flight ([0] = the older one): destination rank, group, first row
  // in the group, rows
  int pend_n = 0;
  int pend_r[2] = {0, 0}, pend_g[2] = {0, 0}, pend_first[2] = {0, 0}, pend_rows[2] = {0, 0};
  auto signal_oldest = [&]() {
    // rows [first, first + rows) of group g on rank r have landed
    unsigned long long* flags = reinterpret_cast<unsigned long long*>(
        reinterpret_cast<uint8_t*>(p.heap_bases[pend_r[0]]) + c.flag_off) + (size_t)pend_g[0] * c.nblk;
    // The item's bulk stores have completed (wait_group in the lanes that issued them, then __syncwarp), so the
    // flag update needs no release of its own; PLANMOE_COPY_DBG=1 restores fence + release for comparison.
    if (p.copy_dbg & 1) __threadfence_system();
    int first = pend_first[0], left = pend_rows[0];
    while (left > 0) {
      const int blk = first / kGateBlock;
      const int n = min(left, (blk + 1) * kGateBlock - first);
      if (p.copy_dbg & 1) red_release_sys_add(flags + blk, (unsigned long long)n);
      else                red_relaxed_sys_add(flags + blk, (unsigned long long)n);
      first += n; left -= n;
    }
  };
  auto pop_oldest = [&]() {
    pend_r[0] = pend_r[1]; pend_g[0] = pend_g[1]; pend_first[0] = pend_first[1]; pend_rows[0] = pend_rows[1];
    --pend_n;
  };

  long long item = blockIdx.x;
  int set = 0;
  if (item < n_items && my_set == 0) start_row(decode(item));
  for (; item < n_items && ok; item += gridDim.x, set ^= 1) {
    const Item it = decode(item);
    // (1) item `item`: rows have landed (or are zeros) -> stores
    if (my_set == set) {
      if (have_row && loaded) {
        ok = mbar_wait(my_bar, phase, ctl, p.budget_ns, p.status, 3, lane);
        phase ^= 1u;
        if (ok) bulk_store(dst, my_slot_s, row_bytes);
      } else if (have_row) {
        for (uint32_t o = 0; o < row_bytes; o += kZeroBytes)     // empty expert slot: a row of zeros
          bulk_store(dst + o, zero_s, min(kZeroBytes, row_bytes - o));
      }
      bulk_commit();                 // one group per lane and item of its set, empty if the item has no row for me
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    // (2) the next item of this CTA goes into the other set
    if (item + gridDim.x < n_items && my_set == (set ^ 1)) start_row(decode(item + gridDim.x));
    // (3) the other set's lanes wait for their stores, those of the item before this one, to complete (the loads
    // of the next item and the stores of this one are in flight meanwhile); this set's lanes keep this item
    // pending.  The item before is then complete and can be published.
    if (my_set == set) bulk_wait_group_1(); else bulk_wait_all();
    __syncwarp();
    if (pend_n == 1) {
      if (lane == 31 && !(p.copy_dbg & 2)) signal_oldest();
      pop_oldest();
    }
    pend_r[pend_n] = it.r; pend_g[pend_n] = it.g; pend_first[pend_n] = p.my_rank * Cc + it.row0;
    pend_rows[pend_n] = it.nrows;
    ++pend_n;
  }
  bulk_wait_all();                                               // nothing of mine is in flight any more
  __syncwarp();
  while (ok && pend_n > 0) {
    if (lane == 31 && !(p.copy_dbg & 2)) signal_oldest();
    pop_oldest();
  }
  if (ok && (p.copy_dbg & 2) && lane == 31) {                    // experiment: all signals at the end
    for (long long it2 = blockIdx.x; it2 < n_items; it2 += gridDim.x) {
      const Item q = decode(it2);
      pend_r[0] = q.r; pend_g[0] = q.g; pend_first[0] = p.my_rank * Cc + q.row0; pend_rows[0] = q.nrows;
      signal_oldest();
    }
  }
}

// ---------------------------------------------------------------------------------------------
// De-quantiser role (warp 11 of every CTA, int8 wire only).  Units of 32 rows, numbered in the order in
// which the tiles of this launch consume them; CTA b takes units b, b + grid, ...  A unit waits (bounded,
// lane 0) until the arrival flag of its 128-row block shows that all of the block's rows have landed, the
// warp expands the rows q * scale + low to bf16 in the A operand, and lane 0 release-adds the unit's row
// count to the block's ready flag.  The role depends only on peers' copy warps, which never wait.
// ---------------------------------------------------------------------------------------------
template <int CG>
__device__ __forceinline__ void dequant_role(const KernelParams& p, __nv_bfloat16* a_base, long long a_row_stride,
                                             long long a_group_stride, int mt_count, Ctl* ctl) {
  const GemmArgs::DequantJob& d = p.dequant;
  const int lane = threadIdx.x & 31;
  const unsigned long long uses = p.gate_want_ptr != nullptr ? *p.gate_want_ptr : p.gate_want;
  constexpr int kUnitsPerBlock = kGateBlock / kDequantRows;
  const long long n_units = (long long)p.groups * mt_count * CG * kUnitsPerBlock;
  const size_t q_row = (size_t)d.M + 16;
  const uint8_t* qbase = reinterpret_cast<const uint8_t*>(d.q);
  // The CTA's units (blockIdx.x, blockIdx.x + grid, ...) are claimed one at a time from a shared counter, in order:
  // the de-quantiser warp starts at once, the copy warp joins when its sends are done.
  while (true) {
    int k = 0;
    if (lane == 0) k = atomicAdd(&ctl->dq_next, 1);
    k = __shfl_sync(0xffffffffu, k, 0);
    const long long u = (long long)blockIdx.x + (long long)k * gridDim.x;
    if (u >= n_units) break;
    const int sub = (int)(u % kUnitsPerBlock);
    long long t = u / kUnitsPerBlock;
    const int b = (int)(t % CG); t /= CG;
    int g, mt;
    mtile_coord(p, (int)t, mt_count, g, mt);
    const int blk = mt * CG + b;
    const int row0 = blk * kGateBlock + sub * kDequantRows;
    if (row0 >= p.M) continue;
    const int rows_blk = min(kGateBlock, p.M - blk * kGateBlock);
    const int nrows = min(kDequantRows, p.M - row0);
    bool ok = true;
    if (lane == 0)
      ok = wait_flag_ge(d.arrival + (size_t)g * p.gate_nblk + blk, uses * (unsigned long long)rows_blk, p.budget_ns,
                        p.status, 2000 + blk);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) return;
    // Four rows at a time, four 16-byte pieces per lane and row in flight (sixteen independent loads per lane), so
    // that the warp streams instead of waiting for one load after the other.
    constexpr int kRB = 4;
    const int pieces = d.M / 16;
    for (int r = 0; r < nrows; r += kRB) {
      const uint8_t* src[kRB];
      __nv_bfloat16* dstp[kRB];
      float2 sl[kRB];
#pragma unroll
      for (int b = 0; b < kRB; ++b) {
        const int rr = min(r + b, nrows - 1);                    // rows past the end repeat the last one (not stored)
        src[b] = qbase + ((size_t)g * p.M + row0 + rr) * q_row;
        dstp[b] = a_base + (long long)g * a_group_stride + (long long)(row0 + rr) * a_row_stride;
        sl[b] = *reinterpret_cast<const float2*>(src[b] + d.M);
      }
      for (int v0 = 0; v0 < pieces; v0 += 128) {
        uint4 raw[kRB][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int v = v0 + i * 32 + lane;
          if (v < pieces) {
#pragma unroll
            for (int b = 0; b < kRB; ++b) raw[b][i] = *reinterpret_cast<const uint4*>(src[b] + (size_t)v * 16);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int v = v0 + i * 32 + lane;
          if (v >= pieces) continue;
#pragma unroll
          for (int b = 0; b < kRB; ++b) {
            if (r + b >= nrows) continue;
            const uint32_t w[4] = {raw[b][i].x, raw[b][i].y, raw[b][i].z, raw[b][i].w};
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float f0 = fmaf((float)(w[j] & 0xffu), sl[b].x, sl[b].y);
              const float f1 = fmaf((float)((w[j] >> 8) & 0xffu), sl[b].x, sl[b].y);
              const float f2 = fmaf((float)((w[j] >> 16) & 0xffu), sl[b].x, sl[b].y);
              const float f3 = fmaf((float)(w[j] >> 24), sl[b].x, sl[b].y);
              o[2 * j] = pack_bf16(f0, f1);
              o[2 * j + 1] = pack_bf16(f2, f3);
            }
            __nv_bfloat16* dst = dstp[b] + (size_t)v * 16;
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
      }
    }
    __threadfence();
    __syncwarp();
    if (lane == 0) red_release_gpu_add(d.ready + (size_t)g * p.gate_nblk + blk, (unsigned long long)nrows);
  }
}

// Bias + activation on one thread's 64 accumulator values: the packed activation goes to `opk`, the
// packed derivative into the thread's row of the (swizzled) staging tile.
template <int ACT>
__device__ __forceinline__ void slab_bias_act(const uint32_t* v, const float* bias, uint8_t* st_row, int lane,
                                              uint4* opk) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const float4 b0 = *reinterpret_cast<const float4*>(bias + c * 8);
    const float4 b1 = *reinterpret_cast<const float4*>(bias + c * 8 + 4);
    const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    float f[8], d[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) act_both<ACT>(__uint_as_float(v[c * 8 + i]) + bb[i], f[i], d[i]);
    *reinterpret_cast<uint4*>(st_row + ((c ^ (lane & 7)) << 4)) =
        make_uint4(pack_bf16(d[0], d[1]), pack_bf16(d[2], d[3]), pack_bf16(d[4], d[5]), pack_bf16(d[6], d[7]));
    opk[c] = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
  }
}

template <int CG, bool A_MN, bool B_MN, int EPI, bool COPY>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ OutMaps om, const KernelParams p) {
  using G = Geo<CG, COPY>;
  constexpr int kStages = G::kStages;
  constexpr uint32_t kStageBytes = G::kStageBytes;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0u) {            // swizzled tiles need 1024-byte aligned stages
    if (threadIdx.x == 0) report_status(p.status, kStatusBadArgument, 1024, (int)(smem_u32(smem) & 1023u), 0);
    return;                                        // same address in every CTA: the whole grid returns
  }
  // A work unit is one output tile of (CG * 128) x 256, computed by CG CTAs; `unit` / `nunits` number
  // the CTA groups of the grid and `cr` is this CTA's rank inside its group (0 issues the MMAs).
  const int cr = CG == 1 ? 0 : (int)cluster_ctarank();
  const int unit = (int)blockIdx.x / CG, nunits = (int)gridDim.x / CG;
  uint8_t* ring = smem;
  uint8_t* staging = smem + G::kSmemRing;
  uint8_t* cring = smem + G::kSmemRing + kSmemStaging;
  float* bias_s = reinterpret_cast<float*>(smem + G::kSmemRing + kSmemStaging + G::kCopyArea);
  uint8_t* scale_s = smem + G::kSmemRing + kSmemStaging + G::kCopyArea + kSmemBias;
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + G::kSmemRing + kSmemStaging + G::kCopyArea + kSmemBias + G::kScaleArea);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned long long* trace = p.trace != nullptr ? p.trace + (size_t)blockIdx.x * kTraceSlots : nullptr;
  if (trace != nullptr && threadIdx.x == 0) trace[0] = global_timer_ns();

  const int mt_count = (p.M + BM * CG - 1) / (BM * CG);
  const int nt_count = (p.N + BN - 1) / BN;
  const int tiles = p.groups * mt_count * nt_count;
  const int kb_per_chunk = (p.K + BK - 1) / BK;
  const int kb_total = kb_per_chunk * p.a_chunks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&ctl->full[s]), 1); mbar_init(smem_u32(&ctl->empty[s]), 1); }
    for (int a = 0; a < kAccStages; ++a) {
      mbar_init(smem_u32(&ctl->acc_full[a]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[a]), kEpiWarps * CG);     // the epilogue warps of every CTA of the group
    }
    for (int i = 0; i < kCopyMaxLanes; ++i) mbar_init(smem_u32(&ctl->copy_full[i]), 1);
    ctl->abort = 0;
    ctl->dq_next = 0;
    ctl->epi_abort[0] = ctl->epi_abort[1] = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc<CG>(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish<CG>();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();       // the partner's barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      unsigned long long gate_wait_ns = 0;
      int traced_tiles = 0;
      const unsigned long long gate_want = p.gate_want_ptr != nullptr ? *p.gate_want_ptr : p.gate_want;
      for (int tile = unit; tile < tiles && ok; tile += nunits) {
        const int nt = tile % nt_count;
        int g, mt;
        mtile_coord(p, tile / nt_count, mt_count, g, mt);
        const int m0 = mt * (BM * CG) + cr * BM;                         // my 128 rows of the tile
        const int n0 = nt * BN + cr * G::kBRows;                         // my share of the B columns
        const int gb = p.chunk_groups > 0 ? g % p.chunk_groups : g;      // group of the B operand
        if (p.gate_flags != nullptr && m0 < p.M) {
          const unsigned long long tw0 = trace != nullptr ? global_timer_ns() : 0ull;
          if (p.gate_mode == 1) {
            // one flag per 128-row block, counting rows: mine is complete after `gate_want` fillings
            const int blk = m0 / kGateBlock;
            const unsigned long long rows_blk = (unsigned long long)min(kGateBlock, p.M - blk * kGateBlock);
            ok = wait_flag_ge(p.gate_flags + (size_t)g * p.gate_nblk + blk, gate_want * rows_blk, p.budget_ns,
                              p.status, 1000 + blk);
          } else {
            const int last_row = min(m0 + BM, p.M) - 1;
            const int s_lo = m0 / p.gate_rows, s_hi = last_row / p.gate_rows;
            for (int s = s_lo; s <= s_hi && ok; ++s)
              ok = wait_flag_ge(p.gate_flags + (p.chunk_groups > 0 ? (g / p.chunk_groups) * p.W : 0) + s, gate_want,
                                p.budget_ns, p.status, s);
          }
          if (!ok) { ctl->abort = 1; break; }
          fence_proxy_async();   // peers' generic-proxy stores -> this thread's async-proxy loads
          if (trace != nullptr) {
            const unsigned long long tw1 = global_timer_ns();
            gate_wait_ns += tw1 - tw0;
            if (traced_tiles < kTraceTiles) {        // when this CTA asked for the tile's rows and when it had them
              trace[8 + 2 * traced_tiles] = tw0;
              trace[9 + 2 * traced_tiles] = tw1;
              ++traced_tiles;
            }
          }
        }
        for (int kb = 0; kb < kb_total; ++kb) {
          ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, ctl, p.budget_ns, p.status, 0, stage);
          if (!ok) break;
          // bytes of every CTA of the group complete on the barrier of the CTA that issues the MMAs
          uint32_t full = smem_u32(&ctl->full[stage]);
          if constexpr (CG == 2) full = map_to_cta(full, 0);
          const uint32_t sa = smem_u32(ring + stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
          const int chunk = kb / kb_per_chunk;
          const int k0 = (kb - chunk * kb_per_chunk) * BK;
          if (cr == 0) mbar_expect_tx(smem_u32(&ctl->full[stage]), kStageBytes * CG);
          if constexpr (!A_MN) {
            tma_load_4d<CG>(sa, &tmA, full, k0, m0, g, chunk);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_4d<CG>(sa + i * (64 * BK * 2), &tmA, full, m0 + i * 64, k0, g, chunk);
          }
          if constexpr (!B_MN) {
            tma_load_4d<CG>(sb, &tmB, full, k0, n0, gb, chunk);
          } else {
#pragma unroll
            for (int i = 0; i < G::kBRows / 64; ++i)
              tma_load_4d<CG>(sb + i * (64 * BK * 2), &tmB, full, n0 + i * 64, k0, gb, chunk);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) __nanosleep(200000);   // let bulk copies already in flight land before teardown
      if (trace != nullptr) trace[3] = gate_wait_ns;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (rank 0 of the group)
    if (lane == 0 && cr == 0) {
      constexpr uint32_t idesc = make_idesc(A_MN, B_MN, BM * CG);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = unit; tile < tiles && ok; tile += nunits) {
        ok = mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, ctl, p.budget_ns, p.status, 1, 100 + acc);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kb_total; ++kb) {
          ok = mbar_wait(smem_u32(&ctl->full[stage]), phase, ctl, p.budget_ns, p.status, 1, stage);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(ring + stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t adesc, bdesc;
            if constexpr (!A_MN) adesc = make_desc(sa + k * (UMMA_K * 2), 16, 1024);
            else                 adesc = make_desc(sa + k * (UMMA_K * 128), 64 * BK * 2, 1024);
            if constexpr (!B_MN) bdesc = make_desc(sb + k * (UMMA_K * 2), 16, 1024);
            else                 bdesc = make_desc(sb + k * (UMMA_K * 128), 64 * BK * 2, 1024);
            umma_bf16<CG>(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the ring stage is free again in every CTA of the group once these MMAs have read it
          umma_commit<CG>(smem_u32(&ctl->empty[stage]));
          if constexpr (CG == 2) umma_commit<CG>(map_to_cta(smem_u32(&ctl->empty[stage]), 1));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit<CG>(smem_u32(&ctl->acc_full[acc]));
        if constexpr (CG == 2) umma_commit<CG>(map_to_cta(smem_u32(&ctl->acc_full[acc]), 1));
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 2 + kEpiWarps) {
    // ------------------------------------------------------------------ dispatch send (copy warp)
    if constexpr (COPY) {
      if (p.copy.ctas > 0) {
        if (trace != nullptr && lane == 0) trace[1] = global_timer_ns();
        copy_role(p, cring, ctl);
        if (trace != nullptr && lane == 0) trace[2] = global_timer_ns();
      }
      if constexpr (!A_MN) {
        if (p.dequant.q != nullptr)              // sends done: help expanding the int8 rows that arrive
          dequant_role<CG>(p, const_cast<__nv_bfloat16*>(reinterpret_cast<const __nv_bfloat16*>(p.a_ptr)), p.a_row_stride,
                           p.a_group_stride, mt_count, ctl);
      }
    }
  } else if (warp == 3 + kEpiWarps) {
    // ------------------------------------------------------------------ de-quantiser warp (int8 wire)
    if constexpr (COPY && !A_MN) {
      if (p.dequant.q != nullptr)
        dequant_role<CG>(p, const_cast<__nv_bfloat16*>(reinterpret_cast<const __nv_bfloat16*>(p.a_ptr)), p.a_row_stride,
                         p.a_group_stride, mt_count, ctl);
      if (trace != nullptr && lane == 0) trace[5] = global_timer_ns();
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (8)
    // Warp pairs share a TMEM lane quarter (warp % 4); each warp of a pair drains one 128-column
    // half of the accumulator, in two 64-column slabs.
    const int ewarp = warp - 2;                   // 0..7
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int half = ewarp >> 2;
    uint8_t* st0 = staging + ewarp * kStagingPerWarp;
    const int etid = threadIdx.x - 64;            // 0..255
    uint32_t acc = 0, acc_phase = 0, iter = 0;
    bool ok = true;
    long long epi_acc_clk = 0, epi_stage_clk = 0;  // trace: SM clocks spent waiting for the accumulator / the staging tile
    const long long epi_t0 = trace != nullptr ? clock64() : 0ll;
    for (int tile = unit; tile < tiles && ok; tile += nunits) {
      const int nt = tile % nt_count;
      int g, mt;
      mtile_coord(p, tile / nt_count, mt_count, g, mt);
      const int m0 = mt * (BM * CG) + cr * BM, n0 = nt * BN;

      // Activation backward: the 32 x 64 slab of saved activation derivatives this warp needs first
      // is requested before the accumulator is awaited, so its latency hides behind the main loop.
      // Loads are full-line (4 rows x 128 bytes per instruction).
      uint4 araw[8];
      auto load_aux_slab = [&](int nb) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r = it * 4 + (lane >> 3), c = lane & 7;
          const int m = m0 + q * 32 + r;
          araw[it] = make_uint4(0, 0, 0, 0);
          if (m < p.M && nb + c * 8 < p.N)
            araw[it] = __ldg(reinterpret_cast<const uint4*>(
                p.aux + (long long)g * p.aux_group_stride + (long long)m * p.aux_row_stride + nb + c * 8));
        }
      };
      if constexpr (EPI == kEpiDAct) load_aux_slab(n0 + half * 128);

      // All epilogue warps take the same exit decision: a warp that timed out raises the flag of
      // this iteration's parity before the barrier, everyone reads it after the barrier.
      const long long tq0 = trace != nullptr ? clock64() : 0ll;
      bool got = mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, ctl, p.budget_ns, p.status, 2, acc);
      got = __all_sync(0xffffffffu, got);
      if (trace != nullptr) epi_acc_clk += clock64() - tq0;
      if (!got && lane == 0) ctl->epi_abort[iter & 1] = 1;
      epi_bar_sync();                              // also: previous tile's readers of bias_s are done
      if (ctl->epi_abort[iter & 1]) { ok = false; break; }
      ++iter;
      for (int i = etid; i < BN; i += kEpiWarps * 32) {
        float b = 0.f;
        if (p.bias != nullptr && n0 + i < p.N)
          b = __bfloat162float(p.bias[(long long)(p.chunk_groups > 0 ? g % p.chunk_groups : g) * p.bias_group_stride + n0 + i]);
        bias_s[i] = b;
      }
      epi_bar_sync();
      tc_fence_after();

      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + half * 128;

      // Push epilogue: where row (m0 + q * 32 + lane) of this tile lives in the combine buffer of the
      // rank that owns the token (0 = row outside the problem).
      unsigned long long push_row = 0ull;
      int push_s = 0, push_drow = 0;               // bulk-store form: rank and row of the slice's first row
      if constexpr (EPI == kEpiPush) {
        {
          const int mf = m0 + q * 32;
          const int s = mf / p.push_rows, cc = mf - s * p.push_rows;
          const int el = p.chunk_groups > 0 ? g % p.chunk_groups : g;
          const int nel = p.chunk_groups > 0 ? p.chunk_groups : p.groups;
          const int c_base = p.chunk_groups > 0 ? (g / p.chunk_groups) * p.push_rows : p.push_c0;
          push_s = s < p.W ? s : 0;
          push_drow = (int)(((long long)p.my_rank * nel + el) * p.push_C + c_base + cc);
        }
        const int m = m0 + q * 32 + lane;
        if (m < p.M) {
          const int s = m / p.push_rows, cc = m - s * p.push_rows;
          const int el = p.chunk_groups > 0 ? g % p.chunk_groups : g;
          const int nel = p.chunk_groups > 0 ? p.chunk_groups : p.groups;
          const int c_base = p.chunk_groups > 0 ? (g / p.chunk_groups) * p.push_rows : p.push_c0;
          const long long drow = ((long long)p.my_rank * nel + el) * p.push_C + c_base + cc;
          push_row = p.heap_bases[s] + p.push_data_off + (unsigned long long)drow * p.N * 2ull;
        }
      }

      // Output of a staging tile.  With tensor maps: one bulk tensor store per tile, issued by lane 0 and
      // tracked in its bulk group (rows and columns outside the tensor are clipped by the copy engine);
      // the tile may be overwritten once the store has read it (stage_free).  Otherwise: coalesced
      // 16-byte stores, each instruction 4 rows x 128 bytes.
      const uint32_t st0_s = smem_u32(st0);
      const int tile_row = m0 + q * 32;            // first row of this warp's 32-row slice
      auto stage_free = [&]() {
        if (p.tma_out) {
          const long long ts0 = trace != nullptr ? clock64() : 0ll;
          if (lane == 0) bulk_wait_read_all();
          __syncwarp();
          if (trace != nullptr) epi_stage_clk += clock64() - ts0;
        }
      };
      auto tma_out = [&](const CUtensorMap* map, int col, int row, int grp) {
        fence_proxy_async();                       // the warp's staging writes -> the copy engine
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(map, st0_s, col, row, grp);
          bulk_commit();
        }
      };
      auto write_out = [&](__nv_bfloat16* dst, long long row_stride, long long group_stride, int nb) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r = it * 4 + (lane >> 3), c = lane & 7;
          const int m = m0 + q * 32 + r;
          if (m < p.M && nb + c * 8 < p.N) {
            const uint4 val = *reinterpret_cast<const uint4*>(st0 + r * 128 + ((c ^ (r & 7)) << 4));
            *reinterpret_cast<uint4*>(dst + (long long)g * group_stride + (long long)m * row_stride + nb + c * 8) = val;
          }
        }
      };

      // int8 push: the warp's 32 rows x 128 columns leave as uint8 with one (scale, low) pair per row: the
      // accumulator is read twice from TMEM (row range first, then quantisation), the bytes are staged as one
      // 32 x 128-byte tile and written with one bulk tensor store, the pairs with one bulk copy (they are
      // contiguous for the slice: the pairs are laid out [column group][row]).
      bool q8_done = false;
      if constexpr (EPI == kEpiPush && !COPY) {
        if (p.push_q8) {
          q8_done = true;
          const int c0 = half * 128;
          const int nb = n0 + c0;
          if (nb < p.N) {
            uint32_t v[64];
            float lo = INFINITY, hi = -INFINITY;
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2) {
              tmem_ld32(t_row + s2 * 64, v);
              tmem_ld32(t_row + s2 * 64 + 32, v + 32);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 64; ++i) {
                const float f = __uint_as_float(v[i]) + bias_s[c0 + s2 * 64 + i];
                lo = fminf(lo, f); hi = fmaxf(hi, f);
              }
            }
            const float range = hi - lo;
            const float inv = range > 0.f ? 255.f / range : 0.f;
            stage_free();                          // the previous tile's stores have left the staging tile
            float2* pair_s = reinterpret_cast<float2*>(scale_s + ewarp * 256);
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2) {
              tmem_ld32(t_row + s2 * 64, v);
              tmem_ld32(t_row + s2 * 64 + 32, v + 32);
              tmem_ld_wait();
#pragma unroll
              for (int c = 0; c < 4; ++c) {        // 16 columns -> one 16-byte piece of the row
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint32_t b[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const int i = c * 16 + j * 4 + e;
                    const float f = __uint_as_float(v[i]) + bias_s[c0 + s2 * 64 + i];
                    b[e] = (uint32_t)fminf(fmaxf(rintf((f - lo) * inv), 0.f), 255.f);
                  }
                  w[j] = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
                }
                const int piece = s2 * 4 + c;
                *reinterpret_cast<uint4*>(st0 + lane * 128 + ((piece ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            }
            pair_s[lane] = make_float2(range * (1.f / 255.f), lo);
            fence_proxy_async();                   // staging tile and pairs -> the copy engine
            __syncwarp();
            if (lane == 0 && tile_row < p.M) {
              tma_store_3d(&om.m[push_s], st0_s, nb, push_drow, 0);
              const int nrows = min(32, p.M - tile_row);
              uint8_t* pairs = reinterpret_cast<uint8_t*>(p.heap_bases[push_s]) + p.push_scale_off +
                               ((size_t)(nb >> 7) * (size_t)p.push_rows_total + (size_t)push_drow) * 8;
              bulk_store(pairs, smem_u32(pair_s), (uint32_t)nrows * 8u);
              bulk_commit();
            }
            __syncwarp();
          }
        }
      }

      // The accumulator is drained in two 64-column slabs.  The TMEM load of the second slab is issued
      // as soon as the first slab's values have been consumed, so it runs under the first slab's stores.
      // (The activation-backward epilogue also holds the saved derivatives in registers and issues each
      // load at the top of its slab instead.)
      constexpr bool kEarlyLd = EPI != kEpiDAct;
      uint32_t v[64];
      if (!q8_done && kEarlyLd && n0 + half * 128 < p.N) {
        tmem_ld32(t_row, v);
        tmem_ld32(t_row + 32, v + 32);
      }
#pragma unroll
      for (int s2 = 0; s2 < 2; ++s2) {
        const int c0 = half * 128 + s2 * 64;       // first accumulator column of this slab
        const int nb = n0 + c0;                    // first global column
        if (nb >= p.N || q8_done) break;
        if constexpr (!kEarlyLd) {
          tmem_ld32(t_row + s2 * 64, v);
          tmem_ld32(t_row + s2 * 64 + 32, v + 32);
        }
        stage_free();                              // the previous slab's store has left the staging tile

        uint4 dact[8];
        if constexpr (EPI == kEpiDAct) {
          // transpose the fetched slab through the staging tile into one row per thread
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + (lane >> 3), c = lane & 7;
            *reinterpret_cast<uint4*>(st0 + r * 128 + ((c ^ (r & 7)) << 4)) = araw[it];
          }
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 8; ++c)
            dact[c] = *reinterpret_cast<const uint4*>(st0 + lane * 128 + ((c ^ (lane & 7)) << 4));
          __syncwarp();
          if (s2 == 0 && nb + 64 < p.N) load_aux_slab(nb + 64);     // prefetch the second slab
        }
        tmem_ld_wait();

        uint4 opk[8];
        if constexpr (EPI == kEpiBiasAct) {
          // derivative goes through the staging tile first; the activation waits in registers
          uint8_t* st_row = st0 + lane * 128;
          switch (p.activation) {
            case kActRelu: slab_bias_act<kActRelu>(v, bias_s + c0, st_row, lane, opk); break;
            case kActGelu: slab_bias_act<kActGelu>(v, bias_s + c0, st_row, lane, opk); break;
            case kActSilu: slab_bias_act<kActSilu>(v, bias_s + c0, st_row, lane, opk); break;
            default: slab_bias_act<kActIdentity>(v, bias_s + c0, st_row, lane, opk); break;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 b0 = *reinterpret_cast<const float4*>(bias_s + c0 + c * 8);
            const float4 b1 = *reinterpret_cast<const float4*>(bias_s + c0 + c * 8 + 4);
            const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[c * 8 + i]) + bb[i];
            if constexpr (EPI == kEpiDAct) {
              const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&dact[c]);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 df = __bfloat1622float2(ph[i]);
                f[2 * i] *= df.x;
                f[2 * i + 1] *= df.y;
              }
            }
            opk[c] = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
          }
        }
        // v is consumed: fetch the next slab while this one is written out
        if (kEarlyLd && EPI != kEpiBiasAct && s2 == 0 && nb + 64 < p.N) {
          tmem_ld32(t_row + 64, v);
          tmem_ld32(t_row + 96, v + 32);
        }
        if constexpr (EPI == kEpiBiasAct) {
          __syncwarp();
          if (p.aux != nullptr) {
            if (p.tma_out) {
              if (tile_row < p.M) tma_out(&om.m[1], nb, tile_row, g);
              stage_free();
            } else {
              write_out(p.aux, p.aux_row_stride, p.aux_group_stride, nb);
            }
          }
          __syncwarp();
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(st0 + lane * 128 + ((c ^ (lane & 7)) << 4)) = opk[c];
        __syncwarp();
        if (EPI == kEpiBiasAct && s2 == 0 && nb + 64 < p.N) {     // both outputs are staged: registers are free
          tmem_ld32(t_row + 64, v);
          tmem_ld32(t_row + 96, v + 32);
        }

        if constexpr (EPI == kEpiPush) {
          if (p.tma_out) {
            // the 32 rows of the slice belong to one source rank and are contiguous in its combine buffer
            if (tile_row < p.M) tma_out(&om.m[push_s], nb, push_drow, 0);
          } else {
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int r = it * 4 + (lane >> 3), c = lane & 7;
              // destination row addresses were computed once per tile, one row per lane
              const unsigned long long rp = __shfl_sync(0xffffffffu, push_row, r);
              if (rp != 0ull && nb + c * 8 < p.N) {
                const uint4 val = *reinterpret_cast<const uint4*>(st0 + r * 128 + ((c ^ (r & 7)) << 4));
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(rp) + nb + c * 8) = val;
              }
            }
          }
        } else {
          if (p.tma_out) {
            if (tile_row < p.M) tma_out(&om.m[0], nb, tile_row, g);
          } else {
            write_out(p.D, p.d_row_stride, p.d_group_stride, nb);
          }
        }
        __syncwarp();
      }

      // accumulator drained: hand the TMEM stage back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CG == 1) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));
        else                   mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->acc_empty[acc]), 0));
      }
      if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }

      if constexpr (EPI == kEpiPush) {
        if (p.tma_out && lane == 0) bulk_wait_all();   // my bulk stores have been performed
        epi_bar_sync();                            // every row of the tile has been stored
        if (etid == 0) {
          // Bulk stores have completed, so the flag update needs no release; rows written with ordinary stores
          // are published by a fence + release.
          if (!p.tma_out) __threadfence_system();
          const int last_row = min(m0 + BM, p.M) - 1;
          const int s_lo = m0 / p.push_rows, s_hi = last_row / p.push_rows;
          for (int s = s_lo; s <= s_hi; ++s) {
            unsigned long long* flags = reinterpret_cast<unsigned long long*>(
                reinterpret_cast<uint8_t*>(p.heap_bases[s]) + p.push_flag_off);
            const int chunk = p.chunk_groups > 0 ? g / p.chunk_groups : p.push_chunk;
            if (p.tma_out) red_relaxed_sys_add(flags + (long long)chunk * p.W + p.my_rank, 1ull);
            else           red_release_sys_add(flags + (long long)chunk * p.W + p.my_rank, 1ull);
          }
        }
      }
    }
    if (p.tma_out && lane == 0) bulk_wait_all();   // no bulk store of mine is in flight at teardown
    if (trace != nullptr && ewarp == 0 && lane == 0) {
      trace[6] = (unsigned long long)epi_acc_clk;
      trace[7] = ((unsigned long long)(clock64() - epi_t0) << 32) | (unsigned long long)(epi_stage_clk & 0xffffffffll);
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();       // nobody leaves while its partner may still touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<CG>(tmem_base, kTmemCols);
  }
  if (trace != nullptr && threadIdx.x == 0) trace[4] = global_timer_ns();
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  });
  return fn;
}

// Encoded tensor maps are cached: a training step encodes the same handful of (address, shape) pairs
// over and over, and an encode costs microseconds of host time.
struct MapKey {
  const void* ptr; unsigned long long d[4]; unsigned long long st[3]; unsigned box[4]; int rank; int dtype;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapCache {
  static constexpr int kSlots = 128;
  MapKey key[kSlots]; CUtensorMap map[kSlots]; int used = 0, next = 0;
  std::mutex mu;
};
MapCache& map_cache() { static MapCache c; return c; }

bool encode_cached(CUtensorMap* out, int rank, const void* ptr, const cuuint64_t* dims, const cuuint64_t* strides,
                   const cuuint32_t* box, CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16) {
  EncodeFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  MapKey k;
  std::memset(&k, 0, sizeof(k));
  k.ptr = ptr; k.rank = rank; k.dtype = (int)dtype;
  for (int i = 0; i < rank; ++i) { k.d[i] = dims[i]; k.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) k.st[i] = strides[i];
  MapCache& c = map_cache();
  std::lock_guard<std::mutex> lock(c.mu);
  for (int i = 0; i < c.used; ++i)
    if (c.key[i] == k) { *out = c.map[i]; return true; }
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, dtype, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  const int slot = c.used < MapCache::kSlots ? c.used++ : (c.next = (c.next + 1) % MapCache::kSlots);
  c.key[slot] = k; c.map[slot] = *out;
  return true;
}

// 3-D output map over (cols, rows, groups) with a (64, 32, 1) box: one epilogue warp's staging tile.
bool make_out_map(CUtensorMap* map, const void* ptr, long long cols, long long rows, long long groups,
                  long long row_stride, long long group_stride) {
  if ((reinterpret_cast<uintptr_t>(ptr) % 16) || (row_stride % 8) || (groups > 1 && (group_stride % 8))) return false;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)(groups > 0 ? groups : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2,
                           (cuuint64_t)(groups > 1 ? group_stride : rows * row_stride) * 2};
  cuuint32_t box[3] = {64, 32, 1};
  return encode_cached(map, 3, ptr, dims, strides, box);
}

// uint8 output map over (bytes per row, rows, 1) with a (128, 32, 1) box: one epilogue warp's int8 staging tile.
bool make_out_map_u8(CUtensorMap* map, const void* ptr, long long cols, long long rows) {
  if ((reinterpret_cast<uintptr_t>(ptr) % 16) || (cols % 16)) return false;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, 1};
  cuuint64_t strides[2] = {(cuuint64_t)cols, (cuuint64_t)(rows * cols)};
  cuuint32_t box[3] = {128, 32, 1};
  return encode_cached(map, 3, ptr, dims, strides, box, CU_TENSOR_MAP_DATA_TYPE_UINT8);
}

// 4-D map over (cols, rows, groups, chunks) with a (64, box_rows, 1, 1) box and 128-byte swizzle.
bool make_map(CUtensorMap* map, const GemmOperand& op, int groups, int box_rows) {
  if (get_encode_fn() == nullptr) return false;
  const cuuint64_t chunks = op.chunks > 0 ? op.chunks : 1;
  cuuint64_t dims[4] = {(cuuint64_t)op.cols, (cuuint64_t)op.rows, (cuuint64_t)groups, chunks};
  long long gs = op.group_stride > 0 ? op.group_stride : op.rows * op.row_stride;
  long long cs = op.chunk_stride > 0 ? op.chunk_stride : gs * groups;
  cuuint64_t strides[3] = {(cuuint64_t)op.row_stride * 2, (cuuint64_t)gs * 2, (cuuint64_t)cs * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  return encode_cached(map, 4, op.ptr, dims, strides, box);
}

template <int CG, bool A_MN, bool B_MN, int EPI, bool COPY>
cudaError_t launch_epi(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& om, const KernelParams& kp, int ctas,
                       cudaStream_t stream) {
  auto kern = grouped_gemm_kernel<CG, A_MN, B_MN, EPI, COPY>;
  constexpr int smem = (int)Geo<CG, COPY>::kSmemTotal;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)ctas, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = CG > 1 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, ta, tb, om, kp);
}

template <int CG, bool A_MN, bool B_MN>
cudaError_t launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& om, const KernelParams& kp,
                           int ctas, cudaStream_t stream) {
  // The variant with a dispatch send (copy and de-quantiser roles, one ring stage less) exists for the launches
  // that consume a dispatched A operand: K-major A with the bias + activation or activation-backward epilogue.
  static int force_copy_variant = -1;              // PLANMOE_GEMM_COPY_VARIANT=1: measure the variant's ring depth alone
  if (force_copy_variant < 0) {
    const char* e = getenv("PLANMOE_GEMM_COPY_VARIANT");
    force_copy_variant = (e != nullptr && e[0] == '1') ? 1 : 0;
  }
  const bool copy = kp.copy.ctas > 0 || kp.dequant.q != nullptr ||
                    (force_copy_variant && !A_MN && (kp.epilogue == kEpiBiasAct || kp.epilogue == kEpiDAct));
  if (copy) {
    if constexpr (!A_MN) {
      if (kp.epilogue == kEpiBiasAct) return launch_epi<CG, A_MN, B_MN, kEpiBiasAct, true>(ta, tb, om, kp, ctas, stream);
      if (kp.epilogue == kEpiDAct) return launch_epi<CG, A_MN, B_MN, kEpiDAct, true>(ta, tb, om, kp, ctas, stream);
    }
    return cudaErrorInvalidValue;
  }
  switch (kp.epilogue) {
    case kEpiStore: return launch_epi<CG, A_MN, B_MN, kEpiStore, false>(ta, tb, om, kp, ctas, stream);
    case kEpiBiasAct: return launch_epi<CG, A_MN, B_MN, kEpiBiasAct, false>(ta, tb, om, kp, ctas, stream);
    case kEpiDAct: return launch_epi<CG, A_MN, B_MN, kEpiDAct, false>(ta, tb, om, kp, ctas, stream);
    case kEpiPush: return launch_epi<CG, A_MN, B_MN, kEpiPush, false>(ta, tb, om, kp, ctas, stream);
    default: return cudaErrorInvalidValue;
  }
}

template <int CG>
cudaError_t launch_layout(const GemmArgs& a, const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& om,
                          const KernelParams& kp, int ctas, cudaStream_t stream) {
  if (!a.A.mn_major && a.B.mn_major) return launch_variant<CG, false, true>(ta, tb, om, kp, ctas, stream);
  if (!a.A.mn_major && !a.B.mn_major) return launch_variant<CG, false, false>(ta, tb, om, kp, ctas, stream);
  if (a.A.mn_major && a.B.mn_major) return launch_variant<CG, true, true>(ta, tb, om, kp, ctas, stream);
  return launch_variant<CG, true, false>(ta, tb, om, kp, ctas, stream);
}

// Largest number of two-CTA clusters of this kernel that can be resident at once.  A persistent grid
// must not exceed it: CTAs that wait on flags fed by the copy warps of *every* CTA of the grid would
// otherwise wait for CTAs that cannot start before they finish.
int max_pair_units() {
  static int units = 0;
  if (units == 0) {
    auto kern = grouped_gemm_kernel<2, false, true, kEpiBiasAct, true>;
    int n = 0;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = Geo<2, true>::kSmemTotal;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Geo<2, true>::kSmemTotal) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 0;
    }
    units = n > 0 ? n : -1;
  }
  return units;
}

int sm_count_cached() {
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  return sm_count;
}

}  // namespace

// CTA-group size of a launch: 2 (a two-CTA cluster per 256 x 256 tile) unless the problem has at most
// 128 rows per group, where the second CTA of a pair would only compute padding, or the caller or the
// environment variable PLANMOE_GEMM_CTA_GROUP asks for 1.
int gemm_cta_group(int M, int requested) {
  static int env = -1;
  if (env < 0) {
    const char* e = getenv("PLANMOE_GEMM_CTA_GROUP");
    env = (e != nullptr && (e[0] == '1' || e[0] == '2')) ? e[0] - '0' : 0;
  }
  if (requested == 1 || requested == 2) return requested;
  if (env != 0) return env;
  return M > BM ? 2 : 1;
}

int gemm_grid_ctas(int groups, int M, int N, int max_ctas, int cta_group) {
  const int cg = gemm_cta_group(M, cta_group);
  const long long tiles = (long long)groups * ((M + BM * cg - 1) / (BM * cg)) * ((N + BN - 1) / BN);
  long long units = (max_ctas > 0 ? max_ctas : sm_count_cached()) / cg;
  if (cg == 2) {
    const int cap = max_pair_units();
    if (cap > 0 && units > cap) units = cap;
  }
  if (units < 1) units = 1;
  if (units > tiles) units = tiles;
  return (int)(units * cg);
}

int gemm_push_arrivals(int groups, int M, int N, int push_rows, int s) {
  const int nt = (N + BN - 1) / BN;
  const int lo = s * push_rows, hi = (s + 1) * push_rows - 1;
  if (lo >= M) return 0;
  const int mt_lo = lo / BM, mt_hi = (hi < M ? hi : M - 1) / BM;
  return groups * nt * (mt_hi - mt_lo + 1);
}

cudaError_t launch_grouped_gemm(const GemmArgs& a, cudaStream_t stream) {
  if (a.groups <= 0 || a.M <= 0 || a.N <= 0 || a.K <= 0) return cudaSuccess;
  // 16-byte rules of TMA and of the vector epilogue
  if ((a.N % 8) || (a.A.cols % 8) || (a.B.cols % 8) || (a.A.row_stride % 8) || (a.B.row_stride % 8) ||
      (reinterpret_cast<uintptr_t>(a.A.ptr) % 16) || (reinterpret_cast<uintptr_t>(a.B.ptr) % 16))
    return cudaErrorInvalidValue;
  if (a.A.chunks != a.B.chunks) return cudaErrorInvalidValue;
  const int cg = gemm_cta_group(a.M, a.cta_group);

  CUtensorMap ta, tb;
  if (!make_map(&ta, a.A, a.groups, a.A.mn_major ? BK : BM)) return cudaErrorInvalidValue;
  const int b_groups = a.chunk_groups > 0 ? a.chunk_groups : a.groups;
  if (!make_map(&tb, a.B, b_groups, a.B.mn_major ? BK : BN / cg)) return cudaErrorInvalidValue;

  KernelParams kp{};
  kp.groups = a.groups; kp.M = a.M; kp.N = a.N; kp.K = a.K;
  kp.a_chunks = a.A.chunks > 0 ? a.A.chunks : 1;
  kp.epilogue = a.epilogue; kp.activation = a.activation;
  kp.D = reinterpret_cast<__nv_bfloat16*>(a.D); kp.d_row_stride = a.d_row_stride; kp.d_group_stride = a.d_group_stride;
  kp.aux = reinterpret_cast<__nv_bfloat16*>(a.aux); kp.aux_row_stride = a.aux_row_stride; kp.aux_group_stride = a.aux_group_stride;
  kp.bias = reinterpret_cast<const __nv_bfloat16*>(a.bias); kp.bias_group_stride = a.bias_group_stride;
  kp.gate_flags = a.gate_flags; kp.gate_rows = a.gate_rows > 0 ? a.gate_rows : a.M; kp.gate_want = a.gate_want;
  kp.gate_want_ptr = a.gate_want_ptr;
  kp.gate_mode = a.gate_mode; kp.gate_nblk = a.gate_nblk;
  kp.perm_w = 0; kp.perm_q = 0; kp.perm_local = 0;
  kp.send_local_first = a.perm_local_first ? 1 : 0;
  if (a.perm_w > 1 && a.perm_seg_rows > BM * cg && a.perm_seg_rows % (BM * cg) == 0 &&
      (long long)a.perm_w * a.perm_seg_rows == a.M) {
    kp.perm_w = a.perm_w; kp.perm_q = a.perm_seg_rows / (BM * cg);   // every segment is perm_q > 1 whole tiles
    kp.perm_local = a.perm_local_first ? 1 : 0;
  }
  kp.a_ptr = a.A.ptr; kp.a_row_stride = a.A.row_stride;
  kp.a_group_stride = a.A.group_stride > 0 ? a.A.group_stride : a.A.rows * a.A.row_stride;
  kp.heap_bases = a.heap_bases; kp.push_data_off = a.push_data_off; kp.push_flag_off = a.push_flag_off;
  kp.push_rows = a.push_rows > 0 ? a.push_rows : a.M; kp.push_C = a.push_C; kp.push_c0 = a.push_c0;
  kp.push_chunk = a.push_chunk; kp.W = a.W; kp.my_rank = a.my_rank;
  kp.push_q8 = (a.epilogue == kEpiPush && a.push_q8) ? 1 : 0; kp.push_scale_off = a.push_scale_off;
  kp.push_rows_total = (long long)a.W * (a.chunk_groups > 0 ? a.chunk_groups : a.groups) * a.push_C;
  kp.chunk_groups = a.chunk_groups;
  kp.budget_ns = a.budget_ns ? a.budget_ns : 20000000000ull;
  kp.status = a.status;
  kp.trace = a.trace;
  {
    static int dbg = -1;
    if (dbg < 0) { const char* e = getenv("PLANMOE_COPY_DBG"); dbg = e != nullptr ? atoi(e) : 0; }
    kp.copy_dbg = dbg;
  }
  kp.copy = a.copy;
  if (kp.copy.ctas > 0) {
    if (kp.copy.x == nullptr || kp.copy.slot_map == nullptr || a.heap_bases == nullptr ||
        kp.copy.chunks <= 0 || (kp.copy.C % kp.copy.chunks) || (reinterpret_cast<uintptr_t>(kp.copy.x) % 16) ||
        kp.copy.row_bytes <= 0 || (size_t)kp.copy.row_bytes > kCopyMaxSlot || (kp.copy.row_bytes % 16) ||
        kp.copy.nblk <= 0)
      return cudaErrorInvalidValue;
  } else {
    kp.copy.ctas = 0;
  }
  kp.dequant = a.dequant;
  if (kp.dequant.q != nullptr) {
    if (a.A.mn_major || a.gate_mode != 1 || kp.dequant.arrival == nullptr || kp.dequant.ready == nullptr ||
        kp.dequant.M != a.K || (a.K % 16) || (a.A.chunks > 1))
      return cudaErrorInvalidValue;
  }

  const int ctas = gemm_grid_ctas(a.groups, a.M, a.N, a.max_ctas, cg);
  if (kp.copy.ctas > 0) kp.copy.ctas = ctas;

  // ---- output tensor maps for the bulk-store epilogue ------------------------------------------
  // Used whenever every 32-row slice of a tile maps to 32 consecutive destination rows: always for
  // plain outputs; for the push epilogue when the rows per source rank are a multiple of 32 and the
  // caller supplied the peers' base addresses.  PLANMOE_GEMM_TMA_STORE=0 keeps the 16-byte store path.
  static int tma_env = -1;
  if (tma_env < 0) {
    const char* e = getenv("PLANMOE_GEMM_TMA_STORE");
    tma_env = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  static OutMaps om;                       // filled per launch; copied into the kernel's parameters at launch
  static std::mutex om_mu;
  std::lock_guard<std::mutex> om_lock(om_mu);
  kp.tma_out = 0;
  if (tma_env) {
    bool okm = true;
    if (a.epilogue == kEpiPush) {
      okm = a.heap_bases_host != nullptr && a.W >= 1 && a.W <= 8 && kp.push_rows % 32 == 0 && a.M % 32 == 0;
      const int nel = a.chunk_groups > 0 ? a.chunk_groups : a.groups;
      for (int r = 0; okm && r < a.W; ++r) {
        const void* base = reinterpret_cast<const void*>(a.heap_bases_host[r] + a.push_data_off);
        okm = kp.push_q8 ? make_out_map_u8(&om.m[r], base, a.N, (long long)a.W * nel * a.push_C)
                         : make_out_map(&om.m[r], base, a.N, (long long)a.W * nel * a.push_C, 1, a.N, 0);
      }
      if (kp.push_q8 && (a.N % 128)) okm = false;
    } else {
      okm = make_out_map(&om.m[0], a.D, a.N, a.M, a.groups, a.d_row_stride, a.d_group_stride);
      if (okm && a.epilogue == kEpiBiasAct && a.aux != nullptr)
        okm = make_out_map(&om.m[1], a.aux, a.N, a.M, a.groups, a.aux_row_stride, a.aux_group_stride);
    }
    kp.tma_out = okm ? 1 : 0;
  }
  if (kp.push_q8 && !kp.tma_out) return cudaErrorInvalidValue;   // the int8 push exists in the bulk-store form only

  if (cg == 2) return launch_layout<2>(a, ta, tb, om, kp, ctas, stream);
  return launch_layout<1>(a, ta, tb, om, kp, ctas, stream);
}

// ---------------------------------------------------------------------------------------------
// Column sums (bias gradients): fp32 [groups / fold][N] = sum over rows (and over `fold` leading
// group blocks, the pipeline chunks) of bf16 [groups][rows][N]; up to two tensors per launch.
// Two stages, deterministic, each one launch for all tensors.  Stage 1: a CTA of 8 row lanes x 32 column threads
// reduces a slab of 128 rows x 256 columns with 16-byte loads (8 columns per thread), combines the row lanes
// through shared memory and writes one fp32 partial row.  Stage 2 adds the partials in slab order.  (A
// single-launch form in which the last CTA to arrive finished the sum measured slower: the fence and the
// atomic that every CTA needs before it may leave cost more than the second launch.)
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int kColsumSlab = 128;
constexpr int kColsumCols = 256;

struct ColsumJobs {
  ColsumJob j[2];
  int z0[3];                                       // job i owns blockIdx.z in [z0[i], z0[i + 1])
  int n;
};

__global__ void __launch_bounds__(256)
colsum_kernel(const ColsumJobs jobs) {
  __shared__ float red[8][kColsumCols + 8];
  const int ji = (jobs.n > 1 && (int)blockIdx.z >= jobs.z0[1]) ? 1 : 0;
  const ColsumJob& J = jobs.j[ji];
  const int g = (int)blockIdx.z - jobs.z0[ji];
  const int slab = blockIdx.y, cb = blockIdx.x;
  const int slabs = (int)((J.rows + kColsumSlab - 1) / kColsumSlab);
  const int colblocks = (J.N + kColsumCols - 1) / kColsumCols;
  if (slab >= slabs || cb >= colblocks) return;    // the grid is sized for the larger job
  const int ct = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int col0 = cb * kColsumCols;
  const int col = col0 + ct * 8;
  const int N = J.N;
  const long long r0 = (long long)slab * kColsumSlab;
  const long long r1 = r0 + kColsumSlab < J.rows ? r0 + kColsumSlab : J.rows;
  float a[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = 0.f;
  if (col < N) {
    const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(J.x) + (long long)g * J.group_stride + col;
#pragma unroll 4
    for (long long r = r0 + rl; r < r1; r += 8) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(base + r * J.row_stride));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        a[2 * i] += f.x; a[2 * i + 1] += f.y;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rl][ct * 8 + i] = a[i];
  __syncthreads();
  const int c = threadIdx.x;
  if (col0 + c < N) {
    float acc = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) acc += red[l][c];
    J.partial[((long long)g * slabs + slab) * N + col0 + c] = acc;
  }
}

// Stage 2 for every job of the launch: 32 columns x 8 slab lanes per CTA; lane l adds partials l, l + 8, ...
// (independent loads in flight), the eight lane sums are then added in lane order, so the result does not
// depend on timing.
__global__ void __launch_bounds__(256)
colsum_final_kernel(const ColsumJobs jobs) {
  __shared__ float red[8][33];
  const int ji = (jobs.n > 1 && (int)blockIdx.y >= jobs.z0[1]) ? 1 : 0;
  const ColsumJob& J = jobs.j[ji];
  const int e = (int)blockIdx.y - jobs.z0[ji];
  const int N = J.N;
  const int ct = threadIdx.x & 31, sl = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + ct;
  if ((int)blockIdx.x * 32 >= N) return;           // the grid is sized for the wider job
  const int slabs = (int)((J.rows + kColsumSlab - 1) / kColsumSlab);
  const int out_groups = J.groups / J.fold;
  float acc = 0.f;
  if (col < N) {
    const int total = J.fold * slabs;
#pragma unroll 4
    for (int i = sl; i < total; i += 8) {
      const int j = i / slabs, s = i - j * slabs;
      acc += J.partial[((long long)(j * out_groups + e) * slabs + s) * N + col];
    }
  }
  red[sl][ct] = acc;
  __syncthreads();
  if (sl == 0 && col < N) {
    float r = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) r += red[l][ct];
    J.out[(long long)e * N + col] = r;
    if (J.out_bf16 != nullptr) reinterpret_cast<__nv_bfloat16*>(J.out_bf16)[(long long)e * N + col] = __float2bfloat16_rn(r);
  }
}
}  // namespace

int colsum_slabs(long long rows) { return (int)((rows + kColsumSlab - 1) / kColsumSlab); }
int colsum_colblocks(int N) { return (N + kColsumCols - 1) / kColsumCols; }

// Two launches (partial sums, then their sum in slab order) for one or two jobs.
void launch_colsum_jobs(const ColsumJob* jobs, int n, cudaStream_t stream) {
  ColsumJobs js{}, jf{};
  js.n = jf.n = n;
  int z = 0, zo = 0, max_slabs = 1, max_cb = 1, max_n = 0;
  for (int i = 0; i < n; ++i) {
    js.j[i] = jobs[i];
    if (js.j[i].fold < 1) js.j[i].fold = 1;
    jf.j[i] = js.j[i];
    js.z0[i] = z;
    jf.z0[i] = zo;
    z += jobs[i].groups;
    zo += jobs[i].groups / js.j[i].fold;
    max_slabs = std::max(max_slabs, colsum_slabs(jobs[i].rows));
    max_cb = std::max(max_cb, colsum_colblocks(jobs[i].N));
    max_n = std::max(max_n, jobs[i].N);
  }
  js.z0[n] = z;
  jf.z0[n] = zo;
  colsum_kernel<<<dim3(max_cb, max_slabs, z), 256, 0, stream>>>(js);
  colsum_final_kernel<<<dim3((max_n + 31) / 32, zo), 256, 0, stream>>>(jf);
}

// `out` must have room for (groups / fold) * N floats, then groups * colsum_slabs(rows) * N floats of scratch,
// then (groups / fold) * colsum_colblocks(N) unused words.  N must be a multiple of 8 and rows of x 16-byte
// aligned.  groups = fold * (groups / fold): group j * (groups / fold) + e is summed into output row e.
// `out_bf16` (optional) receives the same sums rounded to bf16.
void launch_colsum_bf16(const void* x, float* out, int groups, long long rows, int N, long long row_stride,
                        long long group_stride, int fold, void* out_bf16, cudaStream_t stream) {
  if (fold < 1) fold = 1;
  ColsumJob j{};
  j.x = x; j.out = out; j.out_bf16 = out_bf16;
  j.partial = out + (long long)(groups / fold) * N;
  j.counters = reinterpret_cast<unsigned*>(j.partial + (long long)groups * colsum_slabs(rows) * N);
  j.rows = rows; j.row_stride = row_stride; j.group_stride = group_stride;
  j.N = N; j.groups = groups; j.fold = fold;
  launch_colsum_jobs(&j, 1, stream);
}

}  // namespace planmoe
