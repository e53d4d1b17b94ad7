// Grouped bf16 GEMM for the expert FFNs on 5th-generation tensor cores (sm_100a).
//
//   D[g] (M x N) = A[g] (M x K) . B[g] (K x N)          g = 0 .. groups-1, fp32 accumulate
//
// Hand-written tcgen05 pipeline, one persistent CTA per SM, 352 threads in four roles.  By default two
// CTAs form a cluster and compute one 256 x 256 tile with tcgen05.mma.cta_group::2 (each CTA stages
// its own 128 rows of A and 128 of the 256 B columns; the even CTA issues the MMAs for both);
// problems with at most 128 rows per group run the one-CTA variant (128 x 256 tiles).
//   warp 0      TMA producer: cp.async.bulk.tensor (4-D maps, 128-byte swizzle) into a 5-stage
//               shared-memory ring (3-stage in the one-CTA variant), completion on the mbarrier of
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
//               optional gate scaling in shared memory, cp.async.bulk shared -> peer global; seven
//               4 KiB slots are in flight per CTA, one per lane.  Chunks leave in order; after a
//               chunk its stores are awaited and the (chunk, rank) flags on every destination get
//               a release-add.  The producers of the same launch on every rank are the flag-gated
//               consumers, so the all-to-all and the GEMM that follows it are one kernel and
//               overlap tile by tile; the copy never waits on another CTA or rank, so no circular
//               wait can form.
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
constexpr int kThreads = 352;                     // TMA, MMA, 8 epilogue warps, copy warp
constexpr uint32_t kCopySlot = 4096;              // bytes per bulk-copy slot (one bf16 row of 2048, or a piece of a longer row)
constexpr int kCopyLanes = 7;                     // data slots = lanes of the copy warp that drive the bulk-copy engine
constexpr uint32_t kSmemCopy = (kCopyLanes + 1) * kCopySlot;   // + one slot of zeros for empty expert slots
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
template <int CG> struct Geo {
  static constexpr int kBRows = BN / CG;                        // B columns staged per CTA
  static constexpr uint32_t kBBytes = kBRows * BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = CG == 1 ? 3 : 5;
  static constexpr uint32_t kSmemRing = kStages * kStageBytes;
  // ring | epilogue staging | bulk-copy slots of the dispatch send | bias | barriers.
  // No alignment slack: the dynamic shared array is declared 1024-byte aligned.
  static constexpr uint32_t kSmemTotal = kSmemRing + kSmemStaging + kSmemCopy + kSmemBias + kSmemBars;
};
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
  const unsigned long long* heap_bases; unsigned long long push_data_off, push_flag_off;
  int push_rows, push_C, push_c0, push_chunk, W, my_rank;
  // chunk_groups > 0: groups are [chunk][expert] with chunk_groups experts; weights / bias are indexed
  // by the expert, flags and push offsets by the chunk.
  int chunk_groups;
  unsigned long long budget_ns; int* status;
  GemmArgs::CopyJob copy;        // copy.ctas > 0: the copy warp of every CTA runs the dispatch send
  int tma_out;                   // epilogue writes its staging tiles with bulk tensor stores (OutMaps valid)
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
  uint64_t copy_full[kCopyLanes];   // a row has landed in bulk-copy slot i
  uint32_t tmem_base;
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
// Copy role (warp 10 of every CTA): the dispatch send, driven by the bulk-copy engine.
//
// A unit is one token row (or a 4 KiB piece of a longer row) for one destination.  The CTA owns the
// rows blockIdx.x, blockIdx.x + gridDim.x, ... of every (chunk, destination).  Units are handled in
// batches of seven, one per lane: the lane looks up the slot map, starts a bulk load of the token row
// into its shared-memory slot (or, for an empty expert slot, a bulk store of the zero slot), waits
// (bounded) for the row, the warp scales gate-weighted rows in shared memory, and the lane starts the
// bulk store into the receive buffer [chunk][E_local][W_src][C/chunks][M] of the destination rank.
// After a chunk every lane waits for its stores to complete, then the warp fences and adds one
// arrival to the (chunk, my_rank) flag of every destination: one arrival per CTA of the grid.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void copy_role(const KernelParams& p, uint8_t* cring, Ctl* ctl) {
  const GemmArgs::CopyJob& c = p.copy;
  const int lane = threadIdx.x & 31;
  const int Cc = c.C / c.chunks;
  const int rows = c.E_local * Cc;                               // rows per (chunk, destination)
  const uint32_t row_bytes = (uint32_t)c.M * 2u;
  const int pieces = (int)((row_bytes + kCopySlot - 1) / kCopySlot);
  const int my_rows = ((int)blockIdx.x < rows) ? (rows - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int units = p.W * my_rows * pieces;                      // per chunk, for this CTA
  const uint8_t* x = reinterpret_cast<const uint8_t*>(c.x);
  uint8_t* my_slot = cring + lane * kCopySlot;
  const uint32_t my_slot_s = smem_u32(my_slot);
  const uint32_t zero_s = smem_u32(cring + kCopyLanes * kCopySlot);
  const uint32_t my_bar = smem_u32(&ctl->copy_full[lane < kCopyLanes ? lane : 0]);
  uint32_t phase = 0;                                            // parity of my slot's barrier
  bool ok = true;

  for (uint32_t i = lane; i < kCopySlot / 16; i += 32)
    reinterpret_cast<uint4*>(cring + kCopyLanes * kCopySlot)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async();                                           // zeros visible to the bulk-copy engine
  __syncwarp();

  for (int j = 0; j < c.chunks && ok; ++j) {
    for (int base = 0; base < units; base += kCopyLanes) {
      const int u = base + lane;
      const bool mine = lane < kCopyLanes && u < units;
      bool loaded = false;
      float gw = 1.f;
      uint8_t* dst = nullptr;
      uint32_t bytes = 0;
      if (mine) {
        const int piece = u % pieces;
        const int k = (u / pieces) % my_rows;
        const int rr = u / (pieces * my_rows);
        // destinations start at my right-hand neighbour, staggered by CTA so that all links are busy
        const int r = (p.my_rank + 1 + rr + (int)blockIdx.x) % p.W;
        const int row = (int)blockIdx.x + k * (int)gridDim.x;
        const int el = row / Cc, cc = row - el * Cc;
        const int owner = c.slot_map[(size_t)(r * c.E_local + el) * c.C + j * Cc + cc];
        bytes = min(kCopySlot, row_bytes - (uint32_t)piece * kCopySlot);
        dst = reinterpret_cast<uint8_t*>(p.heap_bases[r]) + c.data_off +
              ((((size_t)j * c.E_local + el) * p.W + p.my_rank) * Cc + cc) * row_bytes + (size_t)piece * kCopySlot;
        bulk_wait_read_all();                                    // my previous store has left the slot
        if (owner >= 0) {
          const int t = owner / c.K, kk = owner - t * c.K;
          if (c.gates != nullptr) gw = c.gates[(size_t)kk * c.S + t];
          mbar_expect_tx(my_bar, bytes);
          bulk_load(my_slot_s, x + (size_t)t * row_bytes + (size_t)piece * kCopySlot, bytes, my_bar);
          loaded = true;
        } else {
          bulk_store(dst, zero_s, bytes);                        // empty expert slot: a row of zeros
          bulk_commit();
        }
      }
      if (loaded) {
        ok = mbar_wait(my_bar, phase, ctl, p.budget_ns, p.status, 3, lane);
        phase ^= 1u;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      // gate-weighted rows (pre-score dispatch, gate-weighted dY): scale in shared memory, the whole
      // warp on one slot at a time
      unsigned scaled = __ballot_sync(0xffffffffu, loaded && gw != 1.f);
      while (scaled) {
        const int sl = __ffs(scaled) - 1;
        scaled &= scaled - 1;
        const float g = __shfl_sync(0xffffffffu, gw, sl);
        const uint32_t nb = __shfl_sync(0xffffffffu, bytes, sl);
        uint4* q = reinterpret_cast<uint4*>(cring + sl * kCopySlot);
        for (uint32_t i = lane; i < nb / 16; i += 32) {
          uint4 v = q[i];
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            h[e] = __floats2bfloat162_rn(f.x * g, f.y * g);
          }
          q[i] = v;
        }
        fence_proxy_async();                                     // my writes -> the bulk store below
      }
      __syncwarp();
      if (loaded) {
        bulk_store(dst, my_slot_s, bytes);
        bulk_commit();
      }
    }
    // chunk j handed to the copy engine everywhere: wait for the stores, then publish it
    bulk_wait_all();
    __syncwarp();
    if (lane == 0) __threadfence_system();
    __syncwarp();
    if (lane < p.W) {
      unsigned long long* flags = reinterpret_cast<unsigned long long*>(
          reinterpret_cast<uint8_t*>(p.heap_bases[lane]) + c.flag_off);
      red_release_sys_add(flags + (size_t)j * p.W + p.my_rank, 1ull);
    }
  }
  bulk_wait_all();                                               // nothing of mine is in flight at teardown
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

template <int CG, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ OutMaps om, const KernelParams p) {
  using G = Geo<CG>;
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
  float* bias_s = reinterpret_cast<float*>(smem + G::kSmemRing + kSmemStaging + kSmemCopy);
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + G::kSmemRing + kSmemStaging + kSmemCopy + kSmemBias);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

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
    for (int i = 0; i < kCopyLanes; ++i) mbar_init(smem_u32(&ctl->copy_full[i]), 1);
    ctl->abort = 0;
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
      const unsigned long long gate_want = p.gate_want_ptr != nullptr ? *p.gate_want_ptr : p.gate_want;
      for (int tile = unit; tile < tiles && ok; tile += nunits) {
        const int nt = tile % nt_count;
        const int mt = (tile / nt_count) % mt_count;
        const int g = tile / (nt_count * mt_count);
        const int m0 = mt * (BM * CG) + cr * BM;                         // my 128 rows of the tile
        const int n0 = nt * BN + cr * G::kBRows;                         // my share of the B columns
        const int gb = p.chunk_groups > 0 ? g % p.chunk_groups : g;      // group of the B operand
        if (p.gate_flags != nullptr && m0 < p.M) {
          const int last_row = min(m0 + BM, p.M) - 1;
          const int s_lo = m0 / p.gate_rows, s_hi = last_row / p.gate_rows;
          for (int s = s_lo; s <= s_hi && ok; ++s)
            ok = wait_flag_ge(p.gate_flags + (p.chunk_groups > 0 ? (g / p.chunk_groups) * p.W : 0) + s, gate_want,
                              p.budget_ns, p.status, s);
          if (!ok) { ctl->abort = 1; break; }
          fence_proxy_async();   // peers' generic-proxy stores -> this thread's async-proxy loads
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
  } else if (warp >= 2 + kEpiWarps) {
    // ------------------------------------------------------------------ dispatch send (copy warp)
    if (p.copy.ctas > 0) copy_role(p, cring, ctl);
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
    for (int tile = unit; tile < tiles && ok; tile += nunits) {
      const int nt = tile % nt_count;
      const int mt = (tile / nt_count) % mt_count;
      const int g = tile / (nt_count * mt_count);
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
      bool got = mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, ctl, p.budget_ns, p.status, 2, acc);
      got = __all_sync(0xffffffffu, got);
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
          if (lane == 0) bulk_wait_read_all();
          __syncwarp();
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

      // The accumulator is drained in two 64-column slabs.  The TMEM load of the second slab is issued
      // as soon as the first slab's values have been consumed, so it runs under the first slab's stores.
      // (The activation-backward epilogue also holds the saved derivatives in registers and issues each
      // load at the top of its slab instead.)
      constexpr bool kEarlyLd = EPI != kEpiDAct;
      uint32_t v[64];
      if (kEarlyLd && n0 + half * 128 < p.N) {
        tmem_ld32(t_row, v);
        tmem_ld32(t_row + 32, v + 32);
      }
#pragma unroll
      for (int s2 = 0; s2 < 2; ++s2) {
        const int c0 = half * 128 + s2 * 64;       // first accumulator column of this slab
        const int nb = n0 + c0;                    // first global column
        if (nb >= p.N) break;
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
          __threadfence_system();
          const int last_row = min(m0 + BM, p.M) - 1;
          const int s_lo = m0 / p.push_rows, s_hi = last_row / p.push_rows;
          for (int s = s_lo; s <= s_hi; ++s) {
            unsigned long long* flags = reinterpret_cast<unsigned long long*>(
                reinterpret_cast<uint8_t*>(p.heap_bases[s]) + p.push_flag_off);
            const int chunk = p.chunk_groups > 0 ? g / p.chunk_groups : p.push_chunk;
            red_release_sys_add(flags + (long long)chunk * p.W + p.my_rank, 1ull);
          }
        }
      }
    }
    if (p.tma_out && lane == 0) bulk_wait_all();   // no bulk store of mine is in flight at teardown
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();       // nobody leaves while its partner may still touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<CG>(tmem_base, kTmemCols);
  }
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
  const void* ptr; unsigned long long d[4]; unsigned long long st[3]; unsigned box[4]; int rank;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapCache {
  static constexpr int kSlots = 128;
  MapKey key[kSlots]; CUtensorMap map[kSlots]; int used = 0, next = 0;
  std::mutex mu;
};
MapCache& map_cache() { static MapCache c; return c; }

bool encode_cached(CUtensorMap* out, int rank, const void* ptr, const cuuint64_t* dims, const cuuint64_t* strides,
                   const cuuint32_t* box) {
  EncodeFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  MapKey k;
  std::memset(&k, 0, sizeof(k));
  k.ptr = ptr; k.rank = rank;
  for (int i = 0; i < rank; ++i) { k.d[i] = dims[i]; k.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) k.st[i] = strides[i];
  MapCache& c = map_cache();
  std::lock_guard<std::mutex> lock(c.mu);
  for (int i = 0; i < c.used; ++i)
    if (c.key[i] == k) { *out = c.map[i]; return true; }
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides, box,
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

template <int CG, bool A_MN, bool B_MN, int EPI>
cudaError_t launch_epi(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& om, const KernelParams& kp, int ctas,
                       cudaStream_t stream) {
  auto kern = grouped_gemm_kernel<CG, A_MN, B_MN, EPI>;
  constexpr int smem = (int)Geo<CG>::kSmemTotal;
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
  switch (kp.epilogue) {
    case kEpiStore: return launch_epi<CG, A_MN, B_MN, kEpiStore>(ta, tb, om, kp, ctas, stream);
    case kEpiBiasAct: return launch_epi<CG, A_MN, B_MN, kEpiBiasAct>(ta, tb, om, kp, ctas, stream);
    case kEpiDAct: return launch_epi<CG, A_MN, B_MN, kEpiDAct>(ta, tb, om, kp, ctas, stream);
    case kEpiPush: return launch_epi<CG, A_MN, B_MN, kEpiPush>(ta, tb, om, kp, ctas, stream);
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
    auto kern = grouped_gemm_kernel<2, false, true, kEpiStore>;
    int n = 0;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = Geo<2>::kSmemTotal;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Geo<2>::kSmemTotal) != cudaSuccess ||
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
  kp.heap_bases = a.heap_bases; kp.push_data_off = a.push_data_off; kp.push_flag_off = a.push_flag_off;
  kp.push_rows = a.push_rows > 0 ? a.push_rows : a.M; kp.push_C = a.push_C; kp.push_c0 = a.push_c0;
  kp.push_chunk = a.push_chunk; kp.W = a.W; kp.my_rank = a.my_rank;
  kp.chunk_groups = a.chunk_groups;
  kp.budget_ns = a.budget_ns ? a.budget_ns : 20000000000ull;
  kp.status = a.status;
  kp.copy = a.copy;
  if (kp.copy.ctas > 0) {
    if (kp.copy.x == nullptr || kp.copy.slot_map == nullptr || a.heap_bases == nullptr || (kp.copy.M % 8) ||
        kp.copy.chunks <= 0 || (kp.copy.C % kp.copy.chunks) || (reinterpret_cast<uintptr_t>(kp.copy.x) % 16))
      return cudaErrorInvalidValue;
  } else {
    kp.copy.ctas = 0;
  }

  const int ctas = gemm_grid_ctas(a.groups, a.M, a.N, a.max_ctas, cg);
  // With a copy job every CTA of the grid adds one arrival per (chunk, destination) flag; the caller
  // computed its expected count from gemm_grid_ctas() and passes it back as copy.ctas.
  if (kp.copy.ctas > 0 && kp.copy.ctas != ctas) return cudaErrorInvalidValue;

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
      for (int r = 0; okm && r < a.W; ++r)
        okm = make_out_map(&om.m[r], reinterpret_cast<const void*>(a.heap_bases_host[r] + a.push_data_off), a.N,
                           (long long)a.W * nel * a.push_C, 1, a.N, 0);
    } else {
      okm = make_out_map(&om.m[0], a.D, a.N, a.M, a.groups, a.d_row_stride, a.d_group_stride);
      if (okm && a.epilogue == kEpiBiasAct && a.aux != nullptr)
        okm = make_out_map(&om.m[1], a.aux, a.N, a.M, a.groups, a.aux_row_stride, a.aux_group_stride);
    }
    kp.tma_out = okm ? 1 : 0;
  }

  if (cg == 2) return launch_layout<2>(a, ta, tb, om, kp, ctas, stream);
  return launch_layout<1>(a, ta, tb, om, kp, ctas, stream);
}

// ---------------------------------------------------------------------------------------------
// Column sums (bias gradients): fp32 [groups / fold][N] = sum over rows (and over `fold` leading
// group blocks, the pipeline chunks) of bf16 [groups][rows][N].
// Two-stage and deterministic.  Stage 1: a CTA of 8 row lanes x 32 column threads reduces a slab of
// 128 rows x 256 columns with 16-byte loads (8 columns per thread), combines the row lanes through
// shared memory and writes one fp32 partial row.  Stage 2 adds the partials in slab order.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int kColsumSlab = 128;
constexpr int kColsumCols = 256;

__global__ void __launch_bounds__(256)
colsum_partial_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ partial, long long rows, int N,
                      long long row_stride, long long group_stride, int slabs) {
  __shared__ float red[8][kColsumCols + 8];
  const int ct = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int col0 = blockIdx.x * kColsumCols;
  const int col = col0 + ct * 8;
  const int slab = blockIdx.y, g = blockIdx.z;
  const long long r0 = (long long)slab * kColsumSlab;
  const long long r1 = r0 + kColsumSlab < rows ? r0 + kColsumSlab : rows;
  float a[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = 0.f;
  if (col < N) {
    const __nv_bfloat16* base = x + (long long)g * group_stride + col;
#pragma unroll 4
    for (long long r = r0 + rl; r < r1; r += 8) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(base + r * row_stride));
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
    partial[((long long)g * slabs + slab) * N + col0 + c] = acc;
  }
}

__global__ void __launch_bounds__(256)
colsum_final_kernel(const float* __restrict__ partial, float* __restrict__ out, __nv_bfloat16* __restrict__ out_bf16,
                    int N, int slabs, int fold, int out_groups) {
  // 32 columns x 8 slab lanes per CTA: lane l adds partials l, l + 8, ... (independent loads in flight),
  // the eight lane sums are then added in lane order, so the result does not depend on timing.
  __shared__ float red[8][33];
  const int ct = threadIdx.x & 31, sl = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + ct;
  const int e = blockIdx.y;
  float acc = 0.f;
  if (col < N) {
    const int total = fold * slabs;
#pragma unroll 4
    for (int i = sl; i < total; i += 8) {
      const int j = i / slabs, s = i - j * slabs;
      acc += partial[((long long)(j * out_groups + e) * slabs + s) * N + col];
    }
  }
  red[sl][ct] = acc;
  __syncthreads();
  if (sl == 0 && col < N) {
    float r = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) r += red[l][ct];
    out[(long long)e * N + col] = r;
    if (out_bf16 != nullptr) out_bf16[(long long)e * N + col] = __float2bfloat16_rn(r);
  }
}
}  // namespace

int colsum_slabs(long long rows) { return (int)((rows + kColsumSlab - 1) / kColsumSlab); }

// `out` must have room for (groups / fold) * N floats followed by groups * colsum_slabs(rows) * N floats of
// scratch.  N must be a multiple of 8 and rows of x 16-byte aligned.  groups = fold * (groups / fold):
// group j * (groups / fold) + e is summed into output row e.  `out_bf16` (optional) receives the same sums
// rounded to bf16.
void launch_colsum_bf16(const void* x, float* out, int groups, long long rows, int N, long long row_stride,
                        long long group_stride, int fold, void* out_bf16, cudaStream_t stream) {
  if (fold < 1) fold = 1;
  const int out_groups = groups / fold;
  const int slabs = colsum_slabs(rows);
  float* partial = out + (long long)out_groups * N;
  dim3 g1((N + kColsumCols - 1) / kColsumCols, slabs, groups);
  colsum_partial_kernel<<<g1, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), partial, rows, N,
                                              row_stride, group_stride, slabs);
  dim3 g2((N + 31) / 32, out_groups);
  colsum_final_kernel<<<g2, 256, 0, stream>>>(partial, out, reinterpret_cast<__nv_bfloat16*>(out_bf16), N, slabs, fold,
                                            out_groups);
}

}  // namespace planmoe
