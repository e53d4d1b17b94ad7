// Host-side launch interface of the planmoe_b200 native kernels (sm_100a).
// Every launcher enqueues on the given stream and allocates nothing.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace planmoe {

// ---- CPU reference loops (kernels/cpu_ref.cpp) ---------------------------------------------
template <class T>
void cpu_scatter(const T* x, const int* idx, const int* loc, const T* gates, T* disp, int K, int S,
                 int M, int E, int C);
template <class T>
void cpu_gather(const T* disp, const int* idx, const int* loc, const T* gates, T* out, int K, int S,
                int M, int C);
template <class T>
void cpu_gate_grad(const T* disp, const T* dy, const int* idx, const int* loc, T* dgates, int K,
                   int S, int M, int C);

// ---- peer-push / flag-wait descriptors -------------------------------------------------------
// A buffer in the symmetric heap is named by its byte offset; rank r's copy lives at
// heap_bases[r] + offset (heap_bases is a device array of W peer-mapped base addresses).
struct PushArgs {
  const unsigned long long* heap_bases;  // device [W]
  unsigned long long data_off;           // destination buffer
  unsigned long long flag_off;           // u64 flags [chunks][W] on the destination rank
  unsigned long long scale_off;          // fp32 (range, lo) per row, int8 mode only
  int W, my_rank, chunks;
  int ctas_per_msg;                      // CTAs of the persistent grid = arrivals each flag receives
  int chunk_begin, chunk_count;          // chunks served by this launch (count 0 = all)
};
struct WaitArgs {
  const unsigned long long* flags;  // local device pointer, n_flags consecutive u64
  int n_flags;
  unsigned long long want;          // proceed when every flag >= want
  const unsigned long long* want_ptr;  // if set: `want` is read from this device word instead (CUDA-graph replays)
  unsigned long long budget_ns;     // give up (status word, kernel returns) after this long
  int* status;                      // host-mapped int32[8]
};

// ---- kernels/dispatch.cu ---------------------------------------------------------------------
void launch_build_slot_map(const int* idx, const int* loc, int* slot_map, int K, int S, int E, int C,
                           cudaStream_t stream);
template <class T>
void launch_scatter_rows(const T* x, const int* slot_map, const float* gates, T* local_out, int K,
                         int S, int M, int E, int C, const PushArgs* push, bool quant,
                         cudaStream_t stream);
// scale_bias: null (rows of T), or fp32 (range, low) per row with uint8 rows (int8 codec), or -- with
// group_rows > 0 -- fp32 (scale, low) per (128-column group, row), laid out [M / 128][group_rows], with uint8 rows
// (what the int8 push epilogue of the grouped GEMM writes)
template <class T>
void launch_gather_rows(const void* disp, const float* scale_bias, const int* idx, const int* loc,
                        const float* gates, T* out, int K, int S, int M, int C, const WaitArgs* wait,
                        cudaStream_t stream, long long group_rows = 0);
// `gates` / `scaled` optional: also write scaled[t * K + k] = gates[k][t] * dy[t]
// disp_scales != null: disp holds uint8 rows with fp32 (scale, low) per (128-column group, row), [M / 128][E * C];
// scaled_q (int8 mode only): the gate-weighted dy rows as int8 wire rows [S * K][M + 16] instead of `scaled`
template <class T>
void launch_gate_grad(const T* disp, const T* dy, const int* idx, const int* loc, float* dgates,
                      const float* gates, T* scaled, int K, int S, int M, int C, cudaStream_t stream,
                      const float* disp_scales = nullptr, long long group_rows = 0, unsigned char* scaled_q = nullptr);

// ---- kernels/gate.cu -------------------------------------------------------------------------
int gate_workspace_blocks(int S);
template <class T>
void launch_gate_forward(const T* logits, int S, int E, int K, int C, bool normalize, float eps,
                         int* idx, int* loc, float* gates, float* raw_gate, int* slot_map,
                         int* top1_count, float* l_aux, int* ws_rank, int* ws_blk_count,
                         float* ws_blk_score, cudaStream_t stream);
template <class T>
void launch_gate_backward(const T* logits, int S, int E, int K, bool normalize, float eps,
                          const int* idx, const float* dgates, const float* dl_aux,
                          const int* top1_count, T* dlogits, cudaStream_t stream);
// order of tokens for batch-prioritised routing: rank[t] = position of token t (best top score first, ties by index),
// perm[position] = token; `key` is an fp32 [S] workspace
template <class T>
void launch_importance_order(const T* logits, int S, int E, float* key, int* rank, int* perm, cudaStream_t stream);
void launch_remap_slot_map(int* slot_map, long long n, const int* perm, int K, cudaStream_t stream);
int cumsum_tiles(int S);
void launch_cumsum_sub_one(const int* x, int* out, int* tile_sum, int S, int E, cudaStream_t stream);

// ---- codec/int8.cu ---------------------------------------------------------------------------
template <class T>
void launch_int8_encode(const T* x, unsigned char* q, float* scale, float* bias, int R, int M,
                        cudaStream_t stream);
template <class T>
void launch_int8_decode(const unsigned char* q, const float* scale, const float* bias, T* out, int R,
                        int M, cudaStream_t stream);

// rows of M + 16 bytes: M uint8 + {scale, low, 0, 0} (the wire rows of the fused MoE send); M % 16 == 0
template <class T>
void launch_int8_rows_encode(const T* x, unsigned char* out, int R, int M, cudaStream_t stream);

// ---- kernels/a2a.cu --------------------------------------------------------------------------
// msgs: device int64 [n_msgs][6] = (dest rank or -1, flag index to signal or -1, src_off, dst_off, bytes,
// position in wait_flags this message alone waits for, or -1 = all of wait_idx).
// len_off >= 0: every message is self-describing; the u32 at byte len_off of its source is its payload size and
// only len_base + that many bytes (rounded up to 16) are moved.
void launch_xfer(const void* src_base, const long long* msgs, int n_msgs, int ctas_per_msg,
                 const unsigned long long* heap_bases, unsigned long long flag_off,
                 const unsigned long long* wait_flags, const int* wait_idx, int n_wait, unsigned long long want,
                 unsigned long long budget_ns, int* status, void* local_dst, cudaStream_t stream,
                 long long len_off = -1, unsigned long long len_base = 0);
void launch_wait_flags(const unsigned long long* flags, int n, unsigned long long want, unsigned long long budget_ns,
                       int* status, cudaStream_t stream);
// keeps the stream busy for ns nanoseconds (clamped to 200 ms)
void launch_delay(unsigned long long ns, cudaStream_t stream);

// ---- kernels/gemm_tcgen05.cu -----------------------------------------------------------------
// Grouped bf16 GEMM  D[g] (Mg x N) = A[g] (Mg x K) . B[g] (K x N), fp32 accumulation in TMEM.
enum GemmEpilogue : int {
  kEpiStore = 0,    // D = acc (+ bias)
  kEpiBiasAct = 1,  // t = acc + bias ; D = act(t) ; aux = act'(t)
  kEpiDAct = 2,     // D = acc * aux      (aux = a saved activation derivative)
  kEpiPush = 3,     // (acc + bias) stored into the origin ranks' combine buffers + flags
};
enum Activation : int { kActIdentity = 0, kActRelu = 1, kActGelu = 2, kActSilu = 3 };

struct GemmOperand {
  const void* ptr;     // bf16
  int mn_major;        // 0: rows of the MN dim, K contiguous; 1: rows of K, MN dim contiguous
  // Extents / strides in elements.  Row dim = MN rows (K-major) or K rows (MN-major).
  long long rows, cols;            // cols = contiguous extent
  long long row_stride;            // elements between rows
  long long group_stride;          // elements between groups
  long long chunk_stride;          // elements between split-K chunks (0 if unused)
  int chunks;                      // split-K chunks folded into the K loop (>= 1)
};

struct GemmArgs {
  GemmOperand A, B;
  int groups, M, N, K;             // per-group problem; K is per chunk when chunks > 1
  int epilogue, activation;
  void* D; long long d_row_stride, d_group_stride;          // bf16 output
  void* aux; long long aux_row_stride, aux_group_stride;    // bf16 activation derivative (in or out)
  const void* bias; long long bias_group_stride;            // bf16 [groups][N] or null
  // flag-gated A rows (A is a receive buffer filled by peers): rows [s*gate_rows, (s+1)*gate_rows)
  // of every group become readable when gate_flags[s] >= gate_want.
  const unsigned long long* gate_flags; int gate_rows; unsigned long long gate_want;
  const unsigned long long* gate_want_ptr;   // if set: gate_want is read from this device word at kernel start
  // gate_mode 1 (the fused dispatch send's protocol): one flag per 128-row block of a group,
  // gate_flags[g * gate_nblk + row / 128], counting ROWS; a block is readable when its flag has reached
  // gate_want * (rows in the block), gate_want being the number of times the buffer has been filled.
  int gate_mode, gate_nblk;
  // perm_w > 1: a group's rows are perm_w source segments of perm_seg_rows rows each; when a segment is a whole
  // number (> 1) of tiles, the tiles are visited segment-interleaved (tile 0 of every source, then tile 1, ...),
  // the order in which the fused send delivers rows
  int perm_w, perm_seg_rows;
  // 1: the copy role sends the rows that stay on this rank first (chunk by chunk) and the tile loop starts on this
  // rank's own segments; 0: destinations and sources are interleaved from the first row on
  int perm_local_first;
  // push epilogue: row m of group g belongs to rank s = m / push_rows; it is stored at
  // heap_bases[s] + push_data_off + ((my_rank*groups + g) * push_C + push_c0 + m % push_rows) * N
  // and flag (push_flag_off)[push_chunk * W + my_rank] on rank s is incremented once per tile.
  const unsigned long long* heap_bases; unsigned long long push_data_off, push_flag_off;
  int push_rows, push_C, push_c0, push_chunk, W, my_rank;
  // push_q8: rows are stored as N bytes of uint8 at heap_bases[s] + push_data_off + row * N, and one fp32
  // (scale, low) pair per row and 128-column group at push_scale_off + ((n / 128) * rows_total + row) * 8,
  // value = q * scale + low.  Needs N % 128 == 0 and the bulk-store form (heap_bases_host, rows % 32 == 0).
  int push_q8; unsigned long long push_scale_off;
  // host copy of heap_bases (optional): lets the push epilogue use bulk tensor stores into the peers' buffers
  const unsigned long long* heap_bases_host;
  // chunk_groups > 0: the `groups` of A / D / aux are [chunk][expert] with chunk_groups experts per
  // chunk; B and bias are indexed by the expert (group % chunk_groups); gate flags are
  // gate_flags[chunk * W + s]; pushed rows land at column offset chunk * push_rows and signal
  // flag [chunk * W + my_rank].  One launch then covers all pipeline chunks.
  int chunk_groups;
  unsigned long long budget_ns; int* status;
  // Optional role trace, device u64 [grid][32] (ns of %globaltimer): [0] kernel entry, [1] / [2] copy role begin / end,
  // [3] time the TMA producer spent waiting on gate flags, [4] kernel exit, [5] de-quantiser role end; in SM clocks,
  // from the first epilogue warp: [6] waiting for accumulators, [7] (whole tile loop << 32) | waiting for staging tiles;
  // [8 + 2i] / [9 + 2i]: when the TMA producer began / ended waiting for the rows of its i-th tile (i < 12).
  unsigned long long* trace;
  int max_ctas;                    // 0 = one per SM
  int cta_group;                   // 0 = automatic (gemm_cta_group), 1, or 2 (two-CTA clusters, 256 x 256 tiles)
  // Fused dispatch send ("copy role"): with copy.ctas > 0 one extra warp of every CTA moves token rows
  // of copy.x, picked by slot map, with the bulk-copy engine straight into the receive buffer of the rank
  // that owns each expert, 8 rows at a time, and release-adds the row count to the flag of the 128-row
  // block the rows lie in on the destination (gate_mode 1 on the receiving side).  The producers of the
  // same launch on every rank are the flag-gated consumers of this exchange, so the transfer and the math
  // overlap inside one kernel.  Rows of at most 16 KiB.  Uses heap_bases / W / my_rank above.
  struct CopyJob {
    const void* x;                 // source rows [S][row_bytes]: bf16 tokens, or int8 rows with their 16-byte trailer
    const int* slot_map;           // [E_global * C] -> token * K + k, or -1
    const float* gates;            // unused (gate-weighted rows are prepared by the caller)
    int K, S, M, E_local, C, chunks, ctas;
    unsigned long long data_off, flag_off;   // destination buffer / u64 row-count flags [groups][nblk] in the heap
    int nblk;                      // 128-row blocks per group of the destination buffer (= ceil(W * C / chunks / 128))
    int row_bytes;                 // bytes per row, the same at source and destination (a multiple of 16, <= 16384)
  } copy;
  // De-quantiser role (int8 wire): expands the int8 rows that peers stored into this rank's landing buffer
  // [groups][rows][M + 16] into the bf16 A operand, 32 rows per unit in the order the tiles are consumed, and
  // release-adds the row count to ready_flags[g * nblk + row / 128] (= gate_flags of the same launch).
  struct DequantJob {
    const void* q;                         // local landing buffer, or null (role idle)
    const unsigned long long* arrival;     // local flags the peers' copy warps add rows to
    unsigned long long* ready;             // local flags this role adds rows to
    int M;                                 // elements per row
  } dequant;
};

// Returns cudaSuccess or the launch / tensor-map error.
cudaError_t launch_grouped_gemm(const GemmArgs& args, cudaStream_t stream);
// CTAs the launch of such a problem uses (= arrivals per flag of a fused copy job).
int gemm_cta_group(int M, int requested);
int gemm_grid_ctas(int groups, int M, int N, int max_ctas, int cta_group);
// Number of flag arrivals rank s receives per push launch (host helper for the receiver).
int gemm_push_arrivals(int groups, int M, int N, int push_rows, int s);

// Column sums of a bf16 [groups][rows][N] tensor -> fp32 [groups / fold][N] (bias gradients); the `fold`
// leading blocks of groups (pipeline chunks) are added together.  `out` = (groups / fold) * N results
// followed by groups * colsum_slabs(rows) * N floats of scratch and (groups / fold) * colsum_colblocks(N) counter
// words; `out_bf16` optionally gets bf16 copies.
int colsum_slabs(long long rows);
void launch_colsum_bf16(const void* x, float* out, int groups, long long rows, int N,
                        long long row_stride, long long group_stride, int fold, void* out_bf16,
                        cudaStream_t stream);
// One or two column-sum jobs in the same two launches (see launch_colsum_bf16 for the meaning of the fields).
// `partial`: groups * colsum_slabs(rows) * N floats; `counters` is reserved (the two-stage form does not use it).
struct ColsumJob {
  const void* x; float* out; void* out_bf16; float* partial; unsigned* counters;
  long long rows, row_stride, group_stride;
  int N, groups, fold;
};
int colsum_colblocks(int N);
void launch_colsum_jobs(const ColsumJob* jobs, int n, cudaStream_t stream);

}  // namespace planmoe
