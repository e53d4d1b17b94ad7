// Python bindings of the planmoe_b200 native extension (module planmoe_b200._C).
//
// Thin adapters from torch::Tensor to the raw-pointer launchers of planmoe.h; every CUDA op
// runs on the current torch stream.  The list of exported functions covers what the
// reference binds in PlanMoE/custom/custom_kernel.cpp:292-321 (CPU sparse ops, JIT invoke,
// collective bootstrap, codec/comm pipeline), re-expressed for this design: the NCCL bootstrap
// becomes the symmetric-heap runtime, the FIFO compress/comm/decompress triple becomes explicit
// handles on the Python side.

#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGuard.h>

#include "planmoe.h"
#include "runtime/symm_heap.h"
#include "runtime/jit.h"
#include "codec/codecs.h"
#include "codec/abstract.h"
#include "comm/abstract.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

namespace py = pybind11;
using torch::Tensor;
using namespace planmoe;

namespace {

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

// Kernels of this extension launched so far in this process (benchmarks report the delta).
std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

void check_cuda(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}

#define DISPATCH_FLOAT(t, NAME, ...)                                                     \
  [&] {                                                                                  \
    switch ((t).scalar_type()) {                                                         \
      case at::kFloat: { using scalar_t = float; return __VA_ARGS__(); }                 \
      case at::kBFloat16: { using scalar_t = __nv_bfloat16; return __VA_ARGS__(); }      \
      case at::kHalf: { using scalar_t = __half; return __VA_ARGS__(); }                 \
      default: TORCH_CHECK(false, NAME, ": unsupported dtype ", (t).scalar_type());      \
    }                                                                                    \
  }()

const float* opt_f32(const c10::optional<Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous(), "gates must be contiguous fp32");
  return t->data_ptr<float>();
}

// ---- CPU sparse ops -------------------------------------------------------------------------
template <class T>
const T* opt_ptr(const c10::optional<Tensor>& t) {
  return (t.has_value() && t->defined()) ? t->data_ptr<T>() : nullptr;
}

Tensor cpu_scatter_op(const Tensor& x, const Tensor& idx, const Tensor& loc, const c10::optional<Tensor>& gates,
                      int64_t E, int64_t C) {
  TORCH_CHECK(!x.is_cuda() && x.dim() == 2 && x.is_contiguous());
  const int K = idx.size(0), S = idx.size(1), M = x.size(1);
  Tensor out = torch::empty({E * C, M}, x.options());
  if (x.scalar_type() == at::kFloat)
    cpu_scatter<float>(x.data_ptr<float>(), idx.data_ptr<int>(), loc.data_ptr<int>(), opt_ptr<float>(gates),
                       out.data_ptr<float>(), K, S, M, E, C);
  else
    cpu_scatter<double>(x.data_ptr<double>(), idx.data_ptr<int>(), loc.data_ptr<int>(), opt_ptr<double>(gates),
                        out.data_ptr<double>(), K, S, M, E, C);
  return out;
}
Tensor cpu_gather_op(const Tensor& disp, const Tensor& idx, const Tensor& loc, const c10::optional<Tensor>& gates,
                     int64_t C) {
  TORCH_CHECK(!disp.is_cuda() && disp.dim() == 2 && disp.is_contiguous());
  const int K = idx.size(0), S = idx.size(1), M = disp.size(1);
  Tensor out = torch::empty({S, M}, disp.options());
  if (disp.scalar_type() == at::kFloat)
    cpu_gather<float>(disp.data_ptr<float>(), idx.data_ptr<int>(), loc.data_ptr<int>(), opt_ptr<float>(gates),
                      out.data_ptr<float>(), K, S, M, C);
  else
    cpu_gather<double>(disp.data_ptr<double>(), idx.data_ptr<int>(), loc.data_ptr<int>(), opt_ptr<double>(gates),
                       out.data_ptr<double>(), K, S, M, C);
  return out;
}
Tensor cpu_gate_grad_op(const Tensor& disp, const Tensor& dy, const Tensor& idx, const Tensor& loc, int64_t C) {
  TORCH_CHECK(!disp.is_cuda() && disp.is_contiguous() && dy.is_contiguous());
  const int K = idx.size(0), S = idx.size(1), M = disp.size(1);
  Tensor out = torch::empty({K, S}, disp.options());
  if (disp.scalar_type() == at::kFloat)
    cpu_gate_grad<float>(disp.data_ptr<float>(), dy.data_ptr<float>(), idx.data_ptr<int>(), loc.data_ptr<int>(),
                         out.data_ptr<float>(), K, S, M, C);
  else
    cpu_gate_grad<double>(disp.data_ptr<double>(), dy.data_ptr<double>(), idx.data_ptr<int>(), loc.data_ptr<int>(),
                          out.data_ptr<double>(), K, S, M, C);
  return out;
}

// ---- CUDA dispatch ops ----------------------------------------------------------------------
Tensor build_slot_map_op(const Tensor& idx, const Tensor& loc, int64_t E, int64_t C) {
  count_launch(1);
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kInt && idx.is_contiguous() && loc.is_contiguous());
  c10::cuda::CUDAGuard guard(idx.device());
  Tensor smap = torch::empty({E * C}, idx.options());
  launch_build_slot_map(idx.data_ptr<int>(), loc.data_ptr<int>(), smap.data_ptr<int>(), idx.size(0), idx.size(1), E, C,
                        cur_stream());
  return smap;
}

Tensor dispatch_scatter_op(const Tensor& x, const Tensor& slot_map, const c10::optional<Tensor>& gates, int64_t K,
                           int64_t n_slots) {
  count_launch(1);
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous(), "x must be contiguous [S, M] on CUDA");
  const int S = x.size(0), M = x.size(1);
  TORCH_CHECK((M * x.element_size()) % 16 == 0, "row bytes must be a multiple of 16");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty({n_slots, M}, x.options());
  DISPATCH_FLOAT(x, "dispatch_scatter", [&] {
    launch_scatter_rows<scalar_t>(reinterpret_cast<const scalar_t*>(x.data_ptr()), slot_map.data_ptr<int>(),
                                  opt_f32(gates), reinterpret_cast<scalar_t*>(out.data_ptr()), K, S, M, 1, n_slots,
                                  nullptr, false, cur_stream());
  });
  return out;
}

Tensor dispatch_gather_op(const Tensor& disp, const Tensor& idx, const Tensor& loc, const c10::optional<Tensor>& gates,
                          int64_t C) {
  count_launch(1);
  TORCH_CHECK(disp.is_cuda() && disp.dim() == 2 && disp.is_contiguous());
  const int K = idx.size(0), S = idx.size(1), M = disp.size(1);
  TORCH_CHECK(K <= 8, "top-k above 8 is not supported by the gather kernel");
  TORCH_CHECK((M * disp.element_size()) % 16 == 0, "row bytes must be a multiple of 16");
  c10::cuda::CUDAGuard guard(disp.device());
  Tensor out = torch::empty({S, M}, disp.options());
  DISPATCH_FLOAT(disp, "dispatch_gather", [&] {
    launch_gather_rows<scalar_t>(disp.data_ptr(), nullptr, idx.data_ptr<int>(), loc.data_ptr<int>(), opt_f32(gates),
                                 reinterpret_cast<scalar_t*>(out.data_ptr()), K, S, M, C, nullptr, cur_stream());
  });
  return out;
}

Tensor dispatch_gate_grad_op(const Tensor& disp, const Tensor& dy, const Tensor& idx, const Tensor& loc, int64_t C) {
  count_launch(1);
  TORCH_CHECK(disp.is_cuda() && disp.is_contiguous() && dy.is_contiguous() && disp.scalar_type() == dy.scalar_type());
  const int K = idx.size(0), S = idx.size(1), M = disp.size(1);
  c10::cuda::CUDAGuard guard(disp.device());
  Tensor out = torch::empty({K, S}, disp.options().dtype(at::kFloat));
  DISPATCH_FLOAT(disp, "dispatch_gate_grad", [&] {
    launch_gate_grad<scalar_t>(reinterpret_cast<const scalar_t*>(disp.data_ptr()),
                               reinterpret_cast<const scalar_t*>(dy.data_ptr()), idx.data_ptr<int>(),
                               loc.data_ptr<int>(), out.data_ptr<float>(), nullptr, nullptr, K, S, M, C, cur_stream());
  });
  return out;
}

// Gate gradient plus the gate-weighted copies of dy: returns (dgates [K, S] fp32, scaled [S * K, M]) with
// scaled[t * K + k] = gates[k][t] * dy[t] for every pick that holds a slot (other rows are left unwritten).
std::vector<Tensor> dispatch_gate_grad_scaled_op(const Tensor& disp, const Tensor& dy, const Tensor& idx,
                                                 const Tensor& loc, const Tensor& gates, int64_t C) {
  count_launch(1);
  TORCH_CHECK(disp.is_cuda() && disp.is_contiguous() && dy.is_contiguous() && disp.scalar_type() == dy.scalar_type());
  TORCH_CHECK(gates.is_cuda() && gates.scalar_type() == at::kFloat && gates.is_contiguous());
  const int K = idx.size(0), S = idx.size(1), M = disp.size(1);
  TORCH_CHECK(gates.numel() == (int64_t)K * S && dy.size(0) == S && dy.size(1) == M);
  c10::cuda::CUDAGuard guard(disp.device());
  Tensor out = torch::empty({K, S}, disp.options().dtype(at::kFloat));
  Tensor scaled = torch::empty({(int64_t)S * K, (int64_t)M}, dy.options());
  DISPATCH_FLOAT(disp, "dispatch_gate_grad_scaled", [&] {
    launch_gate_grad<scalar_t>(reinterpret_cast<const scalar_t*>(disp.data_ptr()),
                               reinterpret_cast<const scalar_t*>(dy.data_ptr()), idx.data_ptr<int>(),
                               loc.data_ptr<int>(), out.data_ptr<float>(), gates.data_ptr<float>(),
                               reinterpret_cast<scalar_t*>(scaled.data_ptr()), K, S, M, C, cur_stream());
  });
  return {out, scaled};
}

// The same for expert outputs that arrived as uint8 rows with a (scale, low) pair per 128 columns and row (the int8
// push epilogue's layout): `disp_ptr` uint8 [E * C, M], `scales_ptr` fp32 [M / 128][group_rows][2].  `gates` may be
// absent (then no scaled copies are produced and the second result is empty).  The scaled copies come out as int8 wire
// rows, uint8 [S * K, M + 16]: M quantised bytes + {scale, low, 0, 0}.
std::vector<Tensor> dispatch_gate_grad_q8_op(int64_t disp_ptr, int64_t scales_ptr, int64_t group_rows, const Tensor& dy,
                                             const Tensor& idx, const Tensor& loc, const c10::optional<Tensor>& gates,
                                             int64_t C, bool want_scaled) {
  count_launch(1);
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && dy.dim() == 2 && dy.size(1) % 128 == 0);
  const int K = idx.size(0), S = idx.size(1), M = dy.size(1);
  c10::cuda::CUDAGuard guard(dy.device());
  Tensor out = torch::empty({K, S}, dy.options().dtype(at::kFloat));
  Tensor scaled;       // int8 wire rows [S * K, M + 16] of gate * dy (rows of picks without a slot stay unwritten)
  if (want_scaled) {
    TORCH_CHECK(gates.has_value() && gates->defined(), "scaled copies need the gates");
    scaled = torch::empty({(int64_t)S * K, (int64_t)M + 16}, dy.options().dtype(at::kByte));
  }
  DISPATCH_FLOAT(dy, "dispatch_gate_grad_q8", [&] {
    launch_gate_grad<scalar_t>(reinterpret_cast<const scalar_t*>(disp_ptr), reinterpret_cast<const scalar_t*>(dy.data_ptr()),
                               idx.data_ptr<int>(), loc.data_ptr<int>(), out.data_ptr<float>(), opt_f32(gates),
                               nullptr, K, S, M, C, cur_stream(), reinterpret_cast<const float*>(scales_ptr), group_rows,
                               want_scaled ? scaled.data_ptr<uint8_t>() : nullptr);
  });
  return {out, want_scaled ? scaled : Tensor()};
}

// (rank [S] i32, perm [S] i32) of the batch-prioritised token order
std::vector<Tensor> importance_order_op(const Tensor& logits) {
  count_launch(2);
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous());
  const int S = logits.size(0), E = logits.size(1);
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor key = torch::empty({S}, logits.options().dtype(at::kFloat));
  Tensor rank = torch::empty({S}, logits.options().dtype(at::kInt)), perm = torch::empty({S}, logits.options().dtype(at::kInt));
  DISPATCH_FLOAT(logits, "importance_order", [&] {
    launch_importance_order<scalar_t>(reinterpret_cast<const scalar_t*>(logits.data_ptr()), S, E, key.data_ptr<float>(),
                                      rank.data_ptr<int>(), perm.data_ptr<int>(), cur_stream());
  });
  return {rank, perm};
}
void remap_slot_map_op(Tensor& slot_map, const Tensor& perm, int64_t K) {
  count_launch(1);
  TORCH_CHECK(slot_map.is_cuda() && slot_map.is_contiguous() && slot_map.scalar_type() == at::kInt && perm.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(slot_map.device());
  launch_remap_slot_map(slot_map.data_ptr<int>(), slot_map.numel(), perm.data_ptr<int>(), (int)K, cur_stream());
}

// ---- fused gate -------------------------------------------------------------------------------
// returns (idx[K,S] i32, loc[K,S] i32, gates[K,S] f32, slot_map[E*C] i32, top1_count[E] i32, l_aux[1] f32)
std::vector<Tensor> gate_forward_op(const Tensor& logits, int64_t K, int64_t C, bool normalize) {
  count_launch(2);
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous());
  const int S = logits.size(0), E = logits.size(1);
  TORCH_CHECK(E <= 64 && K <= 4 && K <= E, "fused gate supports up to 64 experts and top-4");
  c10::cuda::CUDAGuard guard(logits.device());
  auto iopt = logits.options().dtype(at::kInt);
  auto fopt = logits.options().dtype(at::kFloat);
  Tensor idx = torch::empty({K, S}, iopt), loc = torch::empty({K, S}, iopt);
  Tensor gates = torch::empty({K, S}, fopt), raw = torch::empty({K, S}, fopt);
  Tensor smap = torch::empty({(int64_t)E * C}, iopt);
  Tensor top1 = torch::empty({E}, iopt), laux = torch::empty({1}, fopt);
  const int nblk = gate_workspace_blocks(S);
  Tensor ws_rank = torch::empty({K, S}, iopt);
  Tensor ws_cnt = torch::empty({nblk, K, E}, iopt);
  Tensor ws_score = torch::empty({nblk, E}, fopt);
  const float eps = logits.scalar_type() == at::kFloat ? 1.1920929e-07f
                    : (logits.scalar_type() == at::kHalf ? 9.765625e-04f : 7.8125e-03f);
  DISPATCH_FLOAT(logits, "gate_forward", [&] {
    launch_gate_forward<scalar_t>(reinterpret_cast<const scalar_t*>(logits.data_ptr()), S, E, K, C, normalize, eps,
                                  idx.data_ptr<int>(), loc.data_ptr<int>(), gates.data_ptr<float>(),
                                  raw.data_ptr<float>(), smap.data_ptr<int>(), top1.data_ptr<int>(),
                                  laux.data_ptr<float>(), ws_rank.data_ptr<int>(), ws_cnt.data_ptr<int>(),
                                  ws_score.data_ptr<float>(), cur_stream());
  });
  return {idx, loc, gates, smap, top1, laux};
}

Tensor gate_backward_op(const Tensor& logits, const Tensor& idx, const c10::optional<Tensor>& dgates,
                        const c10::optional<Tensor>& dl_aux, const Tensor& top1, bool normalize) {
  count_launch(1);
  const int S = logits.size(0), E = logits.size(1), K = idx.size(0);
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor out = torch::empty_like(logits);
  const float eps = logits.scalar_type() == at::kFloat ? 1.1920929e-07f
                    : (logits.scalar_type() == at::kHalf ? 9.765625e-04f : 7.8125e-03f);
  DISPATCH_FLOAT(logits, "gate_backward", [&] {
    launch_gate_backward<scalar_t>(reinterpret_cast<const scalar_t*>(logits.data_ptr()), S, E, K, normalize, eps,
                                   idx.data_ptr<int>(), opt_f32(dgates), opt_f32(dl_aux), top1.data_ptr<int>(),
                                   reinterpret_cast<scalar_t*>(out.data_ptr()), cur_stream());
  });
  return out;
}

Tensor cumsum_sub_one_op(const Tensor& x) {
  count_launch(2);
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kInt && x.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  const int S = x.size(0), E = x.size(1);
  Tensor out = torch::empty_like(x);
  Tensor ws = torch::empty({cumsum_tiles(S), E}, x.options());
  launch_cumsum_sub_one(x.data_ptr<int>(), out.data_ptr<int>(), ws.data_ptr<int>(), S, E, cur_stream());
  return out;
}

// ---- int8 codec ---------------------------------------------------------------------------------
std::vector<Tensor> int8_encode_op(const Tensor& rows) {
  count_launch(1);
  TORCH_CHECK(rows.is_cuda() && rows.dim() == 2 && rows.is_contiguous());
  c10::cuda::CUDAGuard guard(rows.device());
  const int R = rows.size(0), M = rows.size(1);
  Tensor q = torch::empty({R, M}, rows.options().dtype(at::kByte));
  Tensor scale = torch::empty({R}, rows.options().dtype(at::kFloat)), bias = torch::empty_like(scale);
  DISPATCH_FLOAT(rows, "int8_encode", [&] {
    launch_int8_encode<scalar_t>(reinterpret_cast<const scalar_t*>(rows.data_ptr()), q.data_ptr<uint8_t>(),
                                 scale.data_ptr<float>(), bias.data_ptr<float>(), R, M, cur_stream());
  });
  return {q, scale, bias};
}
Tensor int8_decode_op(const Tensor& q, const Tensor& scale, const Tensor& bias, at::ScalarType dtype) {
  count_launch(1);
  TORCH_CHECK(q.is_cuda() && q.dim() == 2 && q.is_contiguous() && q.scalar_type() == at::kByte);
  c10::cuda::CUDAGuard guard(q.device());
  const int R = q.size(0), M = q.size(1);
  Tensor out = torch::empty({R, M}, q.options().dtype(dtype));
  DISPATCH_FLOAT(out, "int8_decode", [&] {
    launch_int8_decode<scalar_t>(q.data_ptr<uint8_t>(), scale.data_ptr<float>(), bias.data_ptr<float>(),
                                 reinterpret_cast<scalar_t*>(out.data_ptr()), R, M, cur_stream());
  });
  return out;
}

// ---- grouped GEMM ---------------------------------------------------------------------------
// Generic entry: operands are 3-D bf16 tensors [groups, rows, cols] with contiguous last dim
// (4-D [chunks, groups, rows, cols] when `chunks` > 1); `*_mn` says the MN dim is the contiguous one.
struct GemmOpts {
  int64_t epilogue = 0, activation = 0;
  c10::optional<Tensor> bias, aux, out;
  // flag gate
  int64_t gate_flags_ptr = 0, gate_rows = 0, gate_want = 0, gate_want_ptr = 0;
  int64_t gate_mode = 0, gate_nblk = 0, perm_w = 0, perm_seg_rows = 0, perm_local_first = 0;
  // push
  int64_t heap_bases_ptr = 0, push_data_off = 0, push_flag_off = 0, push_rows = 0, push_C = 0, push_c0 = 0,
          push_chunk = 0, W = 1, my_rank = 0, chunk_groups = 0, push_q8 = 0, push_scale_off = 0;
  int64_t budget_ms = 0, status_ptr = 0, max_ctas = 0, cta_group = 0;
  std::vector<int64_t> heap_bases_host;      // peers' mapped base addresses (push epilogue with bulk stores)
  // dispatch send fused into the launch (copy role)
  c10::optional<Tensor> copy_x, copy_slot_map, copy_gates;
  int64_t copy_K = 0, copy_E_local = 0, copy_C = 0, copy_chunks = 0, copy_ctas = 0, copy_data_off = 0,
          copy_flag_off = 0, copy_nblk = 0;
  // de-quantiser role (int8 wire): local landing buffer, arrival flags (set by peers), ready flags (set by the role)
  int64_t dq_ptr = 0, dq_arrival_ptr = 0, dq_ready_ptr = 0;
  int64_t trace_ptr = 0;                     // optional u64 [grid][8] role trace (see GemmArgs::trace)
};

GemmOperand operand_of(const Tensor& t, bool mn_major) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, "GEMM operands must be CUDA bf16");
  TORCH_CHECK(t.dim() == 3 || t.dim() == 4, "GEMM operand must be [groups, rows, cols] or [chunks, groups, rows, cols]");
  TORCH_CHECK(t.stride(-1) == 1, "GEMM operand needs a contiguous last dim");
  GemmOperand o{};
  o.ptr = t.data_ptr();
  o.mn_major = mn_major ? 1 : 0;
  const int d = t.dim();
  o.rows = t.size(d - 2); o.cols = t.size(d - 1);
  o.row_stride = t.stride(d - 2);
  o.group_stride = t.size(d - 3) > 1 ? t.stride(d - 3) : 0;
  o.chunks = d == 4 ? t.size(0) : 1;
  o.chunk_stride = (d == 4 && t.size(0) > 1) ? t.stride(0) : 0;
  return o;
}

Tensor grouped_gemm_op(const Tensor& A, bool a_mn, const Tensor& B, bool b_mn, const GemmOpts& o) {
  count_launch(1);
  c10::cuda::CUDAGuard guard(A.device());
  GemmArgs g{};
  g.A = operand_of(A, a_mn);
  g.B = operand_of(B, b_mn);
  const int groups = A.size(A.dim() - 3);
  TORCH_CHECK(o.chunk_groups > 0 ? (groups % o.chunk_groups == 0 && B.size(B.dim() - 3) == o.chunk_groups)
                                 : B.size(B.dim() - 3) == groups, "group count mismatch");
  g.groups = groups;
  g.M = a_mn ? g.A.cols : g.A.rows;
  g.K = a_mn ? g.A.rows : g.A.cols;
  g.N = b_mn ? g.B.cols : g.B.rows;
  const int64_t kb = b_mn ? g.B.rows : g.B.cols;
  TORCH_CHECK(kb == g.K, "contraction extents differ: ", g.K, " vs ", kb);
  g.epilogue = o.epilogue; g.activation = o.activation;

  Tensor out;
  if (o.epilogue != kEpiPush) {
    if (o.out.has_value() && o.out->defined()) {
      out = *o.out;
      TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.stride(-1) == 1 && out.dim() == 3);
    } else {
      out = torch::empty({groups, g.M, g.N}, A.options());
    }
    g.D = out.data_ptr(); g.d_row_stride = out.stride(1); g.d_group_stride = out.stride(0);
  }
  if (o.aux.has_value() && o.aux->defined()) {
    const Tensor& aux = *o.aux;
    TORCH_CHECK(aux.scalar_type() == at::kBFloat16 && aux.stride(-1) == 1 && aux.dim() == 3);
    g.aux = aux.data_ptr(); g.aux_row_stride = aux.stride(1); g.aux_group_stride = aux.stride(0);
  } else {
    TORCH_CHECK(o.epilogue != kEpiDAct, "activation-backward epilogue needs aux");
  }
  if (o.bias.has_value() && o.bias->defined()) {
    const Tensor& b = *o.bias;
    TORCH_CHECK(b.scalar_type() == at::kBFloat16 && b.is_contiguous() &&
                b.numel() == (int64_t)(o.chunk_groups > 0 ? o.chunk_groups : groups) * g.N);
    g.bias = b.data_ptr(); g.bias_group_stride = g.N;
  }
  g.gate_flags = reinterpret_cast<const unsigned long long*>(o.gate_flags_ptr);
  g.gate_rows = o.gate_rows; g.gate_want = o.gate_want;
  g.gate_want_ptr = reinterpret_cast<const unsigned long long*>(o.gate_want_ptr);
  g.gate_mode = o.gate_mode; g.gate_nblk = o.gate_nblk; g.perm_w = o.perm_w; g.perm_seg_rows = o.perm_seg_rows; g.perm_local_first = (int)o.perm_local_first;
  g.heap_bases = reinterpret_cast<const unsigned long long*>(o.heap_bases_ptr);
  g.push_data_off = o.push_data_off; g.push_flag_off = o.push_flag_off; g.push_rows = o.push_rows;
  g.push_C = o.push_C; g.push_c0 = o.push_c0; g.push_chunk = o.push_chunk; g.W = o.W; g.my_rank = o.my_rank;
  g.chunk_groups = o.chunk_groups;
  g.push_q8 = o.push_q8; g.push_scale_off = o.push_scale_off;
  std::vector<unsigned long long> bases_host(o.heap_bases_host.begin(), o.heap_bases_host.end());
  if (!bases_host.empty() && (int64_t)bases_host.size() == o.W) g.heap_bases_host = bases_host.data();
  g.budget_ns = (unsigned long long)o.budget_ms * 1000000ull;
  g.status = reinterpret_cast<int*>(o.status_ptr);
  g.trace = reinterpret_cast<unsigned long long*>(o.trace_ptr);
  g.max_ctas = o.max_ctas;
  g.cta_group = o.cta_group;
  if (o.epilogue == kEpiPush) TORCH_CHECK(g.heap_bases != nullptr, "push epilogue needs heap bases");
  if (o.copy_ctas > 0) {
    TORCH_CHECK(o.copy_x.has_value() && o.copy_slot_map.has_value(), "copy role needs x and slot_map");
    const Tensor& cx = *o.copy_x;
    const Tensor& sm = *o.copy_slot_map;
    TORCH_CHECK(cx.is_cuda() && (cx.scalar_type() == at::kBFloat16 || cx.scalar_type() == at::kByte) && cx.dim() == 2 &&
                cx.is_contiguous(), "copy role: x must be contiguous rows, bf16 [S, M] or uint8 [S, M + 16]");
    TORCH_CHECK(sm.is_cuda() && sm.scalar_type() == at::kInt && sm.is_contiguous(), "copy role: slot_map must be int32");
    TORCH_CHECK(g.heap_bases != nullptr && o.copy_K > 0 && o.copy_E_local > 0 && o.copy_C > 0 && o.copy_chunks > 0,
                "copy role: incomplete geometry");
    TORCH_CHECK(sm.numel() == o.copy_E_local * o.W * o.copy_C, "copy role: slot_map size");
    g.copy.x = cx.data_ptr(); g.copy.slot_map = sm.data_ptr<int>();
    g.copy.S = cx.size(0); g.copy.M = cx.size(1);
    if (o.copy_gates.has_value() && o.copy_gates->defined()) {
      const Tensor& cg = *o.copy_gates;
      TORCH_CHECK(cg.is_cuda() && cg.scalar_type() == at::kFloat && cg.is_contiguous() &&
                  cg.numel() == o.copy_K * cx.size(0), "copy role: gates must be fp32 [K, S]");
      g.copy.gates = cg.data_ptr<float>();
    }
    g.copy.K = o.copy_K; g.copy.E_local = o.copy_E_local; g.copy.C = o.copy_C; g.copy.chunks = o.copy_chunks;
    g.copy.ctas = o.copy_ctas; g.copy.data_off = o.copy_data_off; g.copy.flag_off = o.copy_flag_off;
    g.copy.nblk = o.copy_nblk; g.copy.row_bytes = (int)(cx.size(1) * cx.element_size());
  }
  if (o.dq_ptr != 0) {
    g.dequant.q = reinterpret_cast<const void*>(o.dq_ptr);
    g.dequant.arrival = reinterpret_cast<const unsigned long long*>(o.dq_arrival_ptr);
    g.dequant.ready = reinterpret_cast<unsigned long long*>(o.dq_ready_ptr);
    g.dequant.M = g.K;
  }
  check_cuda(launch_grouped_gemm(g, cur_stream()), "grouped_gemm");
  return out;
}

// fp32 column sums [groups / fold, N] of a bf16 [groups, rows, N] tensor; with `as_bf16` the result is
// returned in bf16 (written by the same kernel).  Two launches: partial sums, then their sum.
static void colsum_check(const Tensor& x, int64_t fold) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 3 && x.stride(2) == 1);
  TORCH_CHECK(fold >= 1 && x.size(0) % fold == 0, "colsum: groups must be a multiple of fold");
  TORCH_CHECK(x.size(2) % 8 == 0 && x.stride(1) % 8 == 0 && x.stride(0) % 8 == 0, "colsum needs 16-byte aligned rows");
}

// scratch of one job: [out][partials][counters]; fills `j`, returns the buffer
static Tensor colsum_job(const Tensor& x, int64_t fold, bool as_bf16, ColsumJob& j, Tensor& ob) {
  const int groups = x.size(0), N = x.size(2);
  const int64_t rows = x.size(1), slabs = colsum_slabs(rows), out_groups = groups / fold;
  const int64_t counters = out_groups * colsum_colblocks(N);
  Tensor buf = torch::empty({out_groups * N + (int64_t)groups * N * slabs + counters}, x.options().dtype(at::kFloat));
  if (as_bf16) ob = torch::empty({out_groups, (int64_t)N}, x.options());
  j.x = x.data_ptr(); j.out = buf.data_ptr<float>(); j.out_bf16 = as_bf16 ? ob.data_ptr() : nullptr;
  j.partial = j.out + out_groups * N;
  j.counters = reinterpret_cast<unsigned*>(j.partial + (int64_t)groups * N * slabs);
  j.rows = rows; j.row_stride = x.stride(1); j.group_stride = x.stride(0);
  j.N = N; j.groups = groups; j.fold = (int)fold;
  return buf;
}

Tensor colsum_op(const Tensor& x, int64_t fold, bool as_bf16) {
  count_launch(2);
  colsum_check(x, fold);
  c10::cuda::CUDAGuard guard(x.device());
  ColsumJob j{};
  Tensor ob;
  Tensor buf = colsum_job(x, fold, as_bf16, j, ob);
  launch_colsum_jobs(&j, 1, cur_stream());
  if (as_bf16) return ob;
  const int64_t out_groups = x.size(0) / fold;
  return buf.narrow(0, 0, out_groups * x.size(2)).view({out_groups, x.size(2)});
}

// Column sums of two tensors in the same two launches (the two bias gradients of the expert FFN).
std::vector<Tensor> colsum2_op(const Tensor& xa, const Tensor& xb, int64_t fold, bool as_bf16) {
  count_launch(2);
  colsum_check(xa, fold);
  colsum_check(xb, fold);
  TORCH_CHECK(xa.device() == xb.device());
  c10::cuda::CUDAGuard guard(xa.device());
  ColsumJob j[2] = {};
  Tensor oa, ob;
  Tensor ba = colsum_job(xa, fold, as_bf16, j[0], oa);
  Tensor bb = colsum_job(xb, fold, as_bf16, j[1], ob);
  launch_colsum_jobs(j, 2, cur_stream());
  if (as_bf16) return {oa, ob};
  const int64_t ga = xa.size(0) / fold, gb = xb.size(0) / fold;
  return {ba.narrow(0, 0, ga * xa.size(2)).view({ga, xa.size(2)}), bb.narrow(0, 0, gb * xb.size(2)).view({gb, xb.size(2)})};
}

// rows [R, M] -> uint8 [R, M + 16]: M quantised bytes + {scale, low, 0, 0} (the wire rows of the fused send)
Tensor int8_rows_encode_op(const Tensor& x) {
  count_launch(1);
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && x.size(1) % 16 == 0,
              "int8_rows_encode: contiguous CUDA [R, M] with M % 16 == 0");
  c10::cuda::CUDAGuard guard(x.device());
  const int R = x.size(0), M = x.size(1);
  Tensor out = torch::empty({(int64_t)R, (int64_t)M + 16}, x.options().dtype(at::kByte));
  DISPATCH_FLOAT(x, "int8_rows_encode", [&] {
    launch_int8_rows_encode<scalar_t>(reinterpret_cast<const scalar_t*>(x.data_ptr()), out.data_ptr<uint8_t>(), R, M,
                                      cur_stream());
  });
  return out;
}

// ---- push / wait wrappers for the fused MoE path ------------------------------------------------
void scatter_push_op(const Tensor& x, const Tensor& slot_map, const c10::optional<Tensor>& gates, int64_t K, int64_t E,
                     int64_t C, int64_t heap_bases_ptr, int64_t data_off, int64_t flag_off, int64_t W, int64_t my_rank,
                     int64_t chunks, int64_t ctas, int64_t chunk_begin, int64_t chunk_count) {
  count_launch(1);
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  PushArgs pa{};
  pa.heap_bases = reinterpret_cast<const unsigned long long*>(heap_bases_ptr);
  pa.data_off = data_off; pa.flag_off = flag_off; pa.scale_off = 0;
  pa.W = W; pa.my_rank = my_rank; pa.chunks = chunks; pa.ctas_per_msg = ctas;
  pa.chunk_begin = chunk_begin; pa.chunk_count = chunk_count;
  TORCH_CHECK(E % W == 0 && C % chunks == 0);
  const int S = x.size(0), M = x.size(1);
  DISPATCH_FLOAT(x, "scatter_push", [&] {
    launch_scatter_rows<scalar_t>(reinterpret_cast<const scalar_t*>(x.data_ptr()), slot_map.data_ptr<int>(),
                                  opt_f32(gates), nullptr, K, S, M, E, C, &pa, false, cur_stream());
  });
}

Tensor gather_wait_op(int64_t disp_ptr, at::ScalarType dtype, int64_t M, const Tensor& idx, const Tensor& loc,
                      const c10::optional<Tensor>& gates, int64_t C, int64_t flags_ptr, int64_t n_flags, int64_t want,
                      int64_t budget_ms, int64_t status_ptr, int64_t want_ptr, int64_t q8_scales_ptr,
                      int64_t q8_group_rows) {
  count_launch(1);
  c10::cuda::CUDAGuard guard(idx.device());
  const int K = idx.size(0), S = idx.size(1);
  Tensor out = torch::empty({S, M}, idx.options().dtype(dtype));
  WaitArgs wa{};
  wa.flags = reinterpret_cast<const unsigned long long*>(flags_ptr);
  wa.n_flags = n_flags; wa.want = want; wa.budget_ns = (unsigned long long)budget_ms * 1000000ull;
  wa.want_ptr = reinterpret_cast<const unsigned long long*>(want_ptr);
  wa.status = reinterpret_cast<int*>(status_ptr);
  DISPATCH_FLOAT(out, "gather_wait", [&] {
    launch_gather_rows<scalar_t>(reinterpret_cast<const void*>(disp_ptr), reinterpret_cast<const float*>(q8_scales_ptr),
                                 idx.data_ptr<int>(), loc.data_ptr<int>(), opt_f32(gates),
                                 reinterpret_cast<scalar_t*>(out.data_ptr()), K, S, M, C, flags_ptr ? &wa : nullptr,
                                 cur_stream(), q8_scales_ptr ? q8_group_rows : 0);
  });
  return out;
}

// ---- ZFP / LZ codecs (CPU or CUDA by the tensor's device) ------------------------------------------
int elem_code(at::ScalarType t) {
  if (t == at::kFloat) return 0;
  if (t == at::kBFloat16) return 1;
  if (t == at::kHalf) return 2;
  TORCH_CHECK(false, "zfp codec: unsupported dtype ", t);
}

Tensor zfp_encode_op(const Tensor& x, int64_t rate) {
  TORCH_CHECK(x.dim() == 3 && x.is_contiguous(), "zfp_encode expects a contiguous [lead, rows, M] tensor");
  TORCH_CHECK(rate == 4 || rate == 8 || rate == 16, "zfp rate must be 4, 8 or 16 bits per value");
  TORCH_CHECK(x.size(2) % 4 == 0, "zfp codec needs the last dim to be a multiple of 4");
  const int64_t lead = x.size(0), rows = x.size(1), M = x.size(2);
  const int64_t bytes = (int64_t)zfp_stream_bytes(rows, M, rate);
  Tensor out = torch::empty({lead, bytes}, x.options().dtype(at::kByte));
  if (x.is_cuda()) {
    count_launch(1);
    c10::cuda::CUDAGuard guard(x.device());
    launch_zfp_encode(x.data_ptr(), elem_code(x.scalar_type()), out.data_ptr<uint8_t>(), lead, rows, M, rate, cur_stream());
  } else {
    zfp_encode_cpu(x.data_ptr(), elem_code(x.scalar_type()), out.data_ptr<uint8_t>(), lead, rows, M, rate);
  }
  return out;
}

Tensor zfp_decode_op(const Tensor& stream, int64_t lead, int64_t rows, int64_t M, int64_t rate, at::ScalarType dtype) {
  TORCH_CHECK(stream.is_contiguous() && stream.scalar_type() == at::kByte);
  TORCH_CHECK(stream.numel() == lead * (int64_t)zfp_stream_bytes(rows, M, rate), "zfp stream size mismatch");
  Tensor out = torch::empty({lead, rows, M}, stream.options().dtype(dtype));
  if (stream.is_cuda()) {
    count_launch(1);
    c10::cuda::CUDAGuard guard(stream.device());
    launch_zfp_decode(stream.data_ptr<uint8_t>(), out.data_ptr(), elem_code(dtype), lead, rows, M, rate, cur_stream());
  } else {
    zfp_decode_cpu(stream.data_ptr<uint8_t>(), out.data_ptr(), elem_code(dtype), lead, rows, M, rate);
  }
  return out;
}

std::vector<Tensor> lz_encode_op(const Tensor& raw, int64_t sym) {
  TORCH_CHECK(raw.dim() == 2 && raw.is_contiguous() && raw.scalar_type() == at::kByte);
  TORCH_CHECK((sym == 2 || sym == 4) && raw.size(1) % sym == 0 && raw.size(1) % 16 == 0,
              "lz codec: slice bytes must be a multiple of 16 and of the symbol size");
  const int64_t slices = raw.size(0), raw_bytes = raw.size(1);
  const int64_t cap = (int64_t)lz_payload_capacity(raw_bytes);
  Tensor payload = torch::empty({slices, cap}, raw.options());
  Tensor sizes = torch::empty({slices}, raw.options().dtype(at::kInt));
  if (raw.is_cuda()) {
    count_launch(3);
    c10::cuda::CUDAGuard guard(raw.device());
    Tensor scratch = torch::empty({(int64_t)lz_scratch_bytes(slices, raw_bytes)}, raw.options());
    launch_lz_encode(raw.data_ptr<uint8_t>(), payload.data_ptr<uint8_t>(), sizes.data_ptr<int>(),
                     scratch.data_ptr<uint8_t>(), slices, raw_bytes, cap, sym, cur_stream());
  } else {
    lz_encode_cpu(raw.data_ptr<uint8_t>(), payload.data_ptr<uint8_t>(), sizes.data_ptr<int>(), slices, raw_bytes, cap, sym);
  }
  return {payload, sizes};
}

Tensor lz_decode_op(const Tensor& payload, const Tensor& sizes, int64_t raw_bytes, int64_t sym) {
  TORCH_CHECK(payload.dim() == 2 && payload.is_contiguous() && payload.scalar_type() == at::kByte);
  const int64_t slices = payload.size(0);
  Tensor raw = torch::empty({slices, raw_bytes}, payload.options());
  if (payload.is_cuda()) {
    count_launch(1);
    c10::cuda::CUDAGuard guard(payload.device());
    launch_lz_decode(payload.data_ptr<uint8_t>(), raw.data_ptr<uint8_t>(), slices, raw_bytes, payload.size(1), sym,
                     cur_stream());
  } else {
    lz_decode_cpu(payload.data_ptr<uint8_t>(), raw.data_ptr<uint8_t>(), slices, raw_bytes, payload.size(1), sym);
  }
  return raw;
}

// ---- C++ extension points: run a registered comm / codec on tensors -----------------------------
// A comm object registered in C++, kept alive across calls (it owns call counters and cached tables).
struct NativeCommHandle {
  std::unique_ptr<AbstractComm> comm;
  NativeCommHandle(const std::string& name, int64_t world_size, int64_t world_rank, int64_t local_size,
                   int64_t heap_bases_ptr, int64_t local_base, int64_t scratch_off, int64_t scratch_bytes,
                   int64_t status_ptr, int64_t budget_ms) {
    CommContext ctx;
    ctx.world_size = world_size; ctx.world_rank = world_rank; ctx.local_size = local_size > 0 ? local_size : world_size;
    ctx.local_rank = world_rank % ctx.local_size;
    ctx.heap_bases = reinterpret_cast<const unsigned long long*>(heap_bases_ptr);
    ctx.local_base = (unsigned long long)local_base;
    ctx.scratch_off = (unsigned long long)scratch_off; ctx.scratch_bytes = (unsigned long long)scratch_bytes;
    ctx.status = reinterpret_cast<int*>(status_ptr);
    if (budget_ms > 0) ctx.budget_ns = (unsigned long long)budget_ms * 1000000ull;
    comm = make_comm(name, ctx);
    TORCH_CHECK(comm != nullptr, "no native comm registered under `", name, "`");
  }
  int64_t scratch_bytes_for(int64_t payload) const { return (int64_t)comm->scratch_bytes_for((size_t)payload); }
  Tensor all_to_all(const Tensor& t) {
    Tensor in = t.contiguous();
    Tensor out = torch::empty_like(in);
    cudaStream_t s = nullptr;
    if (in.is_cuda()) { count_launch(2); s = cur_stream(); }
    c10::cuda::OptionalCUDAGuard guard;
    if (in.is_cuda()) guard.set_device(in.device());
    comm->all_to_all(in.data_ptr(), out.data_ptr(), in.numel() * in.element_size(), s);
    return out;
  }
};

Tensor native_codec_roundtrip_op(const std::string& name, const Tensor& t, int64_t parts, bool decode, int64_t out_bytes) {
  auto codec = make_compressor(name);
  TORCH_CHECK(codec != nullptr, "no native compressor registered under `", name, "`");
  Tensor in = t.contiguous();
  const size_t bytes = decode ? (size_t)out_bytes : in.numel() * in.element_size();
  cudaStream_t s = in.is_cuda() ? cur_stream() : nullptr;
  if (!decode) {
    Tensor wire = torch::empty({(int64_t)codec->wire_bytes(bytes, parts)}, in.options().dtype(at::kByte));
    codec->compress(in.data_ptr(), wire.data_ptr(), bytes, parts, in.element_size(), in.size(-1), s);
    return wire;
  }
  Tensor out = torch::empty({out_bytes}, in.options().dtype(at::kByte));
  codec->decompress(in.data_ptr(), out.data_ptr(), bytes, parts, 1, 1, s);
  return out;
}

// ---- stand-alone transfers --------------------------------------------------------------------
void xfer_op(int64_t src_ptr, const Tensor& msgs, int64_t ctas_per_msg, int64_t heap_bases_ptr, int64_t flag_off,
             int64_t wait_flags_ptr, const c10::optional<Tensor>& wait_idx, int64_t want, int64_t budget_ms,
             int64_t status_ptr, int64_t local_dst_ptr, int64_t len_off, int64_t len_base) {
  count_launch(1);
  TORCH_CHECK(msgs.is_cuda() && msgs.scalar_type() == at::kLong && msgs.is_contiguous() && msgs.dim() == 2 &&
              msgs.size(1) == 6, "msgs must be a contiguous CUDA int64 [n, 6] tensor");
  c10::cuda::CUDAGuard guard(msgs.device());
  const int n_wait = (wait_idx.has_value() && wait_idx->defined()) ? wait_idx->numel() : 0;
  launch_xfer(reinterpret_cast<const void*>(src_ptr), reinterpret_cast<const long long*>(msgs.data_ptr<int64_t>()),
              msgs.size(0), ctas_per_msg, reinterpret_cast<const unsigned long long*>(heap_bases_ptr), flag_off,
              reinterpret_cast<const unsigned long long*>(wait_flags_ptr), n_wait ? wait_idx->data_ptr<int>() : nullptr,
              n_wait, want, (unsigned long long)budget_ms * 1000000ull, reinterpret_cast<int*>(status_ptr),
              reinterpret_cast<void*>(local_dst_ptr), cur_stream(), len_off, (unsigned long long)len_base);
}

void wait_flags_op(int64_t flags_ptr, int64_t n, int64_t want, int64_t budget_ms, int64_t status_ptr) {
  count_launch(1);
  launch_wait_flags(reinterpret_cast<const unsigned long long*>(flags_ptr), n, want,
                    (unsigned long long)budget_ms * 1000000ull, reinterpret_cast<int*>(status_ptr), cur_stream());
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "planmoe_b200 native extension (sm_100a kernels, symmetric heap, CPU reference ops)";
  m.def("cpu_scatter", &cpu_scatter_op);
  m.def("cpu_gather", &cpu_gather_op);
  m.def("cpu_gate_grad", &cpu_gate_grad_op);
  m.def("build_slot_map", &build_slot_map_op);
  m.def("dispatch_scatter", &dispatch_scatter_op);
  m.def("dispatch_gather", &dispatch_gather_op);
  m.def("dispatch_gate_grad", &dispatch_gate_grad_op);
  m.def("dispatch_gate_grad_scaled", &dispatch_gate_grad_scaled_op);
  m.def("dispatch_gate_grad_q8", &dispatch_gate_grad_q8_op);
  m.def("gate_forward", &gate_forward_op);
  m.def("importance_order", &importance_order_op);
  m.def("remap_slot_map", &remap_slot_map_op);
  m.def("gate_backward", &gate_backward_op);
  m.def("cumsum_sub_one", &cumsum_sub_one_op);
  m.def("int8_encode", &int8_encode_op);
  m.def("int8_decode", &int8_decode_op);
  m.def("int8_rows_encode", &int8_rows_encode_op);
  m.def("colsum", &colsum_op, py::arg("x"), py::arg("fold") = 1, py::arg("as_bf16") = false);
  m.def("colsum2", &colsum2_op, py::arg("xa"), py::arg("xb"), py::arg("fold") = 1, py::arg("as_bf16") = false);
  m.def("scatter_push", &scatter_push_op);
  m.def("gather_wait", &gather_wait_op, py::arg("disp_ptr"), py::arg("dtype"), py::arg("M"), py::arg("idx"), py::arg("loc"),
        py::arg("gates"), py::arg("C"), py::arg("flags_ptr"), py::arg("n_flags"), py::arg("want"), py::arg("budget_ms"),
        py::arg("status_ptr"), py::arg("want_ptr") = 0, py::arg("q8_scales_ptr") = 0, py::arg("q8_group_rows") = 0);
  m.def("zfp_encode", &zfp_encode_op);
  m.def("zfp_decode", &zfp_decode_op);
  m.def("lz_encode", &lz_encode_op);
  m.def("lz_decode", &lz_decode_op);
  m.def("native_comm_names", &comm_names);
  m.def("native_compressor_names", &compressor_names);
  py::class_<NativeCommHandle>(m, "NativeCommHandle")
      .def(py::init<const std::string&, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t>(),
           py::arg("name"), py::arg("world_size") = 1, py::arg("world_rank") = 0, py::arg("local_size") = 0,
           py::arg("heap_bases_ptr") = 0, py::arg("local_base") = 0, py::arg("scratch_off") = 0,
           py::arg("scratch_bytes") = 0, py::arg("status_ptr") = 0, py::arg("budget_ms") = 0)
      .def("scratch_bytes_for", &NativeCommHandle::scratch_bytes_for)
      .def("all_to_all", &NativeCommHandle::all_to_all);
  m.def("native_codec_run", &native_codec_roundtrip_op);
  m.def("xfer", &xfer_op, py::arg("src_ptr"), py::arg("msgs"), py::arg("ctas_per_msg"), py::arg("heap_bases_ptr"),
        py::arg("flag_off"), py::arg("wait_flags_ptr"), py::arg("wait_idx"), py::arg("want"), py::arg("budget_ms"),
        py::arg("status_ptr"), py::arg("local_dst_ptr"), py::arg("len_off") = -1, py::arg("len_base") = 0);
  m.def("lz_layout", [](int64_t raw_bytes) {
    // (payload capacity per slice, byte offset of the u32 holding the code size, header bytes) of an LZ slice
    long long len_off = 0, header = 0;
    lz_slice_layout(raw_bytes, &len_off, &header);
    return std::make_tuple((int64_t)lz_payload_capacity(raw_bytes), (int64_t)len_off, (int64_t)header);
  });
  m.def("wait_flags", &wait_flags_op);
  m.def("delay", [](int64_t ns) { count_launch(1); launch_delay((unsigned long long)(ns < 0 ? 0 : ns), cur_stream()); });
  m.def("gemm_push_arrivals", &gemm_push_arrivals);
  m.def("launch_count", [] { return (long long)g_launches.load(); });

  py::class_<GemmOpts>(m, "GemmOpts")
      .def(py::init<>())
      .def_readwrite("epilogue", &GemmOpts::epilogue)
      .def_readwrite("activation", &GemmOpts::activation)
      .def_readwrite("bias", &GemmOpts::bias)
      .def_readwrite("aux", &GemmOpts::aux)
      .def_readwrite("out", &GemmOpts::out)
      .def_readwrite("gate_flags_ptr", &GemmOpts::gate_flags_ptr)
      .def_readwrite("gate_rows", &GemmOpts::gate_rows)
      .def_readwrite("gate_want", &GemmOpts::gate_want)
      .def_readwrite("gate_want_ptr", &GemmOpts::gate_want_ptr)
      .def_readwrite("gate_mode", &GemmOpts::gate_mode)
      .def_readwrite("gate_nblk", &GemmOpts::gate_nblk)
      .def_readwrite("perm_w", &GemmOpts::perm_w)
      .def_readwrite("perm_seg_rows", &GemmOpts::perm_seg_rows)
      .def_readwrite("perm_local_first", &GemmOpts::perm_local_first)
      .def_readwrite("copy_nblk", &GemmOpts::copy_nblk)
      .def_readwrite("trace_ptr", &GemmOpts::trace_ptr)
      .def_readwrite("dq_ptr", &GemmOpts::dq_ptr)
      .def_readwrite("dq_arrival_ptr", &GemmOpts::dq_arrival_ptr)
      .def_readwrite("dq_ready_ptr", &GemmOpts::dq_ready_ptr)
      .def_readwrite("heap_bases_ptr", &GemmOpts::heap_bases_ptr)
      .def_readwrite("push_data_off", &GemmOpts::push_data_off)
      .def_readwrite("push_flag_off", &GemmOpts::push_flag_off)
      .def_readwrite("push_rows", &GemmOpts::push_rows)
      .def_readwrite("push_C", &GemmOpts::push_C)
      .def_readwrite("push_c0", &GemmOpts::push_c0)
      .def_readwrite("push_chunk", &GemmOpts::push_chunk)
      .def_readwrite("push_q8", &GemmOpts::push_q8)
      .def_readwrite("push_scale_off", &GemmOpts::push_scale_off)
      .def_readwrite("W", &GemmOpts::W)
      .def_readwrite("my_rank", &GemmOpts::my_rank)
      .def_readwrite("chunk_groups", &GemmOpts::chunk_groups)
      .def_readwrite("budget_ms", &GemmOpts::budget_ms)
      .def_readwrite("status_ptr", &GemmOpts::status_ptr)
      .def_readwrite("max_ctas", &GemmOpts::max_ctas)
      .def_readwrite("cta_group", &GemmOpts::cta_group)
      .def_readwrite("heap_bases_host", &GemmOpts::heap_bases_host)
      .def_readwrite("copy_x", &GemmOpts::copy_x)
      .def_readwrite("copy_slot_map", &GemmOpts::copy_slot_map)
      .def_readwrite("copy_gates", &GemmOpts::copy_gates)
      .def_readwrite("copy_K", &GemmOpts::copy_K)
      .def_readwrite("copy_E_local", &GemmOpts::copy_E_local)
      .def_readwrite("copy_C", &GemmOpts::copy_C)
      .def_readwrite("copy_chunks", &GemmOpts::copy_chunks)
      .def_readwrite("copy_ctas", &GemmOpts::copy_ctas)
      .def_readwrite("copy_data_off", &GemmOpts::copy_data_off)
      .def_readwrite("copy_flag_off", &GemmOpts::copy_flag_off);
  m.def("gemm_grid_ctas", &gemm_grid_ctas, py::arg("groups"), py::arg("M"), py::arg("N"), py::arg("max_ctas") = 0,
        py::arg("cta_group") = 0);
  m.def("grouped_gemm", &grouped_gemm_op);
  m.def("tensor_from_ptr", [](int64_t ptr, int64_t nbytes, int64_t device) {
    return torch::from_blob(reinterpret_cast<void*>(ptr), {nbytes},
                            torch::TensorOptions().dtype(at::kByte).device(at::kCUDA, device));
  });

  bind_symm_heap(m);
  bind_jit(m);
}
