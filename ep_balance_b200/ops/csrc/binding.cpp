// Python bindings.  Kernels take raw device pointers; tensors are only unwrapped here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <pybind11/stl.h>

#include <cmath>
#include <map>
#include <string>

#include "grouped_gemm.h"
#include "grouped_gemm_fp8.h"
#include "onesided.h"
#include "optim.h"
#include "route.h"
#include "router.h"
#include "runtime.h"
#include "solver.h"

namespace py = pybind11;
using epb::LayerConfig;
using epb::MoeRuntime;

namespace {

cudaStream_t current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void cuda_check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}

template <typename T>
T* dptr(const torch::Tensor& t, const char* name, c10::ScalarType st) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.scalar_type() == st, name, " has the wrong dtype");
  return reinterpret_cast<T*>(t.data_ptr());
}

int get_int(const py::dict& d, const char* key, int fallback) {
  return d.contains(key) ? d[key].cast<int>() : fallback;
}

LayerConfig config_from_dict(const py::dict& d) {
  LayerConfig c;
  c.R = get_int(d, "R", 1);
  c.me = get_int(d, "me", 0);
  c.E = get_int(d, "E", 0);
  c.H = get_int(d, "H", 0);
  c.F = get_int(d, "F", 0);
  c.topk = get_int(d, "topk", 1);
  c.w_slots = get_int(d, "w_slots", 0);
  c.home_cap = get_int(d, "home_cap", 0);
  c.n_slot_plan = get_int(d, "n_slot_plan", 0);
  c.row_capacity = get_int(d, "row_capacity", 0);
  c.max_units = get_int(d, "max_units", 0);
  c.D = get_int(d, "D", 1);
  c.u_min = get_int(d, "u_min", 1);
  c.iters = get_int(d, "iters", 64);
  c.patience = get_int(d, "patience", 8);
  c.allow_cross = get_int(d, "allow_cross", 1);
  c.probe = get_int(d, "probe", 0);
  c.accum_fp32 = get_int(d, "accum_fp32", 0);
  c.s_tok = d.contains("s_tok") ? d["s_tok"].cast<int64_t>() : 0;
  c.num_sms = get_int(d, "num_sms", 148);
  c.multi_rank_sync = get_int(d, "multi_rank_sync", 1);
  c.gemm_ctas = get_int(d, "gemm_ctas", 2);
  c.fused_comm = get_int(d, "fused_comm", 1);
  c.comm_block_rows = get_int(d, "comm_block_rows", 0);
  c.wait_ms = get_int(d, "wait_ms", 1500);
  return c;
}

// Stand-alone solve on tensors (the library API path).  All tensors live on the same device.
void solve_plan(torch::Tensor omega, torch::Tensor dom, torch::Tensor cost, torch::Tensor main_rank,
                torch::Tensor weight_bytes, int64_t s_tok, int64_t D, int64_t n_slot, int64_t u_min, int64_t iters,
                int64_t patience, bool allow_cross, bool probe, torch::Tensor x, torch::Tensor q, torch::Tensor erl,
                torch::Tensor rank_load, torch::Tensor slot_used, torch::Tensor stuck, torch::Tensor theta,
                torch::Tensor control, torch::Tensor sync, torch::Tensor status) {
  const c10::cuda::CUDAGuard guard(omega.device());
  epb::SolverParams p{};
  p.omega = dptr<const int32_t>(omega, "omega", torch::kInt32);
  p.dom = dptr<const int32_t>(dom, "dom", torch::kInt32);
  p.cost = dptr<const int32_t>(cost, "cost", torch::kInt32);
  p.main_rank = dptr<const int32_t>(main_rank, "main_rank", torch::kInt32);
  p.weight_bytes = dptr<const int64_t>(weight_bytes, "weight_bytes", torch::kInt64);
  p.s_tok = s_tok;
  p.R = (int)omega.size(0);
  p.E = (int)omega.size(1);
  TORCH_CHECK(p.R >= 1 && p.R <= 1024, "device solver requires 1 <= R <= 1024");
  TORCH_CHECK(p.E >= 1, "device solver requires E > 0");
  TORCH_CHECK(D >= 1 && D <= p.R, "device solver requires 1 <= num_domains <= R");
  TORCH_CHECK(n_slot > 0 && u_min > 0 && iters > 0 && patience > 0, "solver knobs must be positive");
  p.D = (int)D;
  p.n_slot = (int)n_slot;
  p.u_min = (int)u_min;
  p.iters = (int)iters;
  p.patience = (int)patience;
  p.allow_cross = allow_cross ? 1 : 0;
  p.probe = probe ? 1 : 0;
  p.x = dptr<int8_t>(x, "x", torch::kInt8);
  p.q = dptr<int32_t>(q, "q", torch::kInt32);
  p.erl = dptr<int32_t>(erl, "erl", torch::kInt32);
  p.rank_load = dptr<int32_t>(rank_load, "rank_load", torch::kInt32);
  p.slot_used = dptr<int32_t>(slot_used, "slot_used", torch::kInt32);
  p.stuck = dptr<unsigned char>(stuck, "stuck", torch::kUInt8);
  p.theta = dptr<int64_t>(theta, "theta", torch::kInt64);
  p.control = dptr<int64_t>(control, "control", torch::kInt64);
  p.trace = control.numel() >= 16 ? p.control + 8 : nullptr;  // a control tensor of 16 words also receives phase timestamps
  p.sync = reinterpret_cast<unsigned*>(dptr<int32_t>(sync, "sync", torch::kInt32));
  p.status = dptr<int>(status, "status", torch::kInt32);
  epb::RankTables t{};
  t.me = -1;
  cuda_check(epb::launch_solver(p, t, current_stream()), "launch_solver");
}

// Stand-alone grouped GEMM on tensors (tests and generic use).
//   mode kPlain/kFwd2: C[T, N] = A[T, K] . W[slot]^T with W [S, N, K]
//   mode kFwd1:        h[T, 2N], act[T, N] from A[T, K], W [S, 2N, K]
//   mode kDgrad1:      C[T, N] = A[T, K] . W[slot] with W [S, K, N]
//   mode kDgrad2:      h[T, 2N] updated in place from A = dY[T, K], W [S, K, N]
//   mode kWgrad:       out[S, M_out, N] = P[T, M_out]^T Q[T, N] per group
void grouped_gemm(int64_t mode, torch::Tensor a, torch::Tensor b, torch::Tensor out0, c10::optional<torch::Tensor> out1,
                  torch::Tensor group_off, torch::Tensor group_rows, torch::Tensor group_wslot, torch::Tensor totals,
                  torch::Tensor status, int64_t num_sms, int64_t ctas) {
  const c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(ctas == 1 || ctas == 2, "ctas must be 1 or 2");
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16, "bf16 operands only");
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && out0.is_contiguous(), "operands must be contiguous");
  epb::GemmArgs g{};
  g.mode = (int)mode;
  g.ctas = (int)ctas;
  g.group_off = dptr<const int32_t>(group_off, "group_off", torch::kInt32);
  g.group_rows = dptr<const int32_t>(group_rows, "group_rows", torch::kInt32);
  g.group_wslot = dptr<const int32_t>(group_wslot, "group_wslot", torch::kInt32);
  g.totals = dptr<const int32_t>(totals, "totals", torch::kInt32);
  g.n_groups_cap = (int)group_rows.size(0);
  g.row_capacity = (int)a.size(0);
  g.status = dptr<int>(status, "status", torch::kInt32);
  g.out0 = out0.data_ptr();
  g.out1 = out1.has_value() ? out1->data_ptr() : nullptr;
  CUtensorMap tmA, tmB;
  const uint64_t T = a.size(0);
  bool ok = true;
  switch (mode) {
    case epb::kPlain:
    case epb::kFwd2:
      g.N = (int)b.size(1);
      g.K = (int)a.size(1);
      ok = epb::make_tmap_2d(&tmA, a.data_ptr(), T, a.size(1), 64, 128) &&
           epb::make_tmap_3d(&tmB, b.data_ptr(), b.size(0), b.size(1), b.size(2), 64, 128);
      break;
    case epb::kFwd1:
      g.N = (int)b.size(1) / 2;
      g.K = (int)a.size(1);
      ok = epb::make_tmap_2d(&tmA, a.data_ptr(), T, a.size(1), 64, 128) &&
           epb::make_tmap_3d(&tmB, b.data_ptr(), b.size(0), b.size(1), b.size(2), 64, 128);
      break;
    case epb::kDgrad1:
    case epb::kDgrad2:
      g.N = (int)b.size(2);
      g.K = (int)a.size(1);
      ok = epb::make_tmap_2d(&tmA, a.data_ptr(), T, a.size(1), 64, 128) &&
           epb::make_tmap_3d(&tmB, b.data_ptr(), b.size(0), b.size(1), b.size(2), 64, 64);
      break;
    case epb::kWgrad:
      g.N = (int)b.size(1);
      g.M_out = (int)a.size(1);
      ok = epb::make_tmap_2d(&tmA, a.data_ptr(), T, a.size(1), 64, 64) &&
           epb::make_tmap_2d(&tmB, b.data_ptr(), b.size(0), b.size(1), 64, 64);
      break;
    default:
      TORCH_CHECK(false, "unknown grouped GEMM mode");
  }
  TORCH_CHECK(ok, "cuTensorMapEncodeTiled failed");
  cuda_check(epb::launch_grouped_gemm(tmA, tmB, g, (int)num_sms, current_stream()), "launch_grouped_gemm");
}

// In-place AdamW step on one tensor (param, grad and both moments share dtype and shape).
void adamw_step(torch::Tensor param, torch::Tensor grad, torch::Tensor exp_avg, torch::Tensor exp_avg_sq, double lr,
                double beta1, double beta2, double eps, double weight_decay, int64_t step,
                c10::optional<torch::Tensor> step_tensor, c10::optional<torch::Tensor> status_guard) {
  const c10::cuda::CUDAGuard guard(param.device());
  TORCH_CHECK(param.is_contiguous() && grad.is_contiguous() && exp_avg.is_contiguous() && exp_avg_sq.is_contiguous(),
              "adamw_step needs contiguous tensors");
  const bool grad_f32 = param.scalar_type() == torch::kBFloat16 && grad.scalar_type() == torch::kFloat32;
  TORCH_CHECK((param.scalar_type() == grad.scalar_type() || grad_f32) && param.scalar_type() == exp_avg.scalar_type() &&
                  param.scalar_type() == exp_avg_sq.scalar_type(),
              "adamw_step: moments share the parameter dtype; the gradient does too, or is fp32 for a bf16 parameter");
  TORCH_CHECK(param.scalar_type() == torch::kBFloat16 || param.scalar_type() == torch::kFloat32, "bf16 or fp32 only");
  TORCH_CHECK(grad.numel() == param.numel() && exp_avg.numel() == param.numel() && exp_avg_sq.numel() == param.numel(),
              "adamw_step size mismatch");
  epb::AdamArgs a{};
  a.param = param.data_ptr();
  a.grad = grad.data_ptr();
  a.exp_avg = exp_avg.data_ptr();
  a.exp_avg_sq = exp_avg_sq.data_ptr();
  a.numel = (size_t)param.numel();
  a.lr = (float)lr;
  a.beta1 = (float)beta1;
  a.beta2 = (float)beta2;
  a.eps = (float)eps;
  a.weight_decay = (float)weight_decay;
  a.bias_correction1 = (float)(1.0 - std::pow(beta1, (double)step));
  a.bias_correction2_sqrt = (float)std::sqrt(1.0 - std::pow(beta2, (double)step));
  a.is_bf16 = param.scalar_type() == torch::kBFloat16 ? 1 : 0;
  a.grad_f32 = grad_f32 ? 1 : 0;
  a.step_ptr = nullptr;
  if (step_tensor.has_value() && step_tensor->defined())
    a.step_ptr = dptr<int64_t>(*step_tensor, "step_tensor", torch::kInt64);
  a.guard = nullptr;
  a.guard_rows = 0;
  if (status_guard.has_value() && status_guard->defined()) {
    TORCH_CHECK(status_guard->dim() == 2 && status_guard->size(1) == 4 && status_guard->device() == param.device(),
                "guard must be an int32 [n, 4] tensor of status words on the parameter's device");
    a.guard = dptr<int>(*status_guard, "guard", torch::kInt32);
    a.guard_rows = (int)status_guard->size(0);
  }
  cuda_check(epb::launch_adamw(a, current_stream()), "launch_adamw");
}

void wait_probe(torch::Tensor flag, int64_t target, int64_t budget_ns, torch::Tensor status) {
  const c10::cuda::CUDAGuard guard(flag.device());
  cuda_check(epb::launch_wait_probe(reinterpret_cast<const unsigned*>(dptr<int32_t>(flag, "flag", torch::kInt32)),
                                    (unsigned)target, (unsigned long long)budget_ns,
                                    dptr<int>(status, "status", torch::kInt32), current_stream()),
             "launch_wait_probe");
}

// ---- one-sided transfers over peer-mapped windows (descriptors: int64 [K, 4] on the device)
void copy_batched(bool is_put, torch::Tensor desc, torch::Tensor window_ptrs, uint64_t local_base, bool use_bulk,
                  int64_t blocks_per_desc, torch::Tensor status) {
  const c10::cuda::CUDAGuard guard(desc.device());
  TORCH_CHECK(desc.dim() == 2 && desc.size(1) == 4, "descriptors must be int64 [K, 4]");
  epb::BatchedCopyArgs a{};
  a.desc = reinterpret_cast<const epb::CopyDesc*>(dptr<int64_t>(desc, "desc", torch::kInt64));
  a.K = (int)desc.size(0);
  a.window_ptrs = reinterpret_cast<uint8_t* const*>(dptr<int64_t>(window_ptrs, "window_ptrs", torch::kInt64));
  a.R = (int)window_ptrs.numel();
  a.local_base = reinterpret_cast<uint8_t*>(static_cast<uintptr_t>(local_base));
  a.use_bulk = use_bulk ? 1 : 0;
  a.status = dptr<int>(status, "status", torch::kInt32);
  cuda_check(is_put ? epb::launch_put_batched(a, (int)blocks_per_desc, current_stream())
                    : epb::launch_get_batched(a, (int)blocks_per_desc, current_stream()),
             is_put ? "launch_put_batched" : "launch_get_batched");
}
void get_batched(torch::Tensor desc, torch::Tensor window_ptrs, uint64_t local_base, bool use_bulk,
                 int64_t blocks_per_desc, torch::Tensor status) {
  copy_batched(false, desc, window_ptrs, local_base, use_bulk, blocks_per_desc, status);
}
void put_batched(torch::Tensor desc, torch::Tensor window_ptrs, uint64_t local_base, bool use_bulk,
                 int64_t blocks_per_desc, torch::Tensor status) {
  copy_batched(true, desc, window_ptrs, local_base, use_bulk, blocks_per_desc, status);
}
void signal_peers(torch::Tensor signal_ptrs, int64_t peer, int64_t idx, int64_t value) {
  const c10::cuda::CUDAGuard guard(signal_ptrs.device());
  cuda_check(epb::launch_signal(reinterpret_cast<unsigned* const*>(dptr<int64_t>(signal_ptrs, "signal_ptrs", torch::kInt64)),
                                (int)signal_ptrs.numel(), (int)peer, (int)idx, (unsigned)value, current_stream()),
             "launch_signal");
}
void wait_signal(uint64_t word, int64_t expected, int64_t idx, int64_t budget_ns, torch::Tensor status) {
  const c10::cuda::CUDAGuard guard(status.device());
  cuda_check(epb::launch_wait_signal(reinterpret_cast<const unsigned*>(static_cast<uintptr_t>(word)), (unsigned)expected,
                                     (int)idx, (unsigned long long)budget_ns, dptr<int>(status, "status", torch::kInt32),
                                     current_stream()),
             "launch_wait_signal");
}
void symm_barrier(torch::Tensor signal_ptrs, int64_t slot, int64_t me, torch::Tensor epoch_word, torch::Tensor status) {
  const c10::cuda::CUDAGuard guard(signal_ptrs.device());
  cuda_check(epb::launch_symm_barrier(reinterpret_cast<unsigned* const*>(dptr<int64_t>(signal_ptrs, "signal_ptrs", torch::kInt64)),
                                      (int)slot, (int)signal_ptrs.numel(), (int)me,
                                      reinterpret_cast<unsigned*>(dptr<int32_t>(epoch_word, "epoch_word", torch::kInt32)),
                                      dptr<int>(status, "status", torch::kInt32), current_stream()),
             "launch_symm_barrier");
}

// Owner-side gradient return over explicit tables (the library path's symmetric weight channel).
void grad_reduce(torch::Tensor g_ptrs, int64_t elems_per_slot, torch::Tensor slot_of, torch::Tensor main_rank,
                 torch::Tensor home_index, int64_t me, int64_t home_cap, torch::Tensor accum, bool include_self,
                 bool overwrite) {
  const c10::cuda::CUDAGuard guard(g_ptrs.device());
  epb::GradReduceArgs a{};
  a.g_ptrs = reinterpret_cast<void* const*>(dptr<int64_t>(g_ptrs, "g_ptrs", torch::kInt64));
  a.elems_per_slot = (size_t)elems_per_slot;
  a.slot_of = dptr<int32_t>(slot_of, "slot_of", torch::kInt32);
  a.main_rank = dptr<int32_t>(main_rank, "main_rank", torch::kInt32);
  a.home_index = dptr<int32_t>(home_index, "home_index", torch::kInt32);
  a.E = (int)main_rank.numel();
  a.R = (int)g_ptrs.numel();
  TORCH_CHECK(slot_of.numel() == (int64_t)a.E * a.R, "slot_of must be [E, R]");
  a.me = (int)me;
  a.home_cap = (int)home_cap;
  TORCH_CHECK(accum.is_cuda() && accum.is_contiguous(), "accum must be a contiguous CUDA tensor");
  TORCH_CHECK(accum.scalar_type() == torch::kFloat32 || accum.scalar_type() == torch::kBFloat16, "accum: fp32 or bf16");
  TORCH_CHECK(accum.numel() == home_cap * elems_per_slot, "accum must be [home_cap, elems_per_slot]");
  a.accum = accum.data_ptr();
  a.accum_fp32 = accum.scalar_type() == torch::kFloat32 ? 1 : 0;
  a.include_self = include_self ? 1 : 0;
  a.overwrite = overwrite ? 1 : 0;
  cuda_check(epb::launch_grad_reduce(a, current_stream()), "launch_grad_reduce");
}

// ---- block-scaled fp8 grouped GEMM and its quantisers
void quantize_rows(torch::Tensor x, torch::Tensor q, torch::Tensor sfa) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && q.dim() == 2 && q.sizes() == x.sizes(), "x and q must be [rows, K]");
  const int rows = (int)x.size(0), K = (int)x.size(1);
  TORCH_CHECK(rows % 128 == 0 && K % 128 == 0, "rows and K must be multiples of 128");
  TORCH_CHECK(sfa.numel() == (int64_t)(rows / 128) * ((K / 128 + 3) / 4) * 512, "sfa has the wrong size");
  cuda_check(epb::launch_quantize_rows(dptr<void>(x, "x", torch::kBFloat16), dptr<uint8_t>(q, "q", torch::kUInt8),
                                       dptr<uint8_t>(sfa, "sfa", torch::kUInt8), rows, K, nullptr, current_stream()),
             "launch_quantize_rows");
}
void quantize_weights(torch::Tensor w, torch::Tensor q, torch::Tensor sfb) {
  const c10::cuda::CUDAGuard guard(w.device());
  TORCH_CHECK(w.dim() == 3 && q.sizes() == w.sizes(), "w and q must be [slots, N, K]");
  const int S = (int)w.size(0), N = (int)w.size(1), K = (int)w.size(2);
  TORCH_CHECK(N % 128 == 0 && K % 128 == 0, "N and K must be multiples of 128");
  TORCH_CHECK(sfb.numel() == (int64_t)S * (N / 128) * ((K / 128 + 3) / 4) * 512, "sfb has the wrong size");
  cuda_check(epb::launch_quantize_weights(dptr<void>(w, "w", torch::kBFloat16), dptr<uint8_t>(q, "q", torch::kUInt8),
                                          dptr<uint8_t>(sfb, "sfb", torch::kUInt8), S, N, K, current_stream()),
             "launch_quantize_weights");
}
void grouped_gemm_fp8(torch::Tensor aq, torch::Tensor sfa, torch::Tensor bq, torch::Tensor sfb, torch::Tensor out,
                      torch::Tensor group_off, torch::Tensor group_rows, torch::Tensor group_wslot, torch::Tensor totals,
                      torch::Tensor status, int64_t num_sms, int64_t ctas) {
  const c10::cuda::CUDAGuard guard(aq.device());
  TORCH_CHECK(aq.dim() == 2 && bq.dim() == 3 && out.dim() == 2, "aq [T, K], bq [slots, N, K], out [T, N]");
  const int64_t T = aq.size(0), K = aq.size(1), N = bq.size(1);
  TORCH_CHECK(bq.size(2) == K && out.size(0) == T && out.size(1) == N, "shape mismatch");
  TORCH_CHECK(T % 128 == 0 && K % 128 == 0 && N % 128 == 0, "T, K and N must be multiples of 128");
  const int64_t kgroups = (K / 128 + 3) / 4;
  TORCH_CHECK(sfa.numel() == (T / 128) * kgroups * 512, "sfa has the wrong size");
  TORCH_CHECK(sfb.numel() == bq.size(0) * (N / 128) * kgroups * 512, "sfb has the wrong size");
  epb::Fp8GemmArgs g{};
  g.group_off = dptr<int32_t>(group_off, "group_off", torch::kInt32);
  g.group_rows = dptr<int32_t>(group_rows, "group_rows", torch::kInt32);
  g.group_wslot = dptr<int32_t>(group_wslot, "group_wslot", torch::kInt32);
  g.totals = dptr<int32_t>(totals, "totals", torch::kInt32);
  g.n_groups_cap = (int)group_rows.numel();
  g.row_capacity = (int)T;
  g.N = (int)N;
  g.K = (int)K;
  g.sfa = dptr<uint8_t>(sfa, "sfa", torch::kUInt8);
  g.sfb = dptr<uint8_t>(sfb, "sfb", torch::kUInt8);
  g.out = dptr<void>(out, "out", torch::kBFloat16);
  g.status = dptr<int>(status, "status", torch::kInt32);
  CUtensorMap tmA, tmB;
  TORCH_CHECK(epb::make_tmap_fp8_2d(&tmA, dptr<uint8_t>(aq, "aq", torch::kUInt8), T, K) &&
                  epb::make_tmap_fp8_3d(&tmB, dptr<uint8_t>(bq, "bq", torch::kUInt8), bq.size(0), N, K,
                                        ctas == 2 ? (N % 256 == 0 ? 128 : 64) : 128),
              "cuTensorMapEncodeTiled failed");
  if (ctas == 2) {
    TORCH_CHECK(T % 256 == 0, "the CTA-pair kernel needs T % 256 == 0 and groups that start on multiples of 256 rows");
    CUtensorMap tmSFA, tmSFB;
    TORCH_CHECK(epb::make_tmap_sf(&tmSFA, g.sfa, (uint64_t)(sfa.numel() / 512)) &&
                    epb::make_tmap_sf(&tmSFB, g.sfb, (uint64_t)(sfb.numel() / 512)),
                "cuTensorMapEncodeTiled (scale chunks) failed");
    cuda_check(epb::launch_grouped_gemm_fp8_pair(tmA, tmB, tmSFA, tmSFB, g, (int)num_sms, current_stream()),
               "launch_grouped_gemm_fp8_pair");
    return;
  }
  cuda_check(epb::launch_grouped_gemm_fp8(tmA, tmB, g, (int)num_sms, current_stream()), "launch_grouped_gemm_fp8");
}

// Fused inference router: logits [N, E] -> (expert ids int64 [N, K], gate weights fp32 [N, K]).
void router_topk(torch::Tensor logits, c10::optional<torch::Tensor> bias, int64_t mode, int64_t n_groups,
                 int64_t topk_groups, double scale, torch::Tensor idx, torch::Tensor weights) {
  const c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && idx.dim() == 2 && weights.sizes() == idx.sizes() && idx.size(0) == logits.size(0),
              "logits [N, E], idx/weights [N, K]");
  const float* b = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->numel() == logits.size(1), "bias must be [E]");
    b = dptr<float>(*bias, "bias", torch::kFloat32);
  }
  cuda_check(epb::launch_router_topk(dptr<float>(logits, "logits", torch::kFloat32), b, (int)logits.size(0),
                                     (int)logits.size(1), (int)idx.size(1), (int)mode, (int)n_groups, (int)topk_groups,
                                     (float)scale, dptr<int64_t>(idx, "idx", torch::kInt64),
                                     dptr<float>(weights, "weights", torch::kFloat32), current_stream()),
             "launch_router_topk");
}

// ---- symmetric heap over CUDA IPC: one cudaMalloc per rank, mapped into every peer process
py::tuple ipc_alloc(int64_t nbytes) {
  void* p = nullptr;
  cuda_check(cudaMalloc(&p, (size_t)nbytes), "cudaMalloc(symmetric heap)");
  cuda_check(cudaMemset(p, 0, (size_t)nbytes), "cudaMemset(symmetric heap)");
  cudaIpcMemHandle_t h;
  cuda_check(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle");
  return py::make_tuple((uint64_t)(uintptr_t)p, py::bytes(reinterpret_cast<const char*>(&h), sizeof(h)));
}
uint64_t ipc_open(py::bytes handle) {
  std::string raw = handle;
  TORCH_CHECK(raw.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
  cudaIpcMemHandle_t h;
  memcpy(&h, raw.data(), sizeof(h));
  void* p = nullptr;
  cuda_check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return (uint64_t)(uintptr_t)p;
}
void ipc_close(uint64_t p) { cuda_check(cudaIpcCloseMemHandle(reinterpret_cast<void*>((uintptr_t)p)), "cudaIpcCloseMemHandle"); }
void ipc_free(uint64_t p) { cuda_check(cudaFree(reinterpret_cast<void*>((uintptr_t)p)), "cudaFree"); }
torch::Tensor tensor_from_ptr(uint64_t p, int64_t nbytes, int64_t device) {
  auto opts = torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, (int)device);
  return torch::from_blob(reinterpret_cast<void*>((uintptr_t)p), {nbytes}, [](void*) {}, opts);
}

const void* cp(uint64_t a) { return reinterpret_cast<const void*>(static_cast<uintptr_t>(a)); }
void* mp(uint64_t a) { return reinterpret_cast<void*>(static_cast<uintptr_t>(a)); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "ep_balance_b200 native kernels (sm_100a)";
  m.def("solve_plan", &solve_plan);
  m.def("grouped_gemm", &grouped_gemm);
  m.def("wait_probe", &wait_probe);
  m.def("adamw_step", &adamw_step, py::arg("param"), py::arg("grad"), py::arg("exp_avg"), py::arg("exp_avg_sq"),
        py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("weight_decay"), py::arg("step"),
        py::arg("step_tensor") = py::none(), py::arg("guard") = py::none());
  m.def("get_batched", &get_batched);
  m.def("put_batched", &put_batched);
  m.def("signal_peers", &signal_peers);
  m.def("wait_signal", &wait_signal);
  m.def("symm_barrier", &symm_barrier);
  m.def("grad_reduce", &grad_reduce);
  m.def("router_topk", &router_topk);
  m.def("quantize_rows", &quantize_rows);
  m.def("quantize_weights", &quantize_weights);
  m.def("grouped_gemm_fp8", &grouped_gemm_fp8);
  m.def("ipc_alloc", &ipc_alloc);
  m.def("ipc_open", &ipc_open);
  m.def("ipc_close", &ipc_close);
  m.def("ipc_free", &ipc_free);
  m.def("tensor_from_ptr", &tensor_from_ptr);

  py::class_<MoeRuntime>(m, "MoeRuntime")
      .def(py::init([](const py::dict& cfg, const std::map<std::string, uint64_t>& ptrs) {
        return new MoeRuntime(config_from_dict(cfg), ptrs);
      }))
      .def("launches", &MoeRuntime::launches)
      .def("enable_timing", &MoeRuntime::enable_timing)
      .def("phase_times", &MoeRuntime::phase_times)
      .def("reset_launches", &MoeRuntime::reset_launches)
      .def("publish", [](MoeRuntime& r, uint64_t idx, int u) { r.publish((const int64_t*)cp(idx), u, current_stream()); })
      .def("solve", [](MoeRuntime& r) { r.solve(current_stream()); })
      .def("route", [](MoeRuntime& r, uint64_t idx, int u) { r.route((const int64_t*)cp(idx), u, current_stream()); })
      .def("dispatch_tokens", [](MoeRuntime& r, uint64_t tok, uint64_t prob, int u) {
        r.dispatch_tokens(cp(tok), (const float*)cp(prob), u, current_stream());
      })
      .def("pull_weights", [](MoeRuntime& r) { r.pull_weights(current_stream()); })
      .def("barrier", [](MoeRuntime& r, int slot) { r.barrier(slot, current_stream()); })
      .def("gemm1", [](MoeRuntime& r) { r.gemm1(current_stream()); })
      .def("gemm2", [](MoeRuntime& r) { r.gemm2(current_stream()); })
      .def("gemm1_fused", [](MoeRuntime& r, uint64_t tok, uint64_t prob, int u) {
        r.gemm1_fused(cp(tok), (const float*)cp(prob), u, current_stream());
      })
      .def("dgrad2_fused", [](MoeRuntime& r, uint64_t dout, int u) { r.dgrad2_fused(cp(dout), u, current_stream()); })
      .def("trace_launches", &MoeRuntime::trace_launches)
      .def("launch_log", [](const MoeRuntime& r) { return r.launch_log(); })
      .def("reduce_out", [](MoeRuntime& r, uint64_t out, int n, bool wait_peers, uint64_t unit_scale) {
        r.reduce_out(mp(out), n, current_stream(), wait_peers, (const float*)cp(unit_scale));
      }, py::arg("out"), py::arg("n"), py::arg("wait_peers") = false, py::arg("unit_scale") = 0)
      .def("dispatch_grads", [](MoeRuntime& r, uint64_t dout, int u) { r.dispatch_grads(cp(dout), u, current_stream()); })
      .def("wgrad2", [](MoeRuntime& r) { r.wgrad2(current_stream()); })
      .def("dgrad2", [](MoeRuntime& r) { r.dgrad2(current_stream()); })
      .def("wgrad1", [](MoeRuntime& r) { r.wgrad1(current_stream()); })
      .def("dgrad1", [](MoeRuntime& r) { r.dgrad1(current_stream()); })
      .def("reduce_dtokens", [](MoeRuntime& r, uint64_t dt, uint64_t dprob, int n, bool wait_peers) {
        r.reduce_dtokens(mp(dt), (float*)mp(dprob), n, current_stream(), wait_peers);
      }, py::arg("dtokens"), py::arg("dprob"), py::arg("n"), py::arg("wait_peers") = false)
      .def("reduce_weight_grads", [](MoeRuntime& r) { r.reduce_weight_grads(current_stream()); })
      .def("has_fp8", &MoeRuntime::has_fp8)
      .def("quantize_own_weights", [](MoeRuntime& r) { r.quantize_own_weights(current_stream()); })
      .def("pull_weights_fp8", [](MoeRuntime& r) { r.pull_weights_fp8(current_stream()); })
      .def("dispatch_fp8", [](MoeRuntime& r, uint64_t tok, int u) { r.dispatch_fp8(cp(tok), u, current_stream()); })
      .def("gemm1_fp8", [](MoeRuntime& r) { r.gemm1_fp8(current_stream()); })
      .def("act_fp8", [](MoeRuntime& r) { r.act_fp8(current_stream()); })
      .def("gemm2_fp8", [](MoeRuntime& r) { r.gemm2_fp8(current_stream()); })
      .def("forward_fp8", [](MoeRuntime& r, uint64_t tok, uint64_t idx, uint64_t prob, uint64_t out, int n) {
        r.forward_fp8(cp(tok), (const int64_t*)cp(idx), (const float*)cp(prob), mp(out), n, current_stream());
      })
      .def("forward", [](MoeRuntime& r, uint64_t tok, uint64_t idx, uint64_t prob, uint64_t out, int n) {
        r.forward(cp(tok), (const int64_t*)cp(idx), (const float*)cp(prob), mp(out), n, current_stream());
      })
      .def("backward", [](MoeRuntime& r, uint64_t dout, uint64_t dtok, uint64_t dprob, int n) {
        r.backward(cp(dout), mp(dtok), (float*)mp(dprob), n, current_stream());
      });
}
