// MoeRuntime: wires one layer's buffers into the solver, routing and grouped-GEMM kernels.
//
// Forward:  count+publish -> solve -> route -> [dispatch + replica pull + GEMM1, one kernel] -> GEMM2
// (rows stored to their source ranks, completion signalled to every peer by the last CTA) ->
// reduce_out (waits in the kernel for the peers' signals).
// Backward: [gradient dispatch + Dgrad2, one kernel] -> SwiGLU-gradient pass (applies the gate weight, stores
// the gate-weight gradients to the units' source ranks) -> Wgrad2 -> Wgrad1 -> Dgrad1 (rows stored to
// sources, completion signalled) -> reduce_dtokens (waits); beside
// Dgrad1, on the runtime's side stream: cross-rank barrier -> owners add their replicas' weight gradients.
// There is no stand-alone barrier on the critical path: consumers of transferred rows wait per M-tile
// on arrival counters that the senders advance, consumers of combined rows on one signal per peer.
// Inference with fp8 experts: publish -> solve -> route -> dispatch fused with the 1 x 128 quantisation ->
// fp8 replica pull -> [barrier] -> fp8 gemm1 -> SwiGLU + quantise -> fp8 gemm2 (scattered) -> [barrier] -> reduce_out.
// This is the schedule the reference drives from Python over NCCL on three streams
// (eplb_manager.py:710-886, 905-1167, manual_block.py:127-367, overlap.py:257-328), restated as
// device-side kernels that overlap transfer and compute tile by tile.
#include "runtime.h"

#include <stdexcept>

namespace epb {

template <typename T>
T* MoeRuntime::ptr(const char* name, bool required) const {
  auto it = ptrs_.find(name);
  if (it == ptrs_.end() || it->second == 0) {
    if (required) throw std::runtime_error(std::string("MoeRuntime: missing device pointer '") + name + "'");
    return nullptr;
  }
  return reinterpret_cast<T*>(static_cast<uintptr_t>(it->second));
}

void MoeRuntime::check(cudaError_t e, const char* what) {
  ++launches_;
  if (trace_) launch_log_.emplace_back(on_side_ ? std::string("side:") + what : std::string(what));
  if (e != cudaSuccess) throw std::runtime_error(std::string("MoeRuntime: ") + what + ": " + cudaGetErrorString(e));
}

MoeRuntime::~MoeRuntime() {
  for (auto& m : marks_) cudaEventDestroy(m.second);
  if (ev_fork_) cudaEventDestroy(ev_fork_);
  if (ev_join_) cudaEventDestroy(ev_join_);
  if (side_) cudaStreamDestroy(side_);
}

void MoeRuntime::tmap2(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t bc, uint32_t br) {
  if (!make_tmap_2d(m, base, rows, cols, bc, br)) throw std::runtime_error("MoeRuntime: cuTensorMapEncodeTiled (2-D) failed");
}
void MoeRuntime::tmap3(CUtensorMap* m, const void* base, uint64_t slots, uint64_t rows, uint64_t cols, uint32_t bc,
                       uint32_t br) {
  if (!make_tmap_3d(m, base, slots, rows, cols, bc, br)) throw std::runtime_error("MoeRuntime: cuTensorMapEncodeTiled (3-D) failed");
}

MoeRuntime::MoeRuntime(const LayerConfig& cfg, const std::map<std::string, uint64_t>& ptrs) : cfg_(cfg), ptrs_(ptrs) {
  const LayerConfig& c = cfg_;
  if (c.H % 64 || c.F % 128) throw std::runtime_error("MoeRuntime: need H % 64 == 0 and F % 128 == 0");
  if (c.gemm_ctas != 1 && c.gemm_ctas != 2) throw std::runtime_error("MoeRuntime: gemm_ctas must be 1 or 2");
  if (c.row_capacity % (128 * c.gemm_ctas)) throw std::runtime_error("MoeRuntime: row_capacity must be a multiple of the GEMM M tile");
  if (c.R > 64) throw std::runtime_error("MoeRuntime: the fused layer supports at most 64 expert-parallel ranks (gradient-return host lists)");
  tile_rows_ = 128 * c.gemm_ctas;
  n_tiles_ = c.row_capacity / tile_rows_;
  block_rows_ = c.comm_block_rows;
  if (block_rows_ <= 0) {
    block_rows_ = 32;
    while (block_rows_ * 2 <= tile_rows_ && block_rows_ * 2 <= 32 * c.R) block_rows_ *= 2;
  }
  if (block_rows_ % 32 || tile_rows_ % block_rows_) throw std::runtime_error("MoeRuntime: comm_block_rows must be a multiple of 32 that divides the GEMM M tile");
  if (c.wait_ms <= 0 || c.wait_ms > 60000) throw std::runtime_error("MoeRuntime: wait_ms must be in (0, 60000]");
  wait_ns_ = (unsigned long long)c.wait_ms * 1000000ull;
  if (c.multi_rank_sync && c.R > 1) {
    if (cudaStreamCreateWithFlags(&side_, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&ev_fork_, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&ev_join_, cudaEventDisableTiming) != cudaSuccess)
      throw std::runtime_error("MoeRuntime: could not create the side stream");
  }

  sp_.omega = ptr<const int32_t>("omega");
  sp_.dom = ptr<const int32_t>("dom");
  sp_.cost = ptr<const int32_t>("cost");
  sp_.main_rank = ptr<const int32_t>("main_rank");
  sp_.weight_bytes = ptr<const int64_t>("weight_bytes");
  sp_.s_tok = c.s_tok;
  sp_.R = c.R;
  sp_.E = c.E;
  sp_.D = c.D;
  sp_.n_slot = c.n_slot_plan;
  sp_.u_min = c.u_min;
  sp_.iters = c.iters;
  sp_.patience = c.patience;
  sp_.allow_cross = c.allow_cross;
  sp_.probe = c.probe;
  sp_.x = ptr<int8_t>("x");
  sp_.q = ptr<int32_t>("q");
  sp_.erl = ptr<int32_t>("erl");
  sp_.rank_load = ptr<int32_t>("rank_load");
  sp_.slot_used = ptr<int32_t>("slot_used");
  sp_.stuck = ptr<unsigned char>("stuck");
  sp_.theta = ptr<int64_t>("theta");
  sp_.control = ptr<int64_t>("control", false);
  sp_.sync = ptr<unsigned>("sync");
  sp_.status = ptr<int>("status");
  sp_.omega_signal = ptr<const unsigned>("signals");
  sp_.omega_epoch = ptr<const unsigned>("epochs");

  tables_.me = c.me;
  tables_.n_slot = c.w_slots;
  tables_.row_align = 128 * c.gemm_ctas;
  tables_.row_capacity = c.row_capacity;
  tables_.home_cap = c.home_cap;
  tables_.home_index = ptr<const int32_t>("home_index");
  tables_.slot_of = ptr<int32_t>("slot_of");
  tables_.row_base = ptr<int32_t>("row_base");
  tables_.group_expert = ptr<int32_t>("group_expert");
  tables_.group_wslot = ptr<int32_t>("group_wslot");
  tables_.group_off = ptr<int32_t>("group_off");
  tables_.group_rows = ptr<int32_t>("group_rows");
  tables_.totals = ptr<int32_t>("totals");
  tables_.send_off = ptr<int32_t>("send_off");
  tables_.tiles_of = ptr<int32_t>("tiles_of");
  for (const char* name : {"arrive", "arrive_ptrs", "chunk_hist", "hist_acc", "exp_prefix", "sorted_units", "unit_pos", "done_ctr", "rowp",
                           "rowp_ptrs", "dprob", "dprob_ptrs", "dact", "meta"})
    ptr<void>(name);

  const uint64_t T = c.row_capacity, H = c.H, F = c.F, S = c.w_slots;
  // K-major A operands: box {64 k, 128 rows}
  tmap2(&tm_x_k_, ptr<void>("xbuf"), T, H, 64, 128);
  tmap2(&tm_act_k_, ptr<void>("act"), T, F, 64, 128);
  tmap2(&tm_dy_k_, ptr<void>("dybuf"), T, H, 64, 128);
  tmap2(&tm_dh_k_, ptr<void>("hbuf"), T, 2 * F, 64, 128);
  // weights, K-major B: box {64 k, 128 n, 1}
  tmap3(&tm_w1_k_, ptr<void>("w1"), S, 2 * F, H, 64, 128);
  tmap3(&tm_w2_k_, ptr<void>("w2"), S, H, F, 64, 128);
  // weights, MN-major B: box {64 n, 64 k, 1}
  tmap3(&tm_w1_mn_, ptr<void>("w1"), S, 2 * F, H, 64, 64);
  tmap3(&tm_w2_mn_, ptr<void>("w2"), S, H, F, 64, 64);
  // Wgrad operands, MN-major: box {64 cols, 64 rows}
  tmap2(&tm_dy_mn_, ptr<void>("dybuf"), T, H, 64, 64);
  tmap2(&tm_act_mn_, ptr<void>("act"), T, F, 64, 64);
  tmap2(&tm_dh_mn_, ptr<void>("hbuf"), T, 2 * F, 64, 64);
  tmap2(&tm_x_mn_, ptr<void>("xbuf"), T, H, 64, 64);

  // optional block-scaled fp8 forward
  if (ptr<void>("w1q", false) != nullptr) {
    if (c.H % 128 || c.F % 128) throw std::runtime_error("MoeRuntime: the fp8 path needs H % 128 == 0 and F % 128 == 0");
    for (const char* name : {"w2q", "sfb1", "sfb2", "xq", "sfx", "actq", "sfact", "w1q_ptrs", "w2q_ptrs", "sfb1_ptrs", "sfb2_ptrs",
                             "xq_ptrs", "sfx_ptrs"})
      ptr<void>(name);
    // weight boxes: 128 rows for the single-CTA kernel; the CTA-pair kernel stages half a tile's columns per CTA
    const bool pair = c.gemm_ctas == 2;
    const uint32_t box1 = pair ? ((2 * F) % 256 == 0 ? 128 : 64) : 128, box2 = pair ? (H % 256 == 0 ? 128 : 64) : 128;
    if (!make_tmap_fp8_2d(&tm_xq_, ptr<void>("xq"), T, H) || !make_tmap_fp8_2d(&tm_actq_, ptr<void>("actq"), T, F) ||
        !make_tmap_fp8_3d(&tm_w1q_, ptr<void>("w1q"), S, 2 * F, H, box1) ||
        !make_tmap_fp8_3d(&tm_w2q_, ptr<void>("w2q"), S, H, F, box2))
      throw std::runtime_error("MoeRuntime: cuTensorMapEncodeTiled (fp8) failed");
    if (pair) {
      const uint64_t kg_h = (H / 128 + 3) / 4, kg_f = (F / 128 + 3) / 4;
      if (!make_tmap_sf(&tm_sfx_, ptr<void>("sfx"), (T / 128) * kg_h) ||
          !make_tmap_sf(&tm_sfact_, ptr<void>("sfact"), (T / 128) * kg_f) ||
          !make_tmap_sf(&tm_sfb1_, ptr<void>("sfb1"), S * (2 * F / 128) * kg_h) ||
          !make_tmap_sf(&tm_sfb2_, ptr<void>("sfb2"), S * (H / 128) * kg_f))
        throw std::runtime_error("MoeRuntime: cuTensorMapEncodeTiled (scale chunks) failed");
    }
    fp8_ = true;
  }
}

// ------------------------------------------------------------------ forward pieces
void MoeRuntime::publish(const int64_t* topk_idx, int num_units, cudaStream_t stream) {
  if (num_units > cfg_.max_units) throw std::runtime_error("MoeRuntime: more routing units than max_units");
  CountArgs a{};
  a.unit_expert = topk_idx;
  a.num_units = num_units;
  a.E = cfg_.E;
  a.R = cfg_.R;
  a.me = cfg_.me;
  a.chunk_hist = ptr<int32_t>("chunk_hist");
  a.hist_acc = ptr<int32_t>("hist_acc");
  a.exp_prefix = ptr<int32_t>("exp_prefix");
  a.omega_ptrs = ptr<int32_t* const>("omega_ptrs");
  a.signal_ptrs = ptr<unsigned* const>("signal_ptrs");
  a.epoch_word = ptr<unsigned>("epochs");
  // arrival counters (forward, backward) and replica pull counters of this rank start every step at zero;
  // peers add to them only after their solver has seen this rank's signal
  a.clear = ptr<unsigned>("arrive");
  a.clear_words = 2 * n_tiles_ + 2 * (cfg_.w_slots - cfg_.home_cap) + 2;  // + the two ticket words of the transports
  check(launch_count_publish(a, stream), "count_publish");
}

void MoeRuntime::solve(cudaStream_t stream) { check(launch_solver(sp_, tables_, stream), "solver"); }

void MoeRuntime::route(const int64_t* topk_idx, int num_units, cudaStream_t stream) {
  if (num_units > cfg_.max_units) throw std::runtime_error("MoeRuntime: more routing units than max_units");
  RouteArgs a{};
  a.unit_expert = topk_idx;
  a.num_units = num_units;
  a.E = cfg_.E;
  a.R = cfg_.R;
  a.q_me = sp_.q + (size_t)cfg_.me * cfg_.E * cfg_.R;
  a.row_base = tables_.row_base;
  a.chunk_hist = ptr<const int32_t>("chunk_hist");
  a.exp_prefix = ptr<const int32_t>("exp_prefix");
  a.unit_dst = ptr<int32_t>("unit_dst");
  a.unit_row = ptr<int32_t>("unit_row");
  a.sorted_units = ptr<int32_t>("sorted_units");
  a.unit_pos = ptr<int32_t>("unit_pos");
  a.status = sp_.status;
  check(launch_route_assign(a, stream), "route_assign");
}

CommArgs MoeRuntime::comm_args(bool dispatch, bool pad, bool pull) const {
  CommArgs a{};
  a.do_dispatch = dispatch;
  a.do_pad = pad;
  a.do_pull = pull && cfg_.w_slots > cfg_.home_cap;
  a.R = cfg_.R;
  a.me = cfg_.me;
  a.E = cfg_.E;
  a.H = cfg_.H;
  a.topk = cfg_.topk;
  a.row_capacity = cfg_.row_capacity;
  a.tile_rows = tile_rows_;
  a.block_rows = block_rows_;
  a.sorted_units = ptr<const int32_t>("sorted_units");
  a.exp_prefix = ptr<const int32_t>("exp_prefix");
  a.q_me = sp_.q + (size_t)cfg_.me * cfg_.E * cfg_.R;
  a.row_base = tables_.row_base;
  a.send_off = tables_.send_off;
  a.tiles_of = tables_.tiles_of;
  a.arrive_ptrs = ptr<unsigned* const>("arrive_ptrs");
  a.group_off = tables_.group_off;
  a.group_rows = tables_.group_rows;
  a.n_groups_cap = cfg_.w_slots;
  a.home_cap = cfg_.home_cap;
  a.w_slots = cfg_.w_slots;
  a.group_expert = tables_.group_expert;
  a.group_wslot = tables_.group_wslot;
  a.main_rank = sp_.main_rank;
  a.home_index = tables_.home_index;
  a.w1_ptrs = ptr<void* const>("w1_ptrs");
  a.w2_ptrs = ptr<void* const>("w2_ptrs");
  a.w1_elems = (size_t)2 * cfg_.F * cfg_.H;
  a.w2_elems = (size_t)cfg_.F * cfg_.H;
  a.pull_cnt = ptr<unsigned>("arrive") + 2 * n_tiles_;
  return a;
}

CommArgs MoeRuntime::comm_forward(const void* tokens, const float* topk_prob, bool pad, bool pull) const {
  CommArgs a = comm_args(true, pad, pull);
  a.rows = tokens;
  a.unit_prob = topk_prob;
  a.buf_ptrs = ptr<void* const>("xbuf_ptrs");
  a.meta_ptrs = ptr<int2* const>("meta_ptrs");
  a.rowp_ptrs = ptr<float* const>("rowp_ptrs");
  a.local_buf = ptr<void>("xbuf");
  a.local_meta = ptr<int2>("meta");
  a.arrive_off = 0;
  a.ticket = ptr<unsigned>("arrive") + 2 * n_tiles_ + 2 * (cfg_.w_slots - cfg_.home_cap);  // cleared by count_publish
  return a;
}
CommArgs MoeRuntime::comm_backward(const void* dout) const {
  CommArgs a = comm_args(true, true, false);
  a.rows = dout;
  a.buf_ptrs = ptr<void* const>("dybuf_ptrs");
  a.local_buf = ptr<void>("dybuf");
  a.arrive_off = n_tiles_;
  a.ticket = ptr<unsigned>("arrive") + 2 * n_tiles_ + 2 * (cfg_.w_slots - cfg_.home_cap) + 1;
  return a;
}

void MoeRuntime::dispatch_tokens(const void* tokens, const float* topk_prob, int num_units, cudaStream_t stream, bool zero_pad) {
  if (num_units > cfg_.max_units) throw std::runtime_error("MoeRuntime: more routing units than max_units");
  const CommArgs a = comm_forward(tokens, topk_prob, zero_pad, false);
  check(launch_comm(a, cfg_.num_sms, sp_.status, stream), "dispatch");
}

void MoeRuntime::pull_weights(cudaStream_t stream) {
  if (cfg_.w_slots <= cfg_.home_cap) return;
  CommArgs a = comm_args(false, false, true);
  check(launch_comm(a, cfg_.num_sms, sp_.status, stream), "weight_pull");
}

void MoeRuntime::barrier(int slot, cudaStream_t stream) {
  if (!cfg_.multi_rank_sync || cfg_.R <= 1) return;
  check(launch_symm_barrier(ptr<unsigned* const>("signal_ptrs"), slot, cfg_.R, cfg_.me, ptr<unsigned>("epochs") + slot,
                            sp_.status, stream),
        "symm_barrier");
}

void MoeRuntime::gemm(int mode, const CUtensorMap& a, const CUtensorMap& b, int N, int K, int M_out, void* out0,
                      void* out1, void* const* out_ptrs, const int2* meta, cudaStream_t stream, const GemmExtra& extra) {
  GemmArgs g{};
  g.mode = mode;
  g.ctas = cfg_.gemm_ctas;
  g.group_off = tables_.group_off;
  g.group_rows = tables_.group_rows;
  g.group_wslot = tables_.group_wslot;
  g.totals = tables_.totals;
  g.n_groups_cap = cfg_.w_slots;
  g.row_capacity = cfg_.row_capacity;
  g.N = N;
  g.K = K;
  g.M_out = M_out;
  g.out0 = out0;
  g.out1 = out1;
  g.out_ptrs = out_ptrs;
  g.meta = meta;
  g.status = sp_.status;
  g.wait_ns = wait_ns_;
  if (extra.gate) {
    g.arrive = ptr<const unsigned>("arrive") + (extra.gate == 2 ? n_tiles_ : 0);
    g.arrive_expected = (unsigned)(cfg_.R * (tile_rows_ / block_rows_));
  }
  if (extra.gate_pull && cfg_.w_slots > cfg_.home_cap) {
    g.pull_cnt = ptr<const unsigned>("arrive") + 2 * n_tiles_;  // counters of w1 (the B operand of GEMM1)
    g.pull_expected = pull_chunks((size_t)2 * cfg_.F * cfg_.H);
    g.home_cap = cfg_.home_cap;
  }
  if (extra.done_slot > 0 && peers()) {
    g.done_ctr = ptr<unsigned>("done_ctr");
    g.done_epoch = ptr<unsigned>("epochs") + extra.done_slot;
    g.done_signal_ptrs = ptr<unsigned* const>("signal_ptrs");
    g.done_slot = extra.done_slot;
    g.done_R = cfg_.R;
  }
  g.row_scale = extra.row_scale;
  if (extra.comm != nullptr) {
    g.comm = *extra.comm;
    g.trace = ptr<unsigned long long>("gemm_trace", false);  // optional: phase timestamps of the fused kernels
    if (g.trace != nullptr) g.trace += mode == kFwd1 ? 0 : 12;
  }
  check(launch_grouped_gemm(a, b, g, cfg_.num_sms, stream), extra.comm ? "grouped_gemm+transport" : "grouped_gemm");
}

void MoeRuntime::gemm1(cudaStream_t stream) {
  GemmExtra x;
  x.gate = 1;
  x.gate_pull = true;
  x.row_scale = ptr<const float>("rowp");
  gemm(kFwd1, tm_x_k_, tm_w1_k_, cfg_.F, cfg_.H, 0, ptr<void>("hbuf"), ptr<void>("act"), nullptr, nullptr, stream, x);
}
void MoeRuntime::gemm1_fused(const void* tokens, const float* topk_prob, int num_units, cudaStream_t stream) {
  if (num_units > cfg_.max_units) throw std::runtime_error("MoeRuntime: more routing units than max_units");
  const CommArgs a = comm_forward(tokens, topk_prob, true, true);
  GemmExtra x;
  x.gate = 1;
  x.gate_pull = true;
  x.row_scale = ptr<const float>("rowp");
  x.comm = &a;
  gemm(kFwd1, tm_x_k_, tm_w1_k_, cfg_.F, cfg_.H, 0, ptr<void>("hbuf"), ptr<void>("act"), nullptr, nullptr, stream, x);
}
void MoeRuntime::gemm2(cudaStream_t stream) {
  GemmExtra x;
  x.done_slot = 2;
  gemm(kFwd2, tm_act_k_, tm_w2_k_, cfg_.H, cfg_.F, 0, nullptr, nullptr, ptr<void* const>("ybuf_ptrs"),
       ptr<const int2>("meta"), stream, x);
}
UnitReduceWait MoeRuntime::reduce_wait(int slot) const {
  UnitReduceWait w{};
  w.signal = ptr<const unsigned>("signals") + slot;
  w.epoch = ptr<const unsigned>("epochs") + slot;
  w.R = cfg_.R;
  w.budget_ns = wait_ns_;
  w.status = sp_.status;
  return w;
}
void MoeRuntime::reduce_out(void* out, int num_tokens, cudaStream_t stream, bool wait_peers, const float* unit_scale) {
  const UnitReduceWait w = reduce_wait(2);
  check(launch_unit_reduce(ptr<void>("ybuf"), ptr<const int32_t>("unit_pos"), unit_scale, out, num_tokens, cfg_.topk, cfg_.H,
                           wait_peers && peers() ? &w : nullptr, nullptr, nullptr, stream),
        "unit_reduce");
}

// ------------------------------------------------------------------ block-scaled fp8 forward
namespace {
inline size_t sf_bytes_per_slot(int N, int K) { return (size_t)(N / 128) * ((K / 128 + 3) / 4) * 512; }
}  // namespace

void MoeRuntime::quantize_own_weights(cudaStream_t stream) {
  if (!fp8_) throw std::runtime_error("MoeRuntime: fp8 regions were not provided");
  check(launch_quantize_weights(ptr<void>("w1"), ptr<uint8_t>("w1q"), ptr<uint8_t>("sfb1"), cfg_.home_cap, 2 * cfg_.F,
                                cfg_.H, stream),
        "quantize_weights(w1)");
  check(launch_quantize_weights(ptr<void>("w2"), ptr<uint8_t>("w2q"), ptr<uint8_t>("sfb2"), cfg_.home_cap, cfg_.H,
                                cfg_.F, stream),
        "quantize_weights(w2)");
}

void MoeRuntime::pull_weights_fp8(cudaStream_t stream) {
  if (cfg_.w_slots <= cfg_.home_cap) return;
  WeightPullArgs a{};
  a.slot_of = tables_.slot_of;
  a.main_rank = sp_.main_rank;
  a.home_index = tables_.home_index;
  a.E = cfg_.E;
  a.R = cfg_.R;
  a.me = cfg_.me;
  a.home_cap = cfg_.home_cap;
  a.n_slot = cfg_.w_slots;
  // the pull kernel counts 2-byte elements
  const size_t w1_bytes = (size_t)2 * cfg_.F * cfg_.H, w2_bytes = (size_t)cfg_.F * cfg_.H;
  const struct { const char* name; size_t bytes; } regions[4] = {
      {"w1q_ptrs", w1_bytes}, {"w2q_ptrs", w2_bytes},
      {"sfb1_ptrs", sf_bytes_per_slot(2 * cfg_.F, cfg_.H)}, {"sfb2_ptrs", sf_bytes_per_slot(cfg_.H, cfg_.F)}};
  for (const auto& r : regions) {
    a.w_ptrs = ptr<void* const>(r.name);
    a.elems_per_slot = r.bytes / 2;
    check(launch_weight_pull(a, stream), "weight_pull(fp8)");
  }
}

void MoeRuntime::gemm_fp8(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& sfa_map,
                          const CUtensorMap& sfb_map, int N, int K, const uint8_t* sfa, const uint8_t* sfb, void* out,
                          void* const* out_ptrs, const int2* meta, cudaStream_t stream) {
  Fp8GemmArgs g{};
  g.group_off = tables_.group_off;
  g.group_rows = tables_.group_rows;
  g.group_wslot = tables_.group_wslot;
  g.totals = tables_.totals;
  g.n_groups_cap = cfg_.w_slots;
  g.row_capacity = cfg_.row_capacity;
  g.N = N;
  g.K = K;
  g.sfa = sfa;
  g.sfb = sfb;
  g.out = out;
  g.out_ptrs = out_ptrs;
  g.meta = meta;
  g.status = sp_.status;
  // the single-CTA kernel can share the pair kernel's weight map only when that map has 128-row boxes
  const bool pair = cfg_.gemm_ctas == 2 && (fp8_pair_ || N % 256 != 0);
  if (pair)
    check(launch_grouped_gemm_fp8_pair(a, b, sfa_map, sfb_map, g, cfg_.num_sms, stream), "grouped_gemm_fp8_pair");
  else
    check(launch_grouped_gemm_fp8(a, b, g, cfg_.num_sms, stream), "grouped_gemm_fp8");
}

void MoeRuntime::dispatch_fp8(const void* tokens, int num_units, cudaStream_t stream) {
  DispatchFp8Args a{};
  a.rows = tokens;
  a.num_units = num_units;
  a.topk = cfg_.topk;
  a.H = cfg_.H;
  a.R = cfg_.R;
  a.me = cfg_.me;
  a.unit_dst = ptr<const int32_t>("unit_dst");
  a.unit_row = ptr<const int32_t>("unit_row");
  a.unit_pos = ptr<const int32_t>("unit_pos");
  a.xq_ptrs = ptr<uint8_t* const>("xq_ptrs");
  a.sfx_ptrs = ptr<uint8_t* const>("sfx_ptrs");
  a.meta_ptrs = ptr<int2* const>("meta_ptrs");
  a.row_capacity = cfg_.row_capacity;
  check(launch_dispatch_fp8(a, stream), "dispatch_fp8");
}

void MoeRuntime::gemm1_fp8(cudaStream_t stream) {
  gemm_fp8(tm_xq_, tm_w1q_, tm_sfx_, tm_sfb1_, 2 * cfg_.F, cfg_.H, ptr<uint8_t>("sfx"), ptr<uint8_t>("sfb1"),
           ptr<void>("hbuf"), nullptr, nullptr, stream);
}
void MoeRuntime::act_fp8(cudaStream_t stream) {
  const RowGroups groups{tables_.group_off, tables_.group_rows, tables_.totals, cfg_.w_slots};
  check(launch_swiglu_quantize(ptr<void>("hbuf"), ptr<uint8_t>("actq"), ptr<uint8_t>("sfact"), nullptr, cfg_.row_capacity,
                               cfg_.F, &groups, stream),
        "swiglu_quantize");
}
void MoeRuntime::gemm2_fp8(cudaStream_t stream) {
  gemm_fp8(tm_actq_, tm_w2q_, tm_sfact_, tm_sfb2_, cfg_.H, cfg_.F, ptr<uint8_t>("sfact"), ptr<uint8_t>("sfb2"), nullptr,
           ptr<void* const>("ybuf_ptrs"), ptr<const int2>("meta"), stream);
}

void MoeRuntime::forward_fp8(const void* tokens, const int64_t* topk_idx, const float* topk_prob, void* out,
                             int num_tokens, cudaStream_t stream) {
  if (!fp8_) throw std::runtime_error("MoeRuntime: fp8 regions were not provided");
  const int U = num_tokens * cfg_.topk;
  // about U rows reach this rank; with few rows per expert the 256-row tiles of the pair kernel are mostly padding
  fp8_pair_ = U >= 192 * cfg_.w_slots;
  publish(topk_idx, U, stream);
  solve(stream);
  route(topk_idx, U, stream);
  dispatch_fp8(tokens, U, stream);  // rows cross NVLink as e4m3 + scales; padding rows stay stale (never stored)
  pull_weights_fp8(stream);
  barrier(1, stream);
  gemm1_fp8(stream);
  act_fp8(stream);
  gemm2_fp8(stream);
  barrier(2, stream);
  reduce_out(out, num_tokens, stream, false, topk_prob);
}

// ------------------------------------------------------------------ backward pieces
void MoeRuntime::dispatch_grads(const void* dout, int num_units, cudaStream_t stream) {
  if (num_units > cfg_.max_units) throw std::runtime_error("MoeRuntime: more routing units than max_units");
  const CommArgs a = comm_backward(dout);
  check(launch_comm(a, cfg_.num_sms, sp_.status, stream), "dispatch_grads");
}
void MoeRuntime::wgrad2(cudaStream_t stream) {
  GemmExtra x;
  x.gate = 2;
  gemm(kWgrad, tm_dy_mn_, tm_act_mn_, cfg_.F, 0, cfg_.H, ptr<void>("gw2"), nullptr, nullptr, nullptr, stream, x);
}
void MoeRuntime::swiglu_pass(cudaStream_t stream) {
  SwigluBwdArgs a{};
  a.dact = ptr<void>("dact");
  a.h = ptr<void>("hbuf");
  a.rows = cfg_.row_capacity;
  a.F = cfg_.F;
  a.row_limit = tables_.totals;
  a.rowp = ptr<const float>("rowp");
  a.meta = ptr<const int2>("meta");
  a.dprob_ptrs = ptr<float* const>("dprob_ptrs");
  check(launch_swiglu_backward(a, stream), "swiglu_backward");
}
void MoeRuntime::dgrad2(cudaStream_t stream) {
  GemmExtra x;
  x.gate = 2;
  gemm(kDgrad1, tm_dy_k_, tm_w2_mn_, cfg_.F, cfg_.H, 0, ptr<void>("dact"), nullptr, nullptr, nullptr, stream, x);
  swiglu_pass(stream);
}
void MoeRuntime::dgrad2_fused(const void* dout, int num_units, cudaStream_t stream) {
  if (num_units > cfg_.max_units) throw std::runtime_error("MoeRuntime: more routing units than max_units");
  const CommArgs a = comm_backward(dout);
  GemmExtra x;
  x.gate = 2;
  x.comm = &a;
  gemm(kDgrad1, tm_dy_k_, tm_w2_mn_, cfg_.F, cfg_.H, 0, ptr<void>("dact"), nullptr, nullptr, nullptr, stream, x);
  swiglu_pass(stream);
}
void MoeRuntime::wgrad1(cudaStream_t stream) {
  gemm(kWgrad, tm_dh_mn_, tm_x_mn_, cfg_.H, 0, 2 * cfg_.F, ptr<void>("gw1"), nullptr, nullptr, nullptr, stream);
}
void MoeRuntime::dgrad1(cudaStream_t stream) {
  GemmExtra x;
  x.done_slot = 4;
  gemm(kDgrad1, tm_dh_k_, tm_w1_mn_, cfg_.H, 2 * cfg_.F, 0, nullptr, nullptr, ptr<void* const>("dxbuf_ptrs"),
       ptr<const int2>("meta"), stream, x);
}
void MoeRuntime::reduce_dtokens(void* dtokens, float* dprob, int num_tokens, cudaStream_t stream, bool wait_peers) {
  const UnitReduceWait w = reduce_wait(4);
  check(launch_unit_reduce(ptr<void>("dxbuf"), ptr<const int32_t>("unit_pos"), nullptr, dtokens, num_tokens, cfg_.topk, cfg_.H,
                           wait_peers && peers() ? &w : nullptr, ptr<const float>("dprob"), dprob, stream),
        "unit_reduce(bwd)");
}
void MoeRuntime::reduce_weight_grads(cudaStream_t stream) {
  void* acc1 = ptr<void>("acc_gw1", false);
  void* acc2 = ptr<void>("acc_gw2", false);
  if (cfg_.R <= 1 && acc1 == nullptr) return;
  GradReduceArgs a{};
  a.accum_fp32 = cfg_.accum_fp32;
  a.slot_of = tables_.slot_of;
  a.main_rank = sp_.main_rank;
  a.home_index = tables_.home_index;
  a.E = cfg_.E;
  a.R = cfg_.R;
  a.me = cfg_.me;
  a.home_cap = cfg_.home_cap;
  a.g_ptrs = ptr<void* const>("gw1_ptrs");
  a.accum = acc1;
  a.elems_per_slot = (size_t)2 * cfg_.F * cfg_.H;
  check(launch_grad_reduce(a, stream), "grad_reduce(w1)");
  a.g_ptrs = ptr<void* const>("gw2_ptrs");
  a.accum = acc2;
  a.elems_per_slot = (size_t)cfg_.F * cfg_.H;
  check(launch_grad_reduce(a, stream), "grad_reduce(w2)");
}

// ------------------------------------------------------------------ timing
void MoeRuntime::enable_timing(bool on) {
  timing_ = on;
  for (auto& m : marks_) cudaEventDestroy(m.second);
  marks_.clear();
}
void MoeRuntime::mark(const char* name, cudaStream_t stream) {
  if (!timing_) return;
  cudaEvent_t ev;
  if (cudaEventCreate(&ev) != cudaSuccess) return;
  cudaEventRecord(ev, stream);
  marks_.emplace_back(name, ev);
}
std::vector<std::pair<std::string, float>> MoeRuntime::phase_times() {
  std::vector<std::pair<std::string, float>> out;
  if (marks_.empty()) return out;
  cudaEventSynchronize(marks_.back().second);
  for (size_t i = 1; i < marks_.size(); ++i) {
    float ms = 0.f;
    if (marks_[i - 1].first == "fwd_end") continue;  // gap between forward and backward is not a phase
    cudaEventElapsedTime(&ms, marks_[i - 1].second, marks_[i].second);
    out.emplace_back(marks_[i].first, ms);
  }
  for (auto& m : marks_) cudaEventDestroy(m.second);
  marks_.clear();
  return out;
}

// ------------------------------------------------------------------ whole passes
void MoeRuntime::forward(const void* tokens, const int64_t* topk_idx, const float* topk_prob, void* out,
                         int num_tokens, cudaStream_t stream) {
  const int U = num_tokens * cfg_.topk;
  mark("fwd_begin", stream);
  publish(topk_idx, U, stream);
  mark("publish", stream);
  solve(stream);
  mark("solve", stream);
  route(topk_idx, U, stream);
  mark("route", stream);
  if (cfg_.fused_comm) {
    gemm1_fused(tokens, topk_prob, U, stream);
    mark("dispatch+pull+gemm1", stream);
  } else {
    dispatch_tokens(tokens, topk_prob, U, stream);
    pull_weights(stream);
    mark("dispatch+pull", stream);
    gemm1(stream);
    mark("gemm1", stream);
  }
  gemm2(stream);
  mark("gemm2", stream);
  reduce_out(out, num_tokens, stream, true);
  mark("reduce_out", stream);
  mark("fwd_end", stream);
}

void MoeRuntime::backward(const void* dout, void* dtokens, float* dprob, int num_tokens, cudaStream_t stream) {
  const int U = num_tokens * cfg_.topk;
  mark("bwd_begin", stream);
  if (cfg_.fused_comm) {
    dgrad2_fused(dout, U, stream);
    mark("dispatch_grads+dgrad2", stream);
  } else {
    dispatch_grads(dout, U, stream);
    mark("dispatch_grads", stream);
    dgrad2(stream);
    mark("dgrad2", stream);
  }
  wgrad2(stream);
  mark("wgrad2", stream);
  wgrad1(stream);
  mark("wgrad1", stream);
  const bool side = peers() && side_ != nullptr;
  if (side) {
    // Gradient return beside Dgrad1: once every rank has finished its weight-gradient GEMMs (barrier on
    // the side stream), each owner adds its replicas' slots with peer loads.  Dgrad1 is bound by its
    // outbound row stores, the return by inbound loads, so the two share the link without competing.
    if (cudaEventRecord(ev_fork_, stream) != cudaSuccess || cudaStreamWaitEvent(side_, ev_fork_, 0) != cudaSuccess)
      throw std::runtime_error("MoeRuntime: could not fork the side stream");
    on_side_ = true;
    barrier(5, side_);
    reduce_weight_grads(side_);
    on_side_ = false;
    if (cudaEventRecord(ev_join_, side_) != cudaSuccess) throw std::runtime_error("MoeRuntime: could not record the join event");
  }
  dgrad1(stream);
  mark("dgrad1", stream);
  reduce_dtokens(dtokens, dprob, num_tokens, stream, true);
  mark("reduce_dtokens", stream);
  if (side) {
    if (cudaStreamWaitEvent(stream, ev_join_, 0) != cudaSuccess) throw std::runtime_error("MoeRuntime: could not join the side stream");
  } else {
    reduce_weight_grads(stream);
  }
  mark("reduce_weight_grads", stream);
}

}  // namespace epb
