// Per-layer runtime: owns no memory, holds the device pointers of one MoE layer's buffers and
// launches the step's kernels in order on a caller-provided stream.  The host never reads device
// data on this path; routing, group sizes and slot use stay on the GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <utility>
#include <vector>

#include "grouped_gemm.h"
#include "grouped_gemm_fp8.h"
#include "route.h"
#include "solver.h"

namespace epb {

struct LayerConfig {
  int R = 1, me = 0, E = 0, H = 0, F = 0, topk = 0;
  int w_slots = 0;        // weight slots per rank (home_cap + replica slots)
  int home_cap = 0;       // experts owned per rank (upper bound)
  int n_slot_plan = 0;    // slot budget the solver enforces (C4)
  int row_capacity = 0;   // rows of the receive buffers
  int max_units = 0;      // tokens * topk this rank can route per step
  int D = 1, u_min = 1, iters = 64, patience = 8, allow_cross = 1, probe = 0;
  int64_t s_tok = 0;
  int num_sms = 148;
  int gemm_ctas = 2;        // 2: grouped GEMMs run on CTA pairs (256-row tiles); 1: single CTAs (128-row tiles)
  int accum_fp32 = 0;       // dtype of the optional gradient accumulation buffers (acc_gw1/acc_gw2)
  int multi_rank_sync = 1;  // 0: one process emulates all ranks, kernels are ordered by the stream
  int fused_comm = 1;       // 1: forward()/backward() run the token transport on spare warps of the consuming
                            //    GEMM (dispatch + GEMM1, gradient dispatch + Dgrad2 in one kernel each);
                            //    0: a stand-alone transport kernel runs first (the GEMM is gated either way)
  int comm_block_rows = 0;  // rows per transport block; 0: min(M tile, 32 * R) rounded down to a power of two
  int wait_ms = 1500;       // budget of every cross-rank wait of this layer's kernels, in milliseconds (bounded)
};

class MoeRuntime {
 public:
  MoeRuntime(const LayerConfig& cfg, const std::map<std::string, uint64_t>& ptrs);

  // ---- forward pieces (each enqueues on `stream` and returns)
  void publish(const int64_t* topk_idx, int num_units, cudaStream_t stream);
  void solve(cudaStream_t stream);
  void route(const int64_t* topk_idx, int num_units, cudaStream_t stream);
  // Stand-alone transport of the token rows (CommArgs in route.h): rows stored into the hosts' buffers at
  // their final position, arrival counters advanced per M-tile.
  // zero_pad: clear the padding rows behind every group (needed when a backward pass will contract over them)
  void dispatch_tokens(const void* tokens, const float* topk_prob, int num_units, cudaStream_t stream, bool zero_pad = true);
  void pull_weights(cudaStream_t stream);   // stand-alone replica weight pull (per-slot counters advanced)
  void barrier(int slot, cudaStream_t stream);
  void gemm1(cudaStream_t stream);          // gated per M-tile on the arrival counters, per replica slot on the pull counters
  // One kernel: transport warps send this rank's rows and pull its replica weights while the other
  // warps run GEMM1 on the tiles whose rows have arrived.
  void gemm1_fused(const void* tokens, const float* topk_prob, int num_units, cudaStream_t stream);
  void gemm2(cudaStream_t stream);          // rows stored to their source ranks; the last CTA signals every peer
  // Sum of every token's unit rows (already gate-weighted: the weight was folded into the activation).
  // wait_peers: first wait (bounded, in the kernel) for every rank's completion signal of gemm2.
  // unit_scale (fp8 inference path only): the rows are unweighted and scaled here.
  void reduce_out(void* out, int num_tokens, cudaStream_t stream, bool wait_peers = false, const float* unit_scale = nullptr);
  // ---- backward pieces
  void dispatch_grads(const void* dout, int num_units, cudaStream_t stream);   // pure copy of the gradient rows
  void wgrad2(cudaStream_t stream);
  // Plain Dgrad2 GEMM, then the SwiGLU-gradient pass, which also applies the row's gate weight and stores
  // the row's gate-weight gradient into the source rank's symmetric `dprob` buffer.
  void dgrad2(cudaStream_t stream);
  // One kernel: transport warps send dout while the other warps run the plain Dgrad2 GEMM; then the pass.
  void dgrad2_fused(const void* dout, int num_units, cudaStream_t stream);
  void wgrad1(cudaStream_t stream);
  void dgrad1(cudaStream_t stream);
  // Also hands the gate-weight gradients (stored by the hosts into this rank's symmetric buffer) to `dprob`.
  void reduce_dtokens(void* dtokens, float* dprob, int num_tokens, cudaStream_t stream, bool wait_peers = false);
  void reduce_weight_grads(cudaStream_t stream);

  // ---- block-scaled fp8 forward (inference): present when the fp8 weight regions were given
  bool has_fp8() const { return fp8_; }
  void quantize_own_weights(cudaStream_t stream);   // bf16 home slots -> e4m3 + 128 x 128 scales
  void pull_weights_fp8(cudaStream_t stream);       // replicas pull e4m3 bytes and scale chunks: half the bytes of bf16
  void dispatch_fp8(const void* tokens, int num_units, cudaStream_t stream);  // dispatch fused with the 1 x 128 quantisation
  void gemm1_fp8(cudaStream_t stream);              // h = x W1^T on the quantised rows
  void act_fp8(cudaStream_t stream);                // SwiGLU + quantise
  void gemm2_fp8(cudaStream_t stream);              // y = act W2^T, rows scattered to their sources
  void forward_fp8(const void* tokens, const int64_t* topk_idx, const float* topk_prob, void* out, int num_tokens,
                   cudaStream_t stream);

  // ---- whole passes
  void forward(const void* tokens, const int64_t* topk_idx, const float* topk_prob, void* out, int num_tokens,
               cudaStream_t stream);
  void backward(const void* dout, void* dtokens, float* dprob, int num_tokens, cudaStream_t stream);

  // Optional per-phase device timing: events are recorded around every phase of forward() and
  // backward(); phase_times() synchronises and returns (name, ms) pairs of the last pass pair.
  void enable_timing(bool on);
  std::vector<std::pair<std::string, float>> phase_times();

  int launches() const { return launches_; }
  void reset_launches() { launches_ = 0; }
  const LayerConfig& config() const { return cfg_; }
  // Optional launch log: the name of every kernel enqueued since trace_launches(true), in issue order
  // ("side:" prefix for launches on the runtime's own side stream).
  void trace_launches(bool on) { trace_ = on; launch_log_.clear(); }
  const std::vector<std::string>& launch_log() const { return launch_log_; }
  ~MoeRuntime();
  MoeRuntime(const MoeRuntime&) = delete;
  MoeRuntime& operator=(const MoeRuntime&) = delete;

 private:
  template <typename T>
  T* ptr(const char* name, bool required = true) const;
  void check(cudaError_t e, const char* what);
  struct GemmExtra {
    int gate = 0;        // 1: gate A on the forward arrival counters, 2: on the backward ones
    bool gate_pull = false;
    int done_slot = 0;   // > 0: signal every peer on this slot when the launch is complete
    const float* row_scale = nullptr;
    const CommArgs* comm = nullptr;
  };
  void gemm(int mode, const CUtensorMap& a, const CUtensorMap& b, int N, int K, int M_out, void* out0, void* out1,
            void* const* out_ptrs, const int2* meta, cudaStream_t stream, const GemmExtra& extra);
  void gemm(int mode, const CUtensorMap& a, const CUtensorMap& b, int N, int K, int M_out, void* out0, void* out1,
            void* const* out_ptrs, const int2* meta, cudaStream_t stream) {
    gemm(mode, a, b, N, K, M_out, out0, out1, out_ptrs, meta, stream, GemmExtra{});
  }
  CommArgs comm_args(bool dispatch, bool pad, bool pull) const;
  CommArgs comm_forward(const void* tokens, const float* topk_prob, bool pad, bool pull) const;
  CommArgs comm_backward(const void* dout) const;
  void swiglu_pass(cudaStream_t stream);
  bool peers() const { return cfg_.multi_rank_sync && cfg_.R > 1; }
  UnitReduceWait reduce_wait(int slot) const;
  void tmap2(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t bc, uint32_t br);
  void tmap3(CUtensorMap* m, const void* base, uint64_t slots, uint64_t rows, uint64_t cols, uint32_t bc, uint32_t br);

  LayerConfig cfg_;
  std::map<std::string, uint64_t> ptrs_;
  SolverParams sp_{};
  RankTables tables_{};
  int launches_ = 0;
  bool trace_ = false;
  bool on_side_ = false;
  std::vector<std::string> launch_log_;
  int tile_rows_ = 256, block_rows_ = 32, n_tiles_ = 0;
  unsigned long long wait_ns_ = 0;
  cudaStream_t side_ = nullptr;            // gradient return runs here, beside the last GEMM of backward
  cudaEvent_t ev_fork_ = nullptr, ev_join_ = nullptr;
  bool timing_ = false;
  std::vector<std::pair<std::string, cudaEvent_t>> marks_;
  void mark(const char* name, cudaStream_t stream);
  // tensor maps (built once: every buffer has a fixed address)
  CUtensorMap tm_x_k_, tm_act_k_, tm_dy_k_, tm_dh_k_;           // K-major A operands
  CUtensorMap tm_w1_k_, tm_w2_k_, tm_w1_mn_, tm_w2_mn_;          // weights as B
  CUtensorMap tm_dy_mn_, tm_act_mn_, tm_dh_mn_, tm_x_mn_;        // Wgrad operands (MN-major)
  bool fp8_ = false;
  bool fp8_pair_ = true;   // CTA-pair fp8 kernel (256-row tiles); forward_fp8 falls back to 128-row tiles for tiny batches
  CUtensorMap tm_xq_, tm_actq_, tm_w1q_, tm_w2q_;                // e4m3 operands
  CUtensorMap tm_sfx_, tm_sfact_, tm_sfb1_, tm_sfb2_;            // scale chunks (CTA-pair fp8 kernel)
  void gemm_fp8(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& sfa_map, const CUtensorMap& sfb_map, int N,
                int K, const uint8_t* sfa, const uint8_t* sfb, void* out, void* const* out_ptrs, const int2* meta,
                cudaStream_t stream);
};

}  // namespace epb
