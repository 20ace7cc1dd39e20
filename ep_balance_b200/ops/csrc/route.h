// Token-path and weight-path kernels around the grouped GEMM (route.cu).
//
// "Peer pointer tables" are device arrays of R pointers, one per rank, to the same symmetric
// buffer on every rank.  On one GPU emulating R ranks they simply point at R local buffers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace epb {

// Units are counted and ranked in chunks of kRouteChunk consecutive units, one CTA per chunk.
constexpr int kRouteChunk = 256;
inline int route_chunks(int num_units) { return (num_units + kRouteChunk - 1) / kRouteChunk; }

// Histogram of this rank's routed expert ids (one CTA per chunk; per-chunk histograms are kept for the
// route assignment).  The last CTA to finish stores the histogram as row `me` of omega on every peer,
// writes its exclusive prefix to `exp_prefix`, clears this rank's arrival counters (`clear_words`
// 32-bit words at `clear`, may be null) and then adds 1 (release) to every peer's signal word.
// `epoch_word` (local, may be null) is advanced by one per call.
struct CountArgs {
  const int64_t* unit_expert;   // [U]
  int num_units, E, R, me;
  int32_t* chunk_hist;          // [route_chunks(U), E]
  int32_t* hist_acc;            // [E + 1]: running histogram (zero between calls) and, last, the CTA ticket
  int32_t* exp_prefix;          // [E + 1]
  int32_t* const* omega_ptrs;   // R peers: int32 [R, E]
  unsigned* const* signal_ptrs; // R peers (may be null)
  unsigned* epoch_word;
  unsigned* clear;
  int clear_words;
};
cudaError_t launch_count_publish(const CountArgs& a, cudaStream_t stream);

// Unit -> (dst rank, row in dst's receive buffers), plus the units ordered by expert.  The j-th unit
// (original order) of expert e goes to the host whose quota prefix covers j (eplb/integration/
// physical.py:30-77).  q_me = q[me] as [E, R]; row_base from the solver's RankTables; chunk_hist and
// exp_prefix from launch_count_publish over the same units.  O(U) work: one CTA per chunk of units.
struct RouteArgs {
  const int64_t* unit_expert;
  int num_units, E, R;
  const int32_t* q_me;
  const int32_t* row_base;
  const int32_t* chunk_hist;
  const int32_t* exp_prefix;
  int32_t* unit_dst;            // [U]
  int32_t* unit_row;            // [U]
  int32_t* sorted_units;        // [U] (may be null)
  int32_t* unit_pos;            // [U] position of the unit in sorted_units, -1 if it goes nowhere (may be null)
  int* status;
};
cudaError_t launch_route_assign(const RouteArgs& a, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// Item-driven token transport ("comm"), run either by a stand-alone kernel or by the spare warps of
// the grouped GEMM kernel that consumes the rows (grouped_gemm.cu), so that the transfer overlaps
// the tensor-core tiles.
//
// The sender walks the RECEIVERS' buffers block by block (block = `block_rows` consecutive rows of a
// peer's receive buffer, lowest rows first, peers visited round-robin starting with itself).  For
// every block it stores the rows it owes there -- the plan fixes the final row of every unit, so no
// size exchange is needed -- and then adds 1 (release, system scope) to the peer's arrival counter of
// the GEMM M-tile holding the block.  Every sender signals every block of every used tile, also when
// it owes no row there, so a tile is complete when its counter reaches R * (tile_rows / block_rows).
// Rows therefore arrive in the order the consuming GEMM walks its tile list.
// The same walk moves replica weights (peer loads from the owner's home slot, one counter per
// replica slot and weight tensor) and zero-fills this rank's own padding rows.
// The transport is a pure copy in both directions.  The gate weight of a unit travels with its token
// row in the forward pass (`unit_prob` -> the receiver's `rowp`), where GEMM1's epilogue folds it into
// the activation, so the backward pass sends the output gradient unscaled and the receiver applies
// the weight (and computes the gate-weight gradient) in its SwiGLU-gradient pass.
// Reference counterparts: all_to_all_single dispatch + slot sort (eplb/integration/comm.py:18-36,
// eplb_manager.py:1067-1105), replica broadcast (overlap.py:113-148).
struct CommArgs {
  int do_dispatch, do_pad, do_pull;
  int R, me, E, H, topk, row_capacity;
  int tile_rows;                 // rows of a GEMM M-tile (arrival-counter granularity)
  int block_rows;                // rows of a transport block; divides tile_rows
  // ---- rows to send
  const void* rows;              // bf16 [num_tokens, H]
  const float* unit_prob;        // [U] or null: gate weight of every unit, stored beside its row (forward)
  const int32_t* sorted_units;   // [U] this rank's units ordered by expert (stable)
  const int32_t* exp_prefix;     // [E + 1] first position of each expert in sorted_units
  const int32_t* q_me;           // [E, R] units (me, e) -> dst
  const int32_t* row_base;       // [E, R] first row in dst's buffer for (me, e) -> dst, -1 if none
  const int32_t* send_off;       // [E, R] units of expert e that go to ranks below dst
  const int32_t* tiles_of;       // [R] used M-tiles of every rank's receive buffer
  void* const* buf_ptrs;         // R peers: bf16 [row_capacity, H]
  int2* const* meta_ptrs;        // R peers: int2 [row_capacity] ({src rank, position of the unit in sorted_units}) or null
  float* const* rowp_ptrs;       // R peers: float [row_capacity] (gate weight of the row's unit) or null
  unsigned* const* arrive_ptrs;  // R peers: base of the counter region
  int arrive_off;                // first word of the arrival counters [row_capacity / tile_rows] in that region
  unsigned* ticket;              // local word, zero before the launch: the transport warps draw their blocks from it
                                 // in ascending order, so a warp that got light blocks simply takes more of them
  // ---- padding rows of this rank (zero-filled; their meta entries, if given, become {-1, -1})
  void* local_buf;
  int2* local_meta;
  const int32_t* group_off;      // [n_groups_cap + 1]
  const int32_t* group_rows;     // [n_groups_cap]
  int n_groups_cap;
  // ---- replica weights
  int home_cap, w_slots;
  const int32_t* group_expert;   // [n_groups_cap]
  const int32_t* group_wslot;    // [n_groups_cap]
  const int32_t* main_rank;      // [E]
  const int32_t* home_index;     // [E]
  void* const* w1_ptrs;          // R peers: bf16 [w_slots, w1_elems]
  void* const* w2_ptrs;
  size_t w1_elems, w2_elems;     // elements per slot (multiples of 8)
  unsigned* pull_cnt;            // local [2, w_slots - home_cap]: chunks landed per weight tensor and replica slot
};
constexpr int kPullChunkBytes = 32768;
__host__ __device__ inline unsigned pull_chunks(size_t elems) { return (unsigned)((elems * 2 + kPullChunkBytes - 1) / kPullChunkBytes); }
cudaError_t launch_comm(const CommArgs& a, int num_sms, int* status, cudaStream_t stream);

// out[t] = sum_k scale[u] * rows[pos(u)], u = t*topk+k   (scale may be null: plain sum)
// `unit_pos` (may be null: pos(u) = u) maps a unit to its row: the hosts return a unit's row at the unit's position
// in this rank's expert-sorted order, so that the rows one host returns for one expert are contiguous here and its
// epilogue's peer stores walk this rank's buffer sequentially; a negative position contributes nothing.
// `copy_src`/`copy_dst` (may be null): copy_dst[u] = copy_src[pos(u)] for num_tokens * topk floats (the gate-weight
// gradients that the peers stored into this rank's symmetric buffer, handed to the caller's tensor).
// With `wait_signal != nullptr` every CTA first waits (bounded) until *wait_signal >= *wait_epoch * R:
// the peers' "all my rows are stored" signals of the producing GEMM (GemmArgs::done_*).
struct UnitReduceWait {
  const unsigned* signal;       // this rank's signal word
  const unsigned* epoch;        // local epoch word
  int R;
  unsigned long long budget_ns;
  int* status;
};
cudaError_t launch_unit_reduce(const void* unit_rows, const int32_t* unit_pos, const float* unit_scale, void* out,
                               int num_tokens, int topk, int H, const UnitReduceWait* wait, const float* copy_src,
                               float* copy_dst, cudaStream_t stream);

// Cross-rank barrier on symmetric signal words: every rank adds 1 to word `slot` of every peer,
// then waits (bounded) until its own word reaches (epoch+1)*R.  `epoch_word` lives in local
// device memory and is advanced by the kernel, so the host carries no barrier state.
cudaError_t launch_symm_barrier(unsigned* const* signal_ptrs, int slot, int R, int me, unsigned* epoch_word,
                                int* status, cudaStream_t stream);

// Replica weight pull: for every local weight slot >= home_cap that the plan fills, copy the
// expert's weights from its owner's home slot (peer load) into the local slot.
struct WeightPullArgs {
  void* const* w_ptrs;          // R peers: [n_slot, elems_per_slot] bf16
  size_t elems_per_slot;
  const int32_t* slot_of;       // [E, R] weight slot of e on rank r (-1 none)
  const int32_t* main_rank;     // [E]
  const int32_t* home_index;    // [E] slot of e on its owner
  int E, R, me, home_cap, n_slot;
};
cudaError_t launch_weight_pull(const WeightPullArgs& a, cudaStream_t stream);

// Owner-side gradient return: for every expert owned by `me` with replicas, add the replicas'
// slot gradients (peer loads) into the owner's home slot gradient, accumulating in fp32.
// With `accum != nullptr` the sum (own slot + replicas) of EVERY home slot is added to
// accum[home] (fp32 or bf16, [home_cap, elems_per_slot]) instead of being written back to the slot:
// gradient accumulation over micro-batches, the slots being overwritten by each backward.
struct GradReduceArgs {
  void* const* g_ptrs;          // R peers: [n_slot, elems_per_slot] bf16
  void* accum;                  // optional accumulation buffer (local memory)
  int accum_fp32;               // dtype of accum: 1 fp32, 0 bf16
  int overwrite;                // 1: accum receives the sum (its previous content is not read)
  int include_self;             // 1: the owner's own contribution sits in slot_of[e, me] like any host's
                                //    (slot order = hosted experts by id); 0: it sits in the home slot
  size_t elems_per_slot;
  const int32_t* slot_of;       // [E, R]
  const int32_t* main_rank;     // [E]
  const int32_t* home_index;    // [E]
  int E, R, me, home_cap;
};
cudaError_t launch_grad_reduce(const GradReduceArgs& a, cudaStream_t stream);

// SwiGLU backward over the first *row_limit rows, in place over the saved pre-activations, one warp per
// row (16-byte accesses), after a plain Dgrad2 GEMM that wrote dact = dY W2 for the UNWEIGHTED gradient:
//   h[:, :F] <- p * dact * up * d/dg[g * sigmoid(g)],   h[:, F:] <- p * dact * g * sigmoid(g)
// with p = rowp[row] (null: 1).  With `dprob_ptrs != nullptr` the row's gate-weight gradient
// <dact, g * sigmoid(g) * up> is stored to dprob_ptrs[meta[row].x][meta[row].y] (the unit's source rank).
struct SwigluBwdArgs {
  const void* dact;             // bf16 [rows, F]
  void* h;                      // bf16 [rows, 2F] in/out
  int rows, F;
  const int32_t* row_limit;     // device: rows in use (may be null)
  const float* rowp;            // [rows] or null
  const int2* meta;             // [rows] {src rank, position at the source}; rows with src < 0 are padding
  float* const* dprob_ptrs;     // R peers: float [U] or null
};
cudaError_t launch_swiglu_backward(const SwigluBwdArgs& a, cudaStream_t stream);

// Wait on a flag nobody sets: exercises the bounded-wait / error-status path on one GPU.
cudaError_t launch_wait_probe(const unsigned* flag, unsigned target, unsigned long long budget_ns, int* status,
                              cudaStream_t stream);

}  // namespace epb
