// Host-visible interface of the on-device plan solver (solver.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace epb {

struct SolverParams {
  // inputs (device pointers)
  const int32_t* omega;         // [R, E] units routed from source rank r to expert e
  const int32_t* dom;           // [R] domain of each rank
  const int32_t* cost;          // [R, R] per-token cost
  const int32_t* main_rank;     // [E] owner of each expert
  const int64_t* weight_bytes;  // [E]
  int64_t s_tok;
  int R, E, D, n_slot, u_min, iters, patience, allow_cross, probe;
  int cache_q;                  // set by launch_solver: ... and the quota columns it moves
  int cache_stage2;             // set by launch_solver: repair loop keeps erl/x of its domain in shared memory
  // outputs
  int8_t* x;              // [E, R]
  int32_t* q;             // [R, E, R]; every element is written, no pre-zeroing needed
  int32_t* erl;           // [E, R] units each rank computes for each expert
  int32_t* rank_load;     // [R]
  int32_t* slot_used;     // [R]
  unsigned char* stuck;   // [R]
  int64_t* theta;         // [1]
  int64_t* control;       // [3] probe-mode control words (may be null)
  int64_t* trace;         // optional [8]: CTA 0 stores the global timer (ns) at its phase boundaries (profiling aid)
  // workspace
  unsigned* sync;         // [2] grid-barrier arrival / departure counters, zero when idle
  int* status;            // [4] error status (see common.cuh), zero when healthy
  // optional: wait until *omega_signal >= (*omega_epoch) * R before reading omega.  The epoch
  // word counts this rank's publishes (advanced by count_publish_kernel earlier in the stream).
  const unsigned* omega_signal;
  const unsigned* omega_epoch;
};

// Routing tables of one rank `me`, derived from the final (x, q).
//
// Two orderings exist on a rank.  *Groups* are the row blocks of the receive buffers, each block starting on
// a multiple of `row_align`: with home slots, the experts the rank owns come first and its replicas after
// them, each by ascending id (owned groups can be computed while replica weights are still arriving); without
// home slots, all hosted experts by ascending id.  *Weight slots* say where an expert's weights live: an owner
// keeps expert e in home slot home_index[e] (< home_cap) for ever, replicas land in slots home_cap,
// home_cap+1, ... in ascending expert id.  With home_index == nullptr weight slots equal group indices
// (ascending id, the reference's physical slot order, eplb/integration/physical.py:23-27).
struct RankTables {
  int me;                 // -1: build nothing
  int n_slot;             // capacity of the per-group arrays
  int row_align;          // 128: the GEMM M tile
  int row_capacity;       // rows the receive buffers hold; 0 disables the guard
  int home_cap;
  const int32_t* home_index;  // [E] or null
  int32_t* slot_of;       // [E, R] weight slot of e on rank r, -1 if not hosted (may be null)
  int32_t* row_base;      // [E, R] first row in dst r's buffers for units (me, e) -> r; -1 if none
  int32_t* group_expert;  // [n_slot] expert of each group of `me`, -1 if unused
  int32_t* group_wslot;   // [n_slot] weight slot of each group
  int32_t* group_off;     // [n_slot + 1] first row of each group; last = padded total
  int32_t* group_rows;    // [n_slot] real rows in each group
  int32_t* totals;        // [2] padded rows, number of groups
  // optional, for the senders' transport (route.h, CommArgs):
  int32_t* send_off;      // [E, R] units (me, e) sent to ranks below dst = sum_{d < dst} q[me, e, d] (may be null)
  int32_t* tiles_of;      // [R] row_align-row tiles in use in every rank's receive buffer, clamped to row_capacity (may be null)
};

cudaError_t launch_solver(const SolverParams& p, const RankTables& tables, cudaStream_t stream);
cudaError_t launch_tables(const SolverParams& p, const RankTables& tables, cudaStream_t stream);

}  // namespace epb
