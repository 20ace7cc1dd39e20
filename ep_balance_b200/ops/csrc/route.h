// Token-path and weight-path kernels around the grouped GEMM (route.cu).
//
// "Peer pointer tables" are device arrays of R pointers, one per rank, to the same symmetric
// buffer on every rank.  On one GPU emulating R ranks they simply point at R local buffers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace epb {

// Histogram of this rank's routed expert ids, stored as row `me` of omega on every peer,
// followed by one release-add on every peer's signal word.
// `epoch_word` (local, may be null) is advanced by one per call.
cudaError_t launch_count_publish(const int64_t* unit_expert, int num_units, int E, int R, int me,
                                 int32_t* const* omega_ptrs, unsigned* const* signal_ptrs, unsigned* epoch_word,
                                 cudaStream_t stream);

// Unit -> (dst rank, row in dst's receive buffers).  q_me = q[me] as [E, R]; row_base from the
// solver's RankTables.
cudaError_t launch_route_assign(const int64_t* unit_expert, int num_units, int E, int R,
                                const int32_t* q_me, const int32_t* row_base, int32_t* unit_dst,
                                int32_t* unit_row, int* status, cudaStream_t stream);

// Copy (optionally scale) token rows into the peers' receive buffers and write {src rank, unit}
// beside each row.  Also zero-fills this rank's own padding rows (slot_off/slot_rows layout).
// With `saved_out != nullptr` also computes unit_dot[u] = <rows[t(u)], saved_out[u]> (the gate
// weight gradient) in the same pass.
struct DispatchArgs {
  const void* rows;             // bf16 [num_tokens, H]
  const float* unit_scale;      // [U] or null
  const void* saved_out;        // bf16 [U, H] or null
  float* unit_dot;              // [U] or null
  int num_units, topk, H, R, me;
  const int32_t* unit_dst;      // [U]
  const int32_t* unit_row;      // [U]
  void* const* buf_ptrs;        // R peers: bf16 [row_capacity, H]
  int2* const* meta_ptrs;       // R peers: int2 [row_capacity] or null
  void* local_buf;              // this rank's receive buffer (pad rows are zeroed here)
  const int32_t* slot_off;      // [n_slot + 1]
  const int32_t* slot_rows;     // [n_slot]
  int n_slot;
  int row_capacity;              // rows of every peer buffer; rows past it are dropped
};
cudaError_t launch_dispatch(const DispatchArgs& a, cudaStream_t stream);

// out[t] = sum_k scale[t*topk+k] * rows[t*topk+k]   (scale may be null: plain sum)
cudaError_t launch_unit_reduce(const void* unit_rows, const float* unit_scale, void* out, int num_tokens,
                               int topk, int H, cudaStream_t stream);

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

// SwiGLU backward over the first *row_limit rows, in place over the saved pre-activations:
//   h[:, :F] <- dact * up * d/dg[g * sigmoid(g)],   h[:, F:] <- dact * g * sigmoid(g)
// One fully coalesced pass (16-byte accesses); used after a plain Dgrad2 GEMM that wrote dact.
cudaError_t launch_swiglu_backward(const void* dact, void* h, int rows, int F, const int32_t* row_limit,
                                   cudaStream_t stream);

// Wait on a flag nobody sets: exercises the bounded-wait / error-status path on one GPU.
cudaError_t launch_wait_probe(const unsigned* flag, unsigned target, unsigned long long budget_ns, int* status,
                              cudaStream_t stream);

}  // namespace epb
