// Ragged grouped GEMM on the 5th-generation tensor cores (grouped_gemm.cu).
//
// One persistent kernel (one CTA per SM) covers the six expert GEMMs of an MoE layer step:
//   kFwd1    h = X W1^T  with SwiGLU epilogue        (A K-major, B K-major, gate/up pair per tile)
//   kFwd2    y = act W2^T, rows scattered to sources  (A K-major, B K-major)
//   kDgrad2  dact = dY W2, act-grad fused, in place   (A K-major, B MN-major)
//   kDgrad1  dX = dH W1, rows scattered to sources    (A K-major, B MN-major)
//   kWgrad   dW[slot] = P^T Q over the slot's rows    (A MN-major, B MN-major, K = ragged rows)
//   kPlain   C = A B^T per group, rows kept local      (testing / generic use)
// Group geometry (row offsets, row counts, weight slots) is read from device memory, so the host
// never learns the routing outcome.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "route.h"

namespace epb {

enum GemmMode : int { kFwd1 = 0, kFwd2 = 1, kDgrad2 = 2, kDgrad1 = 3, kWgrad = 4, kPlain = 5 };

struct GemmArgs {
  int mode;
  int ctas;                    // 1: one CTA per 128-row tile; 2: CTA pair (cta_group::2) per 256-row tile.
                               // Groups must start on multiples of 128 * ctas rows.
  // group geometry (device)
  const int32_t* group_off;    // [n_groups_cap + 1] first row of each group (multiple of 128 * ctas)
  const int32_t* group_rows;   // [n_groups_cap]
  const int32_t* group_wslot;  // [n_groups_cap]
  const int32_t* totals;       // [2]: padded rows, number of groups
  int n_groups_cap;
  int row_capacity;            // rows of the token buffers; tiles never write past it
  // problem extents
  int N;                       // output columns (kFwd1: F, gate/up pairs; kWgrad: columns of Q)
  int K;                       // reduction extent (ignored for kWgrad: the group's padded rows)
  int M_out;                   // kWgrad only: rows of the output (columns of P)
  // epilogue operands
  void* out0;                  // kFwd1: h [T, 2N];  kDgrad2: h (in/out);  kWgrad: dW [slots, M_out, N];
                               // kPlain: C [T, N];  scatter modes with out_ptrs == null: local [T, N]
  void* out1;                  // kFwd1: act [T, N]
  const float* row_scale;      // kFwd1: optional [T] factor folded into act (the row's gate weight); null: 1
  void* const* out_ptrs;       // scatter modes: R peer buffers [units, N] (null -> local out0)
  const int2* meta;            // scatter modes: {src rank, row in that rank's buffer} per row
  int* status;
  unsigned long long wait_ns;  // budget of the waits below (0: the library default)
  // ---- operand gating (each may be null).  The TMA producer polls before the first load of a tile:
  // the A rows of M-tile i are complete when arrive[i] >= arrive_expected (counters written by the
  // senders' transport, CommArgs); the weights of replica slot s (wslot - home_cap) are complete when
  // pull_cnt[s] >= pull_expected.  kWgrad waits for every M-tile of the group.
  const unsigned* arrive;
  unsigned arrive_expected;
  const unsigned* pull_cnt;
  unsigned pull_expected;
  int home_cap;
  // ---- completion signal of the scatter modes (null: none).  The last CTA to finish advances the
  // local epoch word and adds 1 (release, system scope) to word `done_slot` of every peer's signal
  // array: "all rows this rank owes you are stored".  done_ctr is zero between launches.
  unsigned* done_ctr;
  unsigned* done_epoch;
  unsigned* const* done_signal_ptrs;
  int done_slot, done_R;
  // ---- fused transport (comm.do_* all zero: none).  Two extra warps per CTA run the item-driven
  // transport of CommArgs while the other warps compute: with kFwd1 they send token rows and pull
  // replica weights, with kDgrad1 (used as the plain Dgrad2) they send output gradients; the producer
  // of the same kernel -- on every rank -- gates its tiles on the arrival counters those warps advance.
  CommArgs comm;
  // ---- optional profiling aid: unsigned long long [12] in device memory, set to {~0, 0, 0, ~0, -, -, -, -, 0, 0, 0, 0}
  // before the launch.  The kernel leaves {earliest start of a transport warp, latest end of a transport warp,
  // latest end of an MMA issuer, earliest moment an MMA issuer had the operands of its first tile} as
  // global-timer values (ns) and, in words 8..11, sums over all transport warps of {ns waiting for loads,
  // ns waiting for stores to release ring slots, ns draining at block ends, segments moved}.
  unsigned long long* trace;
};

// Host-side tensor-map helpers (driver entry point fetched at run time; no -lcuda needed).
// 2-D: tensor [rows, cols] row-major bf16, box {box_cols, box_rows}, 128-byte swizzle.
bool make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols,
                  uint32_t box_rows);
// 3-D: tensor [slots, rows, cols] bf16, box {box_cols, box_rows, 1}.
bool make_tmap_3d(CUtensorMap* out, const void* base, uint64_t slots, uint64_t rows, uint64_t cols,
                  uint32_t box_cols, uint32_t box_rows);

cudaError_t launch_grouped_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& args, int num_sms,
                                cudaStream_t stream);

}  // namespace epb
