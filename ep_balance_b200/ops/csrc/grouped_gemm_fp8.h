// Block-scaled fp8 (e4m3) ragged grouped GEMM on tcgen05 with the scale factors in tensor memory
// (grouped_gemm_fp8.cu), plus the quantisers that produce its operands.
//
// The reference has no fp8 path (its expert GEMMs are torch._grouped_mm in bf16,
// eplb/integration/grouped_mlp.py:88-114); this is the DeepSeek-V3 recipe: activations scaled per
// 1 x 128 block, weights per 128 x 128 block.  Scales are powers of two stored as one biased
// exponent byte (UE8M0, value 2^(b-127)), which is what `tcgen05.mma.kind::mxf8f6f4.block_scale`
// consumes, so the products are rescaled inside the tensor core and the accumulator in TMEM is the
// final fp32 result: no per-k-block promotion pass over the accumulator is needed.
//
// Scale-factor layout ("chunk"): 512 bytes hold the scales of 128 rows (or weight columns) for four
// consecutive 128-wide k-blocks; byte (r % 32) * 16 + (r / 32) * 4 + kb % 4.  This is the order in
// which `tcgen05.cp.32x128b.warpx4` spreads a chunk over the 128 TMEM lanes, so a chunk goes
// global -> shared (bulk copy) -> tensor memory without being rearranged.
//   activations: sfa[row_tile][kgroup][512],  row_tile = row / 128, kgroup = k / 512
//   weights:     sfb[slot][n_tile][kgroup][512], n_tile = n / 128 (all 128 entries of a k-block equal)
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace epb {

struct Fp8GemmArgs {
  // group geometry (device), as in GemmArgs: groups start on multiples of 128 rows
  const int32_t* group_off;
  const int32_t* group_rows;
  const int32_t* group_wslot;
  const int32_t* totals;       // [2]: padded rows, number of groups
  int n_groups_cap;
  int row_capacity;
  int N;                       // output columns, multiple of 128
  int K;                       // reduction extent, multiple of 128
  const uint8_t* sfa;          // [row_capacity / 128][kgroups][512]
  const uint8_t* sfb;          // [slots][N / 128][kgroups][512]
  void* out;                   // bf16 [row_capacity, N] (rows kept local), or
  void* const* out_ptrs;       // R peer buffers [units, N]: row r goes to out_ptrs[meta[r].x] row meta[r].y
  const int2* meta;
  int* status;
};

// Tensor maps over the e4m3 bytes: A [rows, K], B [slots, N, K]; boxes of 128 x 128 bytes, 128-byte swizzle.
bool make_tmap_fp8_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols);
bool make_tmap_fp8_3d(CUtensorMap* out, const void* base, uint64_t slots, uint64_t rows, uint64_t cols,
                      uint32_t box_rows = 128);
// Scale chunks as a [chunks, 128] int32 tensor (one 512-byte chunk per row, no swizzle).
bool make_tmap_sf(CUtensorMap* out, const void* base, uint64_t chunks);

cudaError_t launch_grouped_gemm_fp8(const CUtensorMap& tmA, const CUtensorMap& tmB, const Fp8GemmArgs& args,
                                    int num_sms, cudaStream_t stream);

// Optional description of which rows of a buffer hold data (device tables of the group layout): row r
// is real when group_off[g] <= r < group_off[g] + group_rows[g] for some g < min(totals[1], n_groups_cap).
struct RowGroups {
  const int32_t* group_off;
  const int32_t* group_rows;
  const int32_t* totals;
  int n_groups_cap;
};

// CTA-pair variant (thread-block cluster of two SMs, cta_group::2): 256 x 256 tiles with one accumulator when
// N % 256 == 0 (`tmB` box_rows = 128), else 256 x 128 tiles with two accumulators (`tmB` box_rows = 64).
// Groups must start on multiples of 256 rows; scale chunks are fetched through `tmSFA` / `tmSFB`.
cudaError_t launch_grouped_gemm_fp8_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmSFA,
                                         const CUtensorMap& tmSFB, const Fp8GemmArgs& args, int num_sms,
                                         cudaStream_t stream);

// bf16 [rows, K] -> e4m3 [rows, K] + 1 x 128 scales in chunk layout.  rows % 128 == 0, K % 128 == 0.
// `groups` (may be null): only real rows are processed; the rest keep whatever they held.
cudaError_t launch_quantize_rows(const void* x, uint8_t* q, uint8_t* sfa, int rows, int K, const RowGroups* groups,
                                 cudaStream_t stream);
// h bf16 [rows, 2F] (gate columns, then up columns) -> silu(gate) * up as e4m3 [rows, F] + scales;
// `act` (bf16 [rows, F], may be null) also receives the unquantised activation.
cudaError_t launch_swiglu_quantize(const void* h, uint8_t* q, uint8_t* sfa, void* act, int rows, int F,
                                   const RowGroups* groups, cudaStream_t stream);
// Dispatch fused with the 1 x 128 quantisation: every routed unit's token row is quantised in registers and
// stored as e4m3 bytes (plus its scale bytes) straight into the destination rank's operand buffer, so half
// the bytes of a bf16 dispatch cross NVLink and no separate quantisation pass runs on the receiver.
struct DispatchFp8Args {
  const void* rows;             // bf16 [num_tokens, H]
  int num_units, topk, H, R, me;
  const int32_t* unit_dst;      // [U]
  const int32_t* unit_row;      // [U]
  const int32_t* unit_pos;      // [U] position of the unit in the source's expert-sorted order (where its row returns)
  uint8_t* const* xq_ptrs;      // R peers: e4m3 [row_capacity, H]
  uint8_t* const* sfx_ptrs;     // R peers: scale chunks [row_capacity / 128][kgroups][512]
  int2* const* meta_ptrs;       // R peers: {src rank, position at the source} per row
  int row_capacity;
};
cudaError_t launch_dispatch_fp8(const DispatchFp8Args& a, cudaStream_t stream);

// bf16 [slots, N, K] -> e4m3 + 128 x 128 scales in chunk layout.  N % 128 == 0, K % 128 == 0.
cudaError_t launch_quantize_weights(const void* w, uint8_t* q, uint8_t* sfb, int slots, int N, int K,
                                    cudaStream_t stream);

}  // namespace epb
