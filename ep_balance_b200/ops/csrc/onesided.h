// One-sided transfers over the symmetric heap (onesided.cu).
//
// The reference moves replica weights and their gradients with device-initiated get/put kernels
// on NCCL symmetric windows (nccl_gin/csrc/nccl_gin.cu:730-811 batched get/put, 233-354 signals,
// 823-827 world fence).  On one NVSwitch box every peer window is mapped into this process, so the
// same operations are plain kernels over peer pointers: a batched descriptor copy that streams
// 8 KB tiles through shared memory with bulk async copies (no cluster multicast), signal words
// updated with release-scoped system atomics, and bounded waits that report through a status word.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace epb {

// One copy of `nbytes` between the window of rank `peer` (at byte `remote_off`) and the local
// buffer (at byte `local_off`).  Descriptors live in device memory as 4 x int64; `peer < 0` or
// `nbytes <= 0` marks an unused entry, which is skipped.
struct CopyDesc {
  int64_t peer, remote_off, local_off, nbytes;
};

struct BatchedCopyArgs {
  const CopyDesc* desc;          // [K] device
  int K;
  uint8_t* const* window_ptrs;   // [R] device: base address of the symmetric window on every rank
  uint8_t* local_base;           // base of the local side of every descriptor
  int R;
  int use_bulk;                  // 1: bulk async copies through shared memory; 0: 16-byte vector copies
  int* status;                   // status word (may be null)
};

// get: window[peer] + remote_off -> local_base + local_off.   put: the other direction, followed
// by a system-scope fence so that a later signal orders after the data.
// `blocks_per_desc` CTAs cooperate on each descriptor (grid = K x blocks_per_desc).
cudaError_t launch_get_batched(const BatchedCopyArgs& a, int blocks_per_desc, cudaStream_t stream);
cudaError_t launch_put_batched(const BatchedCopyArgs& a, int blocks_per_desc, cudaStream_t stream);

// Adds `value` to signal word `idx` of rank `peer` (all ranks when peer < 0) with release
// semantics at system scope: everything this stream wrote before is visible to a rank that
// observes the new value with an acquire load.
cudaError_t launch_signal(unsigned* const* signal_ptrs, int R, int peer, int idx, unsigned value,
                          cudaStream_t stream);

// Blocks the stream until the local word reaches `expected` (wrap-safe >=) or `budget_ns` passes;
// on timeout writes {kStatusSignalTimeout, site 70, idx} to `status` and returns.
cudaError_t launch_wait_signal(const unsigned* word, unsigned expected, int idx, unsigned long long budget_ns,
                               int* status, cudaStream_t stream);

}  // namespace epb
