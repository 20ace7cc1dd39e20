// Plan solve for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project.  It exists for code that runs
// where cudaMalloc is off limits: inside a region that has handed all device memory to its own
// pool, in a process that shares a GPU under a fixed memory reservation, or in a plug-in whose
// host forbids allocation calls after start-up.  Such a caller owns its input and output buffers
// and passes them in; everything else the solver needs lives in a fixed array inside this library.
//
// Limits and rules
//   * Problem size is bounded: R <= EPB_NOALLOC_MAX_RANKS and E <= EPB_NOALLOC_MAX_EXPERTS.
//     Larger problems are rejected with EPB_NOALLOC_TOO_LARGE and nothing is launched.
//   * The scratch array (about 260 KB) is part of the loaded library image: every GPU that loads
//     the library holds it until the process exits.
//   * The first call on a device looks up the array's device address.  Make that first call
//     before starting any stream capture on that device.
//   * All calls on one device share the scratch array, and it keeps whatever the last call left
//     there.  The words that must start at zero are cleared on the caller's stream before every
//     launch.  Two calls whose GPU work overlaps (different streams, no ordering) race on the
//     array; order them.
//   * The call enqueues work on `stream` and returns; it does not synchronise.  EPB_NOALLOC_OK therefore
//     only means "enqueued".  Whether the kernel ran to the end is in its status word, which lives in the
//     scratch array: copy it out with epb_noalloc_status() on the same stream and read it once the stream
//     has been synchronised.  A non-zero code (a bounded wait ran out, a rank's domain id was outside
//     0..D-1) means x, q and theta are not a valid plan.
//   * The repair loop runs `iters` rounds per domain; the optional stagnation probe of the tensor entry
//     point (EPLBConfig.stage2_patience_all_scales) is not available here.
//   * Host side: the functions keep a per-device address table and a last-error word without locking.
//     Call them from one thread at a time (per process).
//   * No cudaMalloc, cudaFree or allocating library routine is called.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define EPB_NOALLOC_MAX_RANKS 64
#define EPB_NOALLOC_MAX_EXPERTS 1024

#define EPB_NOALLOC_OK 0
#define EPB_NOALLOC_TOO_LARGE 1     // R or E beyond the maxima above
#define EPB_NOALLOC_BAD_ARGUMENT 2  // null pointer or non-positive size / knob
#define EPB_NOALLOC_CUDA_ERROR 3    // a CUDA call failed; see epb_noalloc_last_cuda_error()

#ifdef __cplusplus
extern "C" {
#endif

// Solve one plan.  All pointers are device pointers on the current device.
//   omega        int32 [R, E]     units routed from source rank r to expert e
//   dom          int32 [R]        domain of each rank (0 .. D-1)
//   cost         int32 [R, R]     per-token cost, zero diagonal
//   main_rank    int32 [E]        owner of each expert
//   weight_bytes int64 [E]
//   x            int8  [E, R]     out: placement
//   q            int32 [R, E, R]  out: routing quota q[src, expert, dst]
//   theta        int64 [1]        out: maximum rank load
// Knobs as in EPLBConfig: n_slot (total slots per rank), u_min, iters (repair rounds per domain),
// allow_cross (0/1).  Returns one of the EPB_NOALLOC_* codes.
int epb_solve_plan_noalloc(const int32_t* omega, const int32_t* dom, const int32_t* cost, const int32_t* main_rank,
                           const int64_t* weight_bytes, int64_t s_tok, int R, int E, int D, int n_slot, int u_min,
                           int iters, int allow_cross, int8_t* x, int32_t* q, int64_t* theta, cudaStream_t stream);

// Copy the status word {code, site, detail, 0} of the last solve enqueued on this device into `out4`
// (device memory of the caller, 4 x int32), ordered after that solve on `stream`.  Codes as in the
// library's status words: 0 ok, 1 barrier timeout, 5 bad argument.  Allocates nothing.
int epb_noalloc_status(int32_t* out4, cudaStream_t stream);

// CUDA error code (cudaError_t as int) of the last failing CUDA call made by the functions above.
int epb_noalloc_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
