// One-sided get/put over peer-mapped symmetric windows, signals and bounded signal waits.
//
// Copy engine: every warp owns a two-stage ring of 8 KB shared-memory tiles.  One lane issues a
// bulk async load (global -> shared, completion on an mbarrier), waits for the previous tile and
// issues its bulk async store (shared -> global).  Two loads per warp are in flight at any time,
// so a CTA of 8 warps keeps 128 KB outstanding, enough to cover NVLink latency with a few CTAs.
// No load names a cluster multicast; the source or the destination may be another GPU's memory.
// Ranges whose addresses are not 16-byte aligned take the vector/byte path.
#include "onesided.h"

#include "common.cuh"

namespace epb {
namespace {

constexpr int kCopyWarps = 8;
constexpr int kCopyThreads = kCopyWarps * 32;
constexpr int kTileBytes = 8192;
constexpr int kStages = 2;
constexpr int kCopySmem = kCopyWarps * kStages * kTileBytes + kCopyWarps * kStages * 8;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_init(uint64_t* bar) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void bar_expect(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded: false once the budget is spent (the caller records the status and stops issuing).
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
  unsigned long long t0 = 0;
  for (unsigned spin = 0;; ++spin) {
    if (bar_try(bar, parity)) return true;
    if ((spin & 1023u) == 1023u) {
      unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitBudgetNs) return false;
    }
  }
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_addr(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_addr(smem_src)), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Copies `nbytes` from src to dst with the CTAs blockIdx.y = 0..gridDim.y-1 of one descriptor.
template <bool kPut>
__device__ void copy_range(uint8_t* dst, const uint8_t* src, int64_t nbytes, int use_bulk, uint8_t* smem, int* status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool aligned = (((uintptr_t)dst | (uintptr_t)src) & 15u) == 0;
  const int64_t body = aligned ? (nbytes & ~(int64_t)15) : 0;  // bytes moved in 16-byte units

  if (use_bulk && aligned) {
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kCopyWarps * kStages * kTileBytes) + warp * kStages;
    uint8_t* ring = smem + (size_t)warp * kStages * kTileBytes;
    if (lane == 0) {
      bar_init(&bars[0]);
      bar_init(&bars[1]);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      const int64_t n_tiles = (body + kTileBytes - 1) / kTileBytes;
      const int64_t warps_total = (int64_t)gridDim.y * kCopyWarps;
      int64_t tile = (int64_t)blockIdx.y * kCopyWarps + warp;
      int64_t prev_off = -1;
      uint32_t prev_bytes = 0;
      bool ok = true;
      int it = 0, late_it = -1;
      for (; tile < n_tiles && ok; tile += warps_total, ++it) {
        const int s = it & 1;
        const int64_t off = tile * kTileBytes;
        const uint32_t bytes = (uint32_t)min((int64_t)kTileBytes, body - off);
        if (it >= 2) bulk_wait_read_all();  // the store that last read this stage has drained it
        bar_expect(&bars[s], bytes);
        bulk_load(ring + s * kTileBytes, src + off, bytes, &bars[s]);
        if (it >= 1) {
          const int ps = (it - 1) & 1;
          ok = bar_wait(&bars[ps], ((it - 1) >> 1) & 1);
          if (ok) bulk_store(dst + prev_off, ring + ps * kTileBytes, prev_bytes);
          else late_it = it - 1;  // this load is still in flight
        }
        prev_off = off;
        prev_bytes = bytes;
      }
      if (it >= 1) {
        // Loads always land eventually (their sources are valid memory).  Wait once more, bounded, for
        // every load still in flight -- the last one issued and, after a timeout, the one that was late --
        // so that no copy targets this CTA's shared memory after it exits.
        const int ps = (it - 1) & 1;
        const bool landed = bar_wait(&bars[ps], ((it - 1) >> 1) & 1);
        if (ok && landed) bulk_store(dst + prev_off, ring + ps * kTileBytes, prev_bytes);
        ok = ok && landed;
        if (late_it >= 0) bar_wait(&bars[late_it & 1], (late_it >> 1) & 1);
      }
      bulk_wait_all();
      if (!ok) set_status(status, kStatusPipeTimeout, 71, (int)blockIdx.x);
      asm volatile("fence.proxy.async;" ::: "memory");
    }
  } else if (aligned) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    const int64_t n = body / 16;
    const int64_t stride = (int64_t)gridDim.y * blockDim.x;
    int64_t i = (int64_t)blockIdx.y * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n; i += 4 * stride) {
      uint4 v0 = s4[i], v1 = s4[i + stride], v2 = s4[i + 2 * stride], v3 = s4[i + 3 * stride];
      d4[i] = v0;
      d4[i + stride] = v1;
      d4[i + 2 * stride] = v2;
      d4[i + 3 * stride] = v3;
    }
    for (; i < n; i += stride) d4[i] = s4[i];
  }
  // tail (or the whole range when unaligned): bytes, spread over the descriptor's CTAs
  {
    const int64_t stride = (int64_t)gridDim.y * blockDim.x;
    for (int64_t i = body + (int64_t)blockIdx.y * blockDim.x + threadIdx.x; i < nbytes; i += stride) dst[i] = src[i];
  }
  if (kPut) __threadfence_system();
}

template <bool kPut>
__global__ void __launch_bounds__(kCopyThreads) copy_batched_kernel(BatchedCopyArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const CopyDesc d = a.desc[blockIdx.x];
  if (d.peer < 0 || d.nbytes <= 0) return;
  if (d.peer >= a.R) {
    if (threadIdx.x == 0) set_status(a.status, kStatusBadArgument, 72, (int)blockIdx.x);
    return;
  }
  uint8_t* remote = a.window_ptrs[d.peer] + d.remote_off;
  uint8_t* local = a.local_base + d.local_off;
  if (kPut) copy_range<true>(remote, local, d.nbytes, a.use_bulk, smem, a.status);
  else copy_range<false>(local, remote, d.nbytes, a.use_bulk, smem, a.status);
}

__global__ void signal_kernel(unsigned* const* signal_ptrs, int R, int peer, int idx, unsigned value) {
  __threadfence_system();
  if (peer >= 0) {
    if (threadIdx.x == 0) red_release_sys_add(signal_ptrs[peer] + idx, value);
  } else if ((int)threadIdx.x < R) {
    red_release_sys_add(signal_ptrs[threadIdx.x] + idx, value);
  }
}

__global__ void wait_signal_kernel(const unsigned* word, unsigned expected, int idx, unsigned long long budget_ns,
                                   int* status) {
  if (threadIdx.x == 0 && !wait_ge<true>(word, expected, budget_ns)) set_status(status, kStatusSignalTimeout, 70, idx);
  __threadfence_system();
}

template <bool kPut>
cudaError_t launch_copy(const BatchedCopyArgs& a, int blocks_per_desc, cudaStream_t stream) {
  if (a.K <= 0) return cudaSuccess;
  if (blocks_per_desc < 1) blocks_per_desc = 1;
  if (blocks_per_desc > 65535) return cudaErrorInvalidValue;
  static bool attr_set[2][kMaxTrackedDevices] = {};
  int dev;
  if (device_needs_setup(attr_set[kPut], &dev)) {
    cudaError_t e = cudaFuncSetAttribute(copy_batched_kernel<kPut>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCopySmem);
    if (e != cudaSuccess) return e;
    device_setup_done(attr_set[kPut], dev);
  }
  dim3 grid(a.K, blocks_per_desc);
  copy_batched_kernel<kPut><<<grid, kCopyThreads, a.use_bulk ? kCopySmem : 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_get_batched(const BatchedCopyArgs& a, int blocks_per_desc, cudaStream_t stream) {
  return launch_copy<false>(a, blocks_per_desc, stream);
}
cudaError_t launch_put_batched(const BatchedCopyArgs& a, int blocks_per_desc, cudaStream_t stream) {
  return launch_copy<true>(a, blocks_per_desc, stream);
}

cudaError_t launch_signal(unsigned* const* signal_ptrs, int R, int peer, int idx, unsigned value, cudaStream_t stream) {
  if (R > 1024 || peer >= R) return cudaErrorInvalidValue;
  const int threads = peer >= 0 ? 32 : ((R + 31) / 32) * 32;
  signal_kernel<<<1, threads, 0, stream>>>(signal_ptrs, R, peer, idx, value);
  return cudaGetLastError();
}

cudaError_t launch_wait_signal(const unsigned* word, unsigned expected, int idx, unsigned long long budget_ns,
                               int* status, cudaStream_t stream) {
  wait_signal_kernel<<<1, 32, 0, stream>>>(word, expected, idx, budget_ns, status);
  return cudaGetLastError();
}

}  // namespace epb
