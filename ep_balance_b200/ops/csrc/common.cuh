// Shared device helpers: bounded waits, status words, small PTX wrappers.
//
// Every wait in this library is bounded.  When a wait runs out the kernel records
// {code, site} in a status word that the host reads after the step, releases what it
// holds and returns; nothing traps, asserts or spins forever.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace epb {

// Status codes written to status[0]; status[1] = site id, status[2] = extra detail.
enum StatusCode : int {
  kStatusOk = 0,
  kStatusBarrierTimeout = 1,   // grid or cross-rank barrier did not complete in time
  kStatusSignalTimeout = 2,    // a peer's signal did not arrive in time
  kStatusPipeTimeout = 3,      // an mbarrier of the GEMM pipeline did not flip in time
  kStatusRowOverflow = 4,      // received rows exceed the buffer capacity
  kStatusBadArgument = 5,
};

__device__ __forceinline__ void set_status(int* status, int code, int site, int detail = 0) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = site;
    status[2] = detail;
  }
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Spin until *p >= target (wrap-safe signed difference) or the time budget is spent.
// Returns false on timeout.  `sys` selects system scope (peer GPUs write the word).
template <bool kSys>
__device__ __forceinline__ bool wait_ge(const unsigned* p, unsigned target, unsigned long long budget_ns) {
  unsigned long long t0 = 0;
  for (unsigned spin = 0;; ++spin) {
    unsigned v = kSys ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if ((int)(v - target) >= 0) return true;
    if ((spin & 255u) == 255u) {
      unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) return false;
    }
    if (spin > 64u) __nanosleep(32);  // back off only after a burst of immediate polls
  }
}

constexpr unsigned long long kWaitBudgetNs = 1500ull * 1000ull * 1000ull;  // 1.5 s

// Host helper: "has this per-device one-time set-up been done on the current device?".  Function
// attributes such as the dynamic shared-memory limit belong to (kernel, device), so a process that
// drives several GPUs must set them on each.  `done` is a caller-owned table of kMaxTrackedDevices
// flags; devices beyond the table are configured on every call.
constexpr int kMaxTrackedDevices = 64;
inline bool device_needs_setup(bool* done, int* dev_out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
  *dev_out = dev;
  return dev < 0 || dev >= kMaxTrackedDevices || !done[dev];
}
inline void device_setup_done(bool* done, int dev) {
  if (dev >= 0 && dev < kMaxTrackedDevices) done[dev] = true;
}

__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ int round_up(int a, int b) { return (a + b - 1) / b * b; }

}  // namespace epb
