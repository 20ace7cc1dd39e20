// Allocation-free variant of the plan solve: the solver's scratch lives in a file-scope device array.
// See no_alloc.h for who needs this and for the rules of use.
#include "no_alloc.h"

#include "solver.h"

namespace {

// Layout of the scratch array (byte offsets, every region 256-byte aligned).
constexpr size_t kAlign = 256;
constexpr size_t up(size_t n) { return (n + kAlign - 1) / kAlign * kAlign; }
constexpr size_t kOffErl = 0;                                                                   // int32 [E, R]
constexpr size_t kOffRankLoad = kOffErl + up(sizeof(int32_t) * EPB_NOALLOC_MAX_EXPERTS * EPB_NOALLOC_MAX_RANKS);
constexpr size_t kOffSlotUsed = kOffRankLoad + up(sizeof(int32_t) * EPB_NOALLOC_MAX_RANKS);      // int32 [R]
constexpr size_t kOffStuck = kOffSlotUsed + up(sizeof(int32_t) * EPB_NOALLOC_MAX_RANKS);         // uint8 [R]
constexpr size_t kOffZeroed = kOffStuck + up(EPB_NOALLOC_MAX_RANKS);  // sync[2] u32, status[4] i32, control[3] i64
constexpr size_t kZeroedBytes = 256;
constexpr size_t kScratchBytes = kOffZeroed + kZeroedBytes;

// In host code this name is only a handle for the runtime's symbol table, never an address a
// kernel can use; the usable device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_solver_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_addr[kMaxDevices] = {};
int g_last_cuda_error = 0;

// Device address of the scratch array on the current device, looked up once per device.
unsigned char* scratch_for_current_device() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    g_last_cuda_error = e != cudaSuccess ? (int)e : (int)cudaErrorInvalidDevice;
    return nullptr;
  }
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_solver_scratch);
    if (e != cudaSuccess || p == nullptr) {
      g_last_cuda_error = (int)e;
      return nullptr;
    }
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int epb_noalloc_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int epb_noalloc_status(int32_t* out4, cudaStream_t stream) {
  if (out4 == nullptr) return EPB_NOALLOC_BAD_ARGUMENT;
  unsigned char* base = scratch_for_current_device();
  if (base == nullptr) return EPB_NOALLOC_CUDA_ERROR;
  cudaError_t e = cudaMemcpyAsync(out4, base + kOffZeroed + 16, 4 * sizeof(int32_t), cudaMemcpyDeviceToDevice, stream);
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    return EPB_NOALLOC_CUDA_ERROR;
  }
  return EPB_NOALLOC_OK;
}

extern "C" int epb_solve_plan_noalloc(const int32_t* omega, const int32_t* dom, const int32_t* cost,
                                      const int32_t* main_rank, const int64_t* weight_bytes, int64_t s_tok, int R,
                                      int E, int D, int n_slot, int u_min, int iters, int allow_cross, int8_t* x,
                                      int32_t* q, int64_t* theta, cudaStream_t stream) {
  if (!omega || !dom || !cost || !main_rank || !weight_bytes || !x || !q || !theta) return EPB_NOALLOC_BAD_ARGUMENT;
  if (R < 1 || E < 1 || D < 1 || D > R || n_slot < 1 || u_min < 1 || iters < 1 || s_tok < 1)
    return EPB_NOALLOC_BAD_ARGUMENT;
  if (R > EPB_NOALLOC_MAX_RANKS || E > EPB_NOALLOC_MAX_EXPERTS) return EPB_NOALLOC_TOO_LARGE;

  unsigned char* base = scratch_for_current_device();
  if (base == nullptr) return EPB_NOALLOC_CUDA_ERROR;

  // Barrier counters, status and control words must read zero when the kernel starts; the rest
  // of the scratch is fully overwritten by the kernel before it is read.
  cudaError_t e = cudaMemsetAsync(base + kOffZeroed, 0, kZeroedBytes, stream);
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    return EPB_NOALLOC_CUDA_ERROR;
  }

  epb::SolverParams p{};
  p.omega = omega;
  p.dom = dom;
  p.cost = cost;
  p.main_rank = main_rank;
  p.weight_bytes = weight_bytes;
  p.s_tok = s_tok;
  p.R = R;
  p.E = E;
  p.D = D;
  p.n_slot = n_slot;
  p.u_min = u_min;
  p.iters = iters;
  p.patience = 8;
  p.allow_cross = allow_cross ? 1 : 0;
  p.probe = 0;
  p.x = x;
  p.q = q;
  p.theta = theta;
  p.erl = reinterpret_cast<int32_t*>(base + kOffErl);
  p.rank_load = reinterpret_cast<int32_t*>(base + kOffRankLoad);
  p.slot_used = reinterpret_cast<int32_t*>(base + kOffSlotUsed);
  p.stuck = base + kOffStuck;
  p.sync = reinterpret_cast<unsigned*>(base + kOffZeroed);
  p.status = reinterpret_cast<int*>(base + kOffZeroed + 16);
  p.control = reinterpret_cast<int64_t*>(base + kOffZeroed + 64);
  p.omega_signal = nullptr;
  p.omega_epoch = nullptr;
  epb::RankTables none{};
  none.me = -1;
  e = epb::launch_solver(p, none, stream);
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    return EPB_NOALLOC_CUDA_ERROR;
  }
  return EPB_NOALLOC_OK;
}
