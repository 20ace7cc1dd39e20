// Ragged grouped GEMM for sm_100a: TMA-fed shared-memory tiles, tcgen05.mma issued by one thread,
// accumulators in tensor memory, epilogue warps reading them back with tcgen05.ld.
//
// CTA = 10 warps: warp 0 issues TMA loads, warp 1 owns TMEM and issues MMAs, warps 2-9 run the
// epilogue (two warps per 32-lane quarter of TMEM, each taking half of the tile's columns).  A 4- to 6-stage
// smem ring (A 16 KB + B 32 or 16 KB per stage, see Geometry) feeds 128x256x16 UMMAs; two 256-column accumulators
// in TMEM let the epilogue of tile i overlap the main loop of tile i+1.  The kernel is persistent: CTA c processes
// tiles c, c+grid, ... of a tile list derived on device from the plan's group table.  The variants with kComm = 1
// carry two more warps that move token (or gradient) rows and replica weights between ranks (comm.cuh) while the
// producer warp gates each tile's first load on the arrival counter of that tile.
//
// This replaces torch._grouped_mm / torch.bmm plus the unfused activation, slot sort, index_add
// and activation-gradient kernels of the reference (eplb/integration/grouped_mlp.py:88-137,
// 219-236; overlap.py:368-408; manual_block.py:184-221, 293-342).
//
// Every mbarrier wait is bounded; on timeout the CTA records a status, stops issuing work,
// lets its outstanding copies land, frees its tensor memory and returns.
#include "grouped_gemm.h"

#include <cuda_bf16.h>

#include "comm.cuh"
#include "common.cuh"

namespace epb {
namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;  // 16 KB: this CTA's 128 rows of the A tile
constexpr int TMEM_COLS = 512;

// kCtas = 1: one CTA computes a 128 x 256 tile.  kCtas = 2: a CTA pair (thread-block cluster of
// two SMs) computes a 256 x 256 tile with tcgen05.mma.cta_group::2; each CTA stages its own 128
// rows of A and its own 128 columns of B, so per-SM operand traffic drops from 48 KB to 32 KB per
// k-block and the shared-memory ring deepens from 4 to 6 stages.
// The fused-transport variants (kComm != 0) give 64 KB of the operand ring to the transport warps' copy rings.
template <int kCtas, int kComm = 0>
struct Geometry {
  static constexpr int STAGES = (kCtas == 2 ? 6 : 4) - (kComm ? (kCtas == 2 ? 2 : 1) : 0);
  static constexpr int COMM_SLOTS = kCtas == 2 ? 8 : 6;  // ring slots of a transport warp: batches of 4 (3) segments of 4 KB
  static constexpr int B_BYTES = BN * BK * 2 / kCtas;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TILE_M = BM * kCtas;
};
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address
constexpr int NUM_THREADS = 320;  // TMA warp + MMA warp + 8 epilogue warps
constexpr int COMM_WARPS = 2;     // transport warps of the fused variants (warps 10, 11): 384 threads keep the 168-register budget
constexpr int MAX_GROUPS = 320;  // barriers + flags + (MAX_GROUPS + 1) ints must fit in kCtrlBytes
constexpr int kCtrlBytes = 1536;
static_assert((6 * 2 + 4) * 8 + 8 + (MAX_GROUPS + 1) * 4 <= kCtrlBytes, "control block does not fit");
constexpr int kStageWarpBytes = 4096;  // staging tile of one epilogue warp

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false (and raises the CTA's abort flag) when the budget is spent.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int site) {
  unsigned long long t0 = 0;
  for (unsigned spin = 0;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 1023u) {
      if (*abort_flag) return false;
      unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitBudgetNs) {
        *abort_flag = 1;
        set_status(status, kStatusPipeTimeout, site, (int)blockIdx.x);
        return false;
      }
    }
  }
}

// Bounded wait on a counter in global memory (kSys: peers write it over NVLink).  Followed by a
// proxy fence: the data it guards was written through the generic proxy (peer or local stores) and is
// read next by TMA, i.e. through the async proxy.
template <bool kSys>
__device__ __forceinline__ bool flag_wait(const unsigned* p, unsigned target, unsigned long long budget_ns,
                                          volatile int* abort_flag, int* status, int site, int detail) {
  unsigned long long t0 = 0;
  for (unsigned spin = 0;; ++spin) {
    const unsigned v = kSys ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if ((int)(v - target) >= 0) break;
    if ((spin & 63u) == 63u) {
      if (*abort_flag) return false;
      unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) {
        *abort_flag = 1;
        set_status(status, kStatusSignalTimeout, site, detail);
        return false;
      }
    }
    if (spin > 16u) __nanosleep(64);
  }
  asm volatile("fence.proxy.async.global;" ::: "memory");
  return true;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// ---- CTA-pair variants (thread-block cluster of 2; no multicast anywhere)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(saddr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Loads of a CTA pair complete on the barrier of the pair's even-ranked CTA (rank bit cleared).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & kPeerBitMask), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & kPeerBitMask), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
template <int kCtas>
__device__ __forceinline__ void tma2(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  if (kCtas == 2) tma_load_2d_pair(dst, map, bar, c0, c1);
  else tma_load_2d(dst, map, bar, c0, c1);
}
template <int kCtas>
__device__ __forceinline__ void tma3(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  if (kCtas == 2) tma_load_3d_pair(dst, map, bar, c0, c1, c2);
  else tma_load_3d(dst, map, bar, c0, c1, c2);
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on ONE barrier (own or the peer's, given as a shared::cluster address) once every MMA
// issued so far by the pair has completed.  Both CTAs are told with two of these.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor, 128-byte swizzle, tile base 1024-byte aligned.
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 version (1 on sm_100)   bits 61-63 layout (2 = SW128)
// K-major:  rows are 128 B apart, 8-row groups are SBO = 1024 B apart; LBO is unused.
// MN-major: 64 contiguous MN elements per 128-B row of k; 8-k groups are SBO = 1024 B apart and
//           the next 64 MN elements start LBO = BK*128 B = 8192 B further (one TMA box each).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor for kind::f16: bf16 x bf16 -> fp32; M = 128 (one CTA) or 256 (CTA pair).
__host__ __device__ constexpr uint32_t make_idesc(bool a_mn, bool b_mn, int n, int m) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---------------------------------------------------------------- tiles
struct Tile {
  int g, mt, nt;
  int rows;      // real rows of the group
  int row0;      // first buffer row of the group
  int wslot;
  int kblocks;
};

struct Shape {
  int n_groups, n_tiles_n, tile_n, m_tiles_fixed, kblocks_fixed;
};

template <int kMode, int kCtas>
__device__ __forceinline__ Shape make_shape(const GemmArgs& a) {
  Shape s;
  int ng = a.totals[1];
  s.n_groups = ng < a.n_groups_cap ? ng : a.n_groups_cap;
  s.tile_n = kMode == kFwd1 ? 128 : BN;
  s.n_tiles_n = ceil_div(a.N, s.tile_n);
  s.m_tiles_fixed = kMode == kWgrad ? ceil_div(a.M_out, Geometry<kCtas>::TILE_M) : 0;
  s.kblocks_fixed = kMode == kWgrad ? 0 : ceil_div(a.K, BK);
  return s;
}

template <int kMode>
__device__ __forceinline__ bool find_tile(const GemmArgs& a, const Shape& s, const int* tile_prefix, int t, Tile& out) {
  int g = 0;
  while (g < s.n_groups && t >= tile_prefix[g + 1]) ++g;
  if (g >= s.n_groups) return false;
  const int local = t - tile_prefix[g];
  out.g = g;
  out.mt = local / s.n_tiles_n;
  out.nt = local - out.mt * s.n_tiles_n;
  out.rows = a.group_rows[g];
  out.row0 = a.group_off[g];
  out.wslot = a.group_wslot[g];
  out.kblocks = kMode == kWgrad ? ceil_div(out.rows, BK) : s.kblocks_fixed;
  return true;
}

// ---------------------------------------------------------------- epilogue helpers
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
}
__device__ __forceinline__ float sigmoidf_fast(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// ---------------------------------------------------------------- staged, row-contiguous stores
// A warp's staging tile holds 32 rows x 64 B (4 pieces of 16 B per row).  Piece p of row r lives at
// index r*4 + (p ^ ((r >> 1) & 3)), which makes both the row-wise writes (lane = row) and the
// flush reads (8 rows x 4 pieces per instruction) free of bank conflicts.
__device__ __forceinline__ int stage_index(int r, int p) { return r * 4 + (p ^ ((r >> 1) & 3)); }

__device__ __forceinline__ void pack_row(const uint32_t (&r)[32], uint4 (&out)[4], bool keep) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[i].x = keep ? pack_bf16(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1])) : 0u;
    out[i].y = keep ? pack_bf16(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3])) : 0u;
    out[i].z = keep ? pack_bf16(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5])) : 0u;
    out[i].w = keep ? pack_bf16(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7])) : 0u;
  }
}
// lane = row: write the lane's 64 B
__device__ __forceinline__ void stage_store(uint4* tile, int lane, const uint4 (&p)[4]) {
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) tile[stage_index(lane, i)] = p[i];
  __syncwarp();
}
// Direct per-thread access to 64 B of the lane's own row (null row: zeros / skipped).
__device__ __forceinline__ void row_load(const char* rowptr, int byte_off, uint4 (&regs)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
    regs[i] = rowptr ? *reinterpret_cast<const uint4*>(rowptr + byte_off + i * 16) : make_uint4(0, 0, 0, 0);
}
__device__ __forceinline__ void row_store(char* rowptr, int byte_off, const uint4 (&regs)[4]) {
  if (rowptr == nullptr) return;
#pragma unroll
  for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(rowptr + byte_off + i * 16) = regs[i];
}
// Write the tile out: instruction `it` covers rows it*8 .. it*8+7, four lanes per row.  `rowptr`
// is each lane's own row base (null: skip the row); the owner lane's pointer is fetched by shuffle.
__device__ __forceinline__ void stage_flush(const uint4* tile, int lane, char* rowptr, int byte_off) {
  const unsigned long long mine = reinterpret_cast<unsigned long long>(rowptr);
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int r = it * 8 + (lane >> 2), p = lane & 3;
    const unsigned long long base = __shfl_sync(0xffffffffu, mine, r);
    if (base != 0ull) *reinterpret_cast<uint4*>(base + byte_off + p * 16) = tile[stage_index(r, p)];
  }
}
// Wide variant for rows that may live on another GPU: the tile holds 32 rows x 128 B (8 pieces per
// row, piece p of row r at r*8 + (p ^ (r & 7))), filled 64 B at a time and flushed with four rows x
// 128 contiguous bytes per instruction, so peer stores leave the SM as full 128-byte segments.
__device__ __forceinline__ int wide_index(int r, int p) { return r * 8 + (p ^ (r & 7)); }
__device__ __forceinline__ void wide_store_half(uint4* tile, int lane, const uint4 (&p)[4], int half) {
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) tile[wide_index(lane, half * 4 + i)] = p[i];
  __syncwarp();
}
// `pieces` = 8 (both halves valid) or 4 (only the first 64 B of each row).
__device__ __forceinline__ void wide_flush(const uint4* tile, int lane, char* rowptr, int byte_off, int pieces) {
  const unsigned long long mine = reinterpret_cast<unsigned long long>(rowptr);
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + (lane >> 3), p = lane & 7;
    const unsigned long long base = __shfl_sync(0xffffffffu, mine, r);
    if (base != 0ull && p < pieces) *reinterpret_cast<uint4*>(base + byte_off + p * 16) = tile[wide_index(r, p)];
  }
}
// ---------------------------------------------------------------- kernel
// kComm: 0 = GEMM only; 1 = plus two transport warps (token or gradient rows to their hosts, replica weights in).
template <int kMode, int kCtas, int kComm>
__global__ void __launch_bounds__(NUM_THREADS + (kComm ? COMM_WARPS * 32 : 0), 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ GemmArgs args) {
  using G = Geometry<kCtas, kComm>;
  constexpr int STAGES = G::STAGES, STAGE_BYTES = G::STAGE_BYTES, TILE_M = G::TILE_M;
  constexpr bool kAMn = kMode == kWgrad;
  constexpr bool kBMn = kMode == kWgrad || kMode == kDgrad2 || kMode == kDgrad1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);  // barriers start 8-byte aligned
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;  // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  int* tile_prefix = abort_flag + 1;  // [MAX_GROUPS + 1]
  uint4* stage_tiles = reinterpret_cast<uint4*>(smem + STAGES * STAGE_BYTES + kCtrlBytes);  // 8 warps x 4 KB

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Shape shape = make_shape<kMode, kCtas>(args);
  const int cta_rank = kCtas == 2 ? (int)cluster_ctarank() : 0;  // rank 0 of a pair issues the MMAs
  const int tile_first = blockIdx.x / kCtas, tile_stride = gridDim.x / kCtas;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8 * kCtas);
    }
    *abort_flag = 0;
    int acc = 0;
    tile_prefix[0] = 0;
    for (int g = 0; g < shape.n_groups; ++g) {
      int mt = kMode == kWgrad ? shape.m_tiles_fixed : ceil_div(args.group_rows[g], TILE_M);
      acc += mt * shape.n_tiles_n;
      tile_prefix[g + 1] = acc;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (kCtas == 2) tmem_alloc_pair(tmem_slot, TMEM_COLS);
    else tmem_alloc(tmem_slot, TMEM_COLS);
  }
  tc_fence_before();
  __syncthreads();
  if (kCtas == 2) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = tile_prefix[shape.n_groups];
  volatile int* abort_v = abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // The warp walks the tile list together; lane 0 issues the TMA loads.
    int stage = 0;
    uint32_t phase = 0;
    Tile t;
    const unsigned long long wait_ns = args.wait_ns ? args.wait_ns : kWaitBudgetNs;
    int seen_mtile = -1, seen_group = -1, seen_slot = -1;  // waits already satisfied
    for (int ti = tile_first; ti < total_tiles; ti += tile_stride) {
      int go = 1;
      if (lane == 0) {
        if (*abort_v || !find_tile<kMode>(args, shape, tile_prefix, ti, t)) go = 0;
        if (go && args.arrive != nullptr) {
          // rows of this tile (kWgrad: of the whole group) must have arrived from every sender
          const int first = t.row0 / TILE_M;
          if (kMode == kWgrad) {
            if (t.g != seen_group) {
              const int n = ceil_div(min(t.rows, args.row_capacity - t.row0), TILE_M);
              for (int i = 0; i < n && go; ++i)
                if (!flag_wait<true>(args.arrive + first + i, args.arrive_expected, wait_ns, abort_v, args.status, 5, first + i)) go = 0;
              seen_group = t.g;
            }
          } else if (first + t.mt != seen_mtile && (t.row0 + t.mt * TILE_M) < args.row_capacity) {
            if (!flag_wait<true>(args.arrive + first + t.mt, args.arrive_expected, wait_ns, abort_v, args.status, 5, first + t.mt)) go = 0;
            seen_mtile = first + t.mt;
          }
        }
        if (go && args.pull_cnt != nullptr && t.wslot >= args.home_cap && t.wslot != seen_slot) {
          if (!flag_wait<false>(args.pull_cnt + (t.wslot - args.home_cap), args.pull_expected, wait_ns, abort_v, args.status, 6, t.wslot)) go = 0;
          seen_slot = t.wslot;
        }
        if (go) {
          const int m_off = t.mt * TILE_M + cta_rank * BM;            // this CTA's rows of the tile
          const int n_off = t.nt * BN + cta_rank * (BN / 2) * (kCtas - 1);  // this CTA's columns of B
          constexpr int kBoxesB = 4 / kCtas;                          // 64-wide MN-major boxes of B
          for (int kb = 0; kb < t.kblocks; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_v, args.status, 1)) {
              go = 0;
              break;
            }
            uint8_t* sA = tiles + stage * STAGE_BYTES;
            uint8_t* sB = sA + A_BYTES;
            uint64_t* fb = &full_bar[stage];
            if (cta_rank == 0) mbar_expect_tx(fb, STAGE_BYTES * kCtas);  // both CTAs' bytes land on the leader's barrier
            if (kMode == kWgrad) {
              const int krow = t.row0 + kb * BK;
              for (int i = 0; i < 2; ++i) tma2<kCtas>(sA + i * 8192, &tmA, fb, m_off + 64 * i, krow);
              for (int j = 0; j < kBoxesB; ++j) tma2<kCtas>(sB + j * 8192, &tmB, fb, n_off + 64 * j, krow);
            } else {
              tma2<kCtas>(sA, &tmA, fb, kb * BK, t.row0 + m_off);
              if (kMode == kFwd1) {
                // gate rows [nt*128, +128) and up rows [F + nt*128, +128): one half per CTA of a pair
                if (kCtas == 2) {
                  tma3<kCtas>(sB, &tmB, fb, kb * BK, cta_rank * args.N + t.nt * 128, t.wslot);
                } else {
                  tma3<kCtas>(sB, &tmB, fb, kb * BK, t.nt * 128, t.wslot);
                  tma3<kCtas>(sB + 16384, &tmB, fb, kb * BK, args.N + t.nt * 128, t.wslot);
                }
              } else if (kBMn) {
                for (int j = 0; j < kBoxesB; ++j) tma3<kCtas>(sB + j * 8192, &tmB, fb, n_off + 64 * j, kb * BK, t.wslot);
              } else {
                tma3<kCtas>(sB, &tmB, fb, kb * BK, n_off, t.wslot);
                if (kCtas == 1) tma3<kCtas>(sB + 16384, &tmB, fb, kb * BK, n_off + 128, t.wslot);
              }
            }
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
      go = __shfl_sync(0xffffffffu, go, 0);
      if (!go) break;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && cta_rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local = 0;
      Tile t;
      for (int ti = tile_first; ti < total_tiles && !*abort_v; ti += tile_stride, ++local) {
        if (!find_tile<kMode>(args, shape, tile_prefix, ti, t)) break;
        const int buf = local & 1;
        if (!mbar_wait(&acc_empty[buf], acc_phase[buf] ^ 1u, abort_v, args.status, 2)) break;
        acc_phase[buf] ^= 1u;
        tc_fence_after();
        if (args.trace != nullptr && local == 0) {
          // first operands of this CTA's first tile have landed?  (start of useful tensor work)
          if (mbar_wait(&full_bar[stage], phase, abort_v, args.status, 3)) atomicMin(args.trace + 3, globaltimer_ns());
        }
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        // columns the MMA must produce for this tile (multiple of 16, at most 256); a CTA pair
        // always produces all 256 because each CTA holds a fixed half of them
        int ncols = BN;
        if (kMode != kFwd1 && kCtas == 1) {
          int left = args.N - t.nt * BN;
          if (left < BN) ncols = round_up(left, 16);
        }
        const uint32_t idesc = make_idesc(kAMn, kBMn, ncols, TILE_M);
        bool failed = false;
        for (int kb = 0; kb < t.kblocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_v, args.status, 3)) {
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(tiles + stage * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
          const uint64_t da = kAMn ? make_desc(sA, 8192, 1024) : make_desc(sA, 16, 1024);
          const uint64_t db = kBMn ? make_desc(sB, 8192, 1024) : make_desc(sB, 16, 1024);
          constexpr uint32_t a_step = kAMn ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
          constexpr uint32_t b_step = kBMn ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if (kCtas == 2)
              umma_bf16_pair(tmem_d, da + (uint64_t)(k * a_step), db + (uint64_t)(k * b_step), idesc, (kb | k) ? 1u : 0u);
            else
              umma_bf16(tmem_d, da + (uint64_t)(k * a_step), db + (uint64_t)(k * b_step), idesc, (kb | k) ? 1u : 0u);
          }
          // frees the smem stage (in both CTAs of a pair) once these MMAs have read it
          if (kCtas == 2) {
            const uint32_t eb = smem_u32(&empty_bar[stage]);
            umma_commit_pair(eb);
            umma_commit_pair(map_to_cta(eb, 1));
          } else {
            umma_commit(&empty_bar[stage]);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (failed) break;
        if (args.trace != nullptr) atomicMax(args.trace + 2, globaltimer_ns());
        // accumulator ready for the epilogue warps (of both CTAs)
        if (kCtas == 2) {
          const uint32_t ab = smem_u32(&acc_full[buf]);
          umma_commit_pair(ab);
          umma_commit_pair(map_to_cta(ab, 1));
        } else {
          umma_commit(&acc_full[buf]);
        }
      }
    }
    __syncwarp();
  } else if (kComm != 0 && warp >= NUM_THREADS / 32) {
    // ------------------------------------------------------------ transport (warps 10, 11)
    uint8_t* comm_smem_base = reinterpret_cast<uint8_t*>(stage_tiles) + 8 * kStageWarpBytes +
                              (warp - NUM_THREADS / 32) * comm_warp_bytes<G::COMM_SLOTS>();
    if (args.trace != nullptr && lane == 0) atomicMin(args.trace, globaltimer_ns());
    comm_run<G::COMM_SLOTS>(args.comm, (int)blockIdx.x * COMM_WARPS + (warp - NUM_THREADS / 32), (int)gridDim.x * COMM_WARPS,
             comm_smem_base, args.status, args.trace != nullptr ? args.trace + 8 : nullptr);
    if (args.trace != nullptr && lane == 0) atomicMax(args.trace + 1, globaltimer_ns());
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    // Each warp owns 32 accumulator rows.  Columns are processed 32 at a time: the TMEM load of
    // chunk c+1 is in flight while chunk c is converted, staged through a private 2 KB shared
    // tile and written out with row-contiguous 16-byte stores (8 rows x 64 B per instruction).
    const int quarter = warp & 3;      // TMEM lanes [32*quarter, 32*quarter + 32)
    const int half = (warp - 2) >> 2;  // which half of the tile's column chunks this warp handles
    uint4* stg = stage_tiles + (warp - 2) * (kStageWarpBytes / 16);
    uint32_t acc_phase[2] = {0, 0};
    int local = 0;
    Tile t;
    char* out0 = reinterpret_cast<char*>(args.out0);
    char* out1 = reinterpret_cast<char*>(args.out1);
    for (int ti = tile_first; ti < total_tiles && !*abort_v; ti += tile_stride, ++local) {
      if (!find_tile<kMode>(args, shape, tile_prefix, ti, t)) break;
      const int buf = local & 1;
      if (!mbar_wait(&acc_full[buf], acc_phase[buf], abort_v, args.status, 4)) break;
      acc_phase[buf] ^= 1u;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
      const int r_in_tile = cta_rank * BM + quarter * 32 + lane;  // row inside the (pair's) M tile

      if (kMode == kFwd1) {
        const int row_in_group = t.mt * TILE_M + r_in_tile;
        const size_t row = (size_t)t.row0 + row_in_group;  // rows up to the padded end exist in the buffers
        const bool in_buf = row < (size_t)args.row_capacity;
        const bool real = row_in_group < t.rows && in_buf;
        const int F = args.N;
        char* hrow = in_buf ? out0 + (row * (size_t)(2 * F) + t.nt * 128) * 2 : nullptr;
        char* arow = in_buf ? out1 + (row * (size_t)F + t.nt * 128) * 2 : nullptr;
        const float rs = (real && args.row_scale != nullptr) ? __ldcg(args.row_scale + row) : 1.f;  // the row's gate weight
        uint32_t g[2][32], u[2][32];
        const int cb = half * 2;  // this warp's two 32-column chunks of the gate (and up) half
        tmem_ld32(taddr + cb * 32, g[0]);
        tmem_ld32(taddr + 128 + cb * 32, u[0]);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int c = cb + k;
          tmem_ld_wait();
          if (k + 1 < 2) {
            tmem_ld32(taddr + (c + 1) * 32, g[(k + 1) & 1]);
            tmem_ld32(taddr + 128 + (c + 1) * 32, u[(k + 1) & 1]);
          }
          uint32_t(&gv)[32] = g[k & 1];
          uint32_t(&uv)[32] = u[k & 1];
          uint4 pg[4], pu[4], pa[4];
          pack_row(gv, pg, real);
          pack_row(uv, pu, real);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            // activation from the bf16-rounded pre-activations, exactly what backward will read
            float2 g2 = unpack_bf16((&pg[0].x)[i]), u2 = unpack_bf16((&pu[0].x)[i]);
            (&pa[0].x)[i] = pack_bf16(rs * g2.x * sigmoidf_fast(g2.x) * u2.x, rs * g2.y * sigmoidf_fast(g2.y) * u2.y);
          }
          stage_store(stg, lane, pg);
          stage_flush(stg, lane, hrow, c * 64);
          stage_store(stg, lane, pu);
          stage_flush(stg, lane, hrow, F * 2 + c * 64);
          stage_store(stg, lane, pa);
          stage_flush(stg, lane, arow, c * 64);
        }
      } else if (kMode == kDgrad2) {
        const int row_in_group = t.mt * TILE_M + r_in_tile;
        const size_t row = (size_t)t.row0 + row_in_group;
        const bool in_buf = row < (size_t)args.row_capacity;
        const bool real = row_in_group < t.rows && in_buf;
        const int F = args.N;
        char* hrow = in_buf ? out0 + row * (size_t)(2 * F) * 2 : nullptr;
        const int col0 = t.nt * BN;
        const int nchunks = min(BN / 32, (F - col0) / 32);
        uint32_t v[2][32];
        uint4 lg[2][4], lu[2][4];  // this row's saved gate / up pre-activations, one chunk ahead
        const int cb = half * 4;  // this warp's four 32-column chunks
        if (cb < nchunks) {
          tmem_ld32(taddr + cb * 32, v[0]);
          row_load(hrow, (col0 + cb * 32) * 2, lg[0]);
          row_load(hrow, (F + col0 + cb * 32) * 2, lu[0]);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = cb + k;
          if (c < nchunks) {
            tmem_ld_wait();
            if (k + 1 < 4 && c + 1 < nchunks) {
              tmem_ld32(taddr + (c + 1) * 32, v[(k + 1) & 1]);
              row_load(hrow, (col0 + (c + 1) * 32) * 2, lg[(k + 1) & 1]);
              row_load(hrow, (F + col0 + (c + 1) * 32) * 2, lu[(k + 1) & 1]);
            }
            uint4 dg[4], du[4];
            uint4(&pg)[4] = lg[k & 1];
            uint4(&pu)[4] = lu[k & 1];
            uint32_t(&dv)[32] = v[k & 1];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float2 g2 = unpack_bf16((&pg[0].x)[i]), u2 = unpack_bf16((&pu[0].x)[i]);
              float d0 = __uint_as_float(dv[2 * i]), d1 = __uint_as_float(dv[2 * i + 1]);
              float s0 = sigmoidf_fast(g2.x), s1 = sigmoidf_fast(g2.y);
              // d/dg [g*s(g)] = s + g*s*(1-s)
              const uint32_t vg = pack_bf16(d0 * u2.x * (s0 + g2.x * s0 * (1.f - s0)), d1 * u2.y * (s1 + g2.y * s1 * (1.f - s1)));
              const uint32_t vu = pack_bf16(d0 * g2.x * s0, d1 * g2.y * s1);
              (&dg[0].x)[i] = real ? vg : 0u;  // padding rows are written as exact zeros
              (&du[0].x)[i] = real ? vu : 0u;
            }
            row_store(hrow, (col0 + c * 32) * 2, dg);
            row_store(hrow, (F + col0 + c * 32) * 2, du);
          }
        }
      } else {
        // kFwd2 / kDgrad1 / kPlain: plain rows, optionally scattered to the unit's source rank.
        // kWgrad: rows of the weight gradient of this group's slot.
        char* orow = nullptr;
        int n_total = args.N;
        bool have_acc = true;
        if (kMode == kWgrad) {
          const int m = t.mt * TILE_M + r_in_tile;
          if (m < args.M_out) orow = out0 + ((size_t)t.wslot * args.M_out + m) * (size_t)args.N * 2;
          have_acc = t.kblocks > 0;  // an expert that received no rows has a zero gradient
        } else {
          const int row_in_group = t.mt * TILE_M + r_in_tile;
          const size_t row = (size_t)t.row0 + row_in_group;
          if (row_in_group < t.rows && row < (size_t)args.row_capacity) {
            if (args.meta != nullptr) {
              const int2 mt = args.meta[row];
              char* base = args.out_ptrs ? reinterpret_cast<char*>(args.out_ptrs[mt.x]) : out0;
              orow = base + (size_t)mt.y * args.N * 2;
            } else {
              orow = out0 + row * (size_t)args.N * 2;
            }
          }
        }
        const int col0 = t.nt * BN;
        const int nchunks = min(BN / 32, (n_total - col0) / 32);
        uint32_t v[2][32];
        const int cb = half * 4;  // this warp's four 32-column chunks
        if (have_acc && cb < nchunks) tmem_ld32(taddr + cb * 32, v[0]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = cb + k;
          if (c < nchunks) {
            uint4 pk[4];
            if (have_acc) {
              tmem_ld_wait();
              if (k + 1 < 4 && c + 1 < nchunks) tmem_ld32(taddr + (c + 1) * 32, v[(k + 1) & 1]);
              pack_row(v[k & 1], pk, true);
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i) pk[i] = make_uint4(0, 0, 0, 0);
            }
            wide_store_half(stg, lane, pk, k & 1);
            if ((k & 1) || c + 1 >= nchunks) wide_flush(stg, lane, orow, (col0 + (c - (k & 1)) * 32) * 2, (k & 1) ? 8 : 4);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {  // the accumulator buffer is free again: tell the MMA issuer (leader CTA)
        if (kCtas == 2) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
        else mbar_arrive(&acc_empty[buf]);
      }
    }
    if (args.done_ctr != nullptr) __threadfence_system();  // this warp's (peer) stores before the completion signal
  }

  // ------------------------------------------------------------ teardown
  __syncthreads();
  if (args.done_ctr != nullptr && threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(args.done_ctr, 1u) == gridDim.x - 1) {
      // last CTA of the launch: every CTA's rows are stored and fenced
      *args.done_ctr = 0u;
      __threadfence_system();
      *args.done_epoch += 1u;
      for (int r = 0; r < args.done_R; ++r) red_release_sys_add(args.done_signal_ptrs[r] + args.done_slot, 1u);
    }
  }
  if (*abort_v && threadIdx.x == 0) {
    // let copies that were already issued land before the shared memory is released
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  __syncthreads();
  if (kCtas == 2) cluster_sync_all();  // neither CTA leaves while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    if (kCtas == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int kCtas, int kComm>
constexpr size_t smem_bytes() {
  return Geometry<kCtas, kComm>::STAGES * Geometry<kCtas, kComm>::STAGE_BYTES + 1024 /*align*/ +
         kCtrlBytes /*barriers, flags, tile prefix*/ + 8 * kStageWarpBytes /*staging*/ +
         (kComm ? COMM_WARPS * comm_warp_bytes<Geometry<kCtas, kComm>::COMM_SLOTS>() : 0) /*transport rings*/;
}
static_assert(smem_bytes<2, 1>() <= 232448 && smem_bytes<1, 1>() <= 232448 && smem_bytes<2, 0>() <= 232448, "shared memory budget");

// ---------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

}  // namespace

bool make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols,
                  uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_tmap_3d(CUtensorMap* out, const void* base, uint64_t slots, uint64_t rows, uint64_t cols, uint32_t box_cols,
                  uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[3] = {cols, rows, slots};
  cuuint64_t strides[2] = {cols * 2, rows * cols * 2};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int kMode, int kCtas, int kComm>
static cudaError_t launch_mode(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& args, int num_sms,
                               cudaStream_t stream) {
  static bool configured[kMaxTrackedDevices] = {};
  constexpr size_t smem = smem_bytes<kCtas, kComm>();
  int dev;
  if (device_needs_setup(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<kMode, kCtas, kComm>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return e;
    device_setup_done(configured, dev);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(num_sms / kCtas * kCtas));
  cfg.blockDim = dim3(NUM_THREADS + (kComm ? COMM_WARPS * 32 : 0));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCtas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<kMode, kCtas, kComm>, tmA, tmB, args);
}

template <int kCtas>
static cudaError_t launch_ctas(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& args, int num_sms,
                               cudaStream_t stream) {
  const bool comm = args.comm.do_dispatch || args.comm.do_pad || args.comm.do_pull;
  if (comm) {
    // fused transport exists for the two GEMMs that consume freshly dispatched rows
    if (args.mode == kFwd1) return launch_mode<kFwd1, kCtas, 1>(tmA, tmB, args, num_sms, stream);
    if (args.mode == kDgrad1) return launch_mode<kDgrad1, kCtas, 1>(tmA, tmB, args, num_sms, stream);
    return cudaErrorInvalidValue;
  }
  switch (args.mode) {
    case kFwd1: return launch_mode<kFwd1, kCtas, 0>(tmA, tmB, args, num_sms, stream);
    case kFwd2: return launch_mode<kFwd2, kCtas, 0>(tmA, tmB, args, num_sms, stream);
    case kDgrad2: return launch_mode<kDgrad2, kCtas, 0>(tmA, tmB, args, num_sms, stream);
    case kDgrad1: return launch_mode<kDgrad1, kCtas, 0>(tmA, tmB, args, num_sms, stream);
    case kWgrad: return launch_mode<kWgrad, kCtas, 0>(tmA, tmB, args, num_sms, stream);
    case kPlain: return launch_mode<kPlain, kCtas, 0>(tmA, tmB, args, num_sms, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_grouped_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& args, int num_sms,
                                cudaStream_t stream) {
  if (args.n_groups_cap > MAX_GROUPS) return cudaErrorInvalidValue;
  if (args.mode == kFwd1 && args.N % 128 != 0) return cudaErrorInvalidValue;
  if (args.N % 32 != 0) return cudaErrorInvalidValue;
  if (args.ctas == 2) return launch_ctas<2>(tmA, tmB, args, num_sms, stream);
  return launch_ctas<1>(tmA, tmB, args, num_sms, stream);
}

}  // namespace epb
