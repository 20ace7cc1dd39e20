// Block-scaled fp8 grouped GEMM: out[rows, N] = A_q[rows, K] * B_q[slot][N, K]^T with 1 x 128 activation
// scales and 128 x 128 weight scales applied by the tensor core (kind::mxf8f6f4.block_scale).
//
// One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer: per k-block one 128 x 128-byte tile of A and of B (128-byte swizzle) and,
//               at every fourth k-block, the two 512-byte scale chunks (bulk copies on the same barrier)
//   warp 1      one thread copies the scale chunks shared -> tensor memory (tcgen05.cp) and issues four
//               128 x 128 x 32 MMAs per k-block; accumulators: two 128-column fp32 buffers in TMEM
//   warps 2-9   epilogue: tcgen05.ld, bf16 pack, staged 128-byte row stores (optionally to peer buffers)
// Every mbarrier wait is bounded; on a timeout the CTA raises its abort flag, records a status,
// lets issued copies land, frees its tensor memory and returns.
#include "grouped_gemm_fp8.h"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace epb {
namespace {

constexpr int BM = 128, BN = 128, BK = 128;       // BK in elements = bytes
constexpr int UMMA_K = 32;
constexpr int STAGES = 5;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, TILE_BYTES = A_BYTES + B_BYTES;
constexpr int SF_BYTES = 1024;                     // 512 B for A + 512 B for B per stage
constexpr int NUM_THREADS = 320;
constexpr int MAX_GROUPS = 320;
constexpr int kCtrlBytes = 1536;
constexpr int kStageWarpBytes = 4096;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t kSfCol = 256;                   // scale factors live behind the two accumulators
static_assert((STAGES * 2 + 4) * 8 + 8 + (MAX_GROUPS + 1) * 4 <= kCtrlBytes, "control block does not fit");

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
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols));
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 512-byte scale chunk (32 rows x 16 B) -> 4 TMEM columns, replicated to the four 32-lane groups
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_fp8_scaled(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
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

// Shared-memory matrix descriptors (version 1).  Operand tiles: K-major, 128-byte swizzle, 8-row groups
// 1024 B apart.  Scale chunks: no swizzle, 8-row x 16-byte core matrices 128 B apart.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(16 >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ uint64_t make_desc_sf(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(128 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}
// Instruction descriptor of the block-scaled kind: e4m3 x e4m3, both K-major, UE8M0 scales;
// sf ids select which of the four scale bytes of a TMEM word this MMA uses.
__device__ __forceinline__ uint32_t make_idesc_scaled(int n, int m, uint32_t a_sf_id, uint32_t b_sf_id) {
  return (b_sf_id << 4) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(m >> 4) << 24) | (a_sf_id << 29);
}

struct Tile {
  int g, mt, nt, rows, row0, wslot;
};

__device__ __forceinline__ bool find_tile(const Fp8GemmArgs& a, int n_groups, int n_tiles_n, const int* tile_prefix,
                                          int t, Tile& out) {
  int g = 0;
  while (g < n_groups && t >= tile_prefix[g + 1]) ++g;
  if (g >= n_groups) return false;
  const int local = t - tile_prefix[g];
  out.g = g;
  out.mt = local / n_tiles_n;
  out.nt = local - out.mt * n_tiles_n;
  out.rows = a.group_rows[g];
  out.row0 = a.group_off[g];
  out.wslot = a.group_wslot[g];
  return true;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void pack_row(const uint32_t (&r)[32], uint4 (&out)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[i].x = pack_bf16(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
    out[i].y = pack_bf16(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
    out[i].z = pack_bf16(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
    out[i].w = pack_bf16(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
  }
}
// 32 rows x 128 B staging tile; piece p (16 B) of row r at r*8 + (p ^ (r & 7)): conflict-free for the
// row-wise writes and for the flush, which stores four rows x 128 contiguous bytes per instruction.
__device__ __forceinline__ int wide_index(int r, int p) { return r * 8 + (p ^ (r & 7)); }
__device__ __forceinline__ void wide_store_half(uint4* tile, int lane, const uint4 (&p)[4], int half) {
#pragma unroll
  for (int i = 0; i < 4; ++i) tile[wide_index(lane, half * 4 + i)] = p[i];
}
__device__ __forceinline__ void wide_flush(const uint4* tile, int lane, char* rowptr, int byte_off) {
  const unsigned long long mine = reinterpret_cast<unsigned long long>(rowptr);
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + (lane >> 3), p = lane & 7;
    const unsigned long long base = __shfl_sync(0xffffffffu, mine, r);
    if (base != 0ull) *reinterpret_cast<uint4*>(base + byte_off + p * 16) = tile[wide_index(r, p)];
  }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        Fp8GemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles = smem;
  uint8_t* sf_tiles = smem + STAGES * TILE_BYTES;                       // [STAGES][1024]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sf_tiles + STAGES * SF_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;  // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  int* tile_prefix = abort_flag + 1;        // [MAX_GROUPS + 1]
  uint4* stage_tiles = reinterpret_cast<uint4*>(sf_tiles + STAGES * SF_BYTES + kCtrlBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int n_groups = args.totals[1];
  if (n_groups > args.n_groups_cap) n_groups = args.n_groups_cap;
  const int n_tiles_n = args.N / BN;
  const int kblocks = args.K / BK;
  const int kgroups = (kblocks + 3) / 4;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);
    }
    *abort_flag = 0;
    int acc = 0;
    tile_prefix[0] = 0;
    for (int g = 0; g < n_groups; ++g) {
      acc += ceil_div(args.group_rows[g], BM) * n_tiles_n;
      tile_prefix[g + 1] = acc;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = tile_prefix[n_groups];
  volatile int* abort_v = abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    Tile t;
    for (int ti = blockIdx.x; ti < total_tiles; ti += gridDim.x) {
      int go = 1;
      if (lane == 0) {
        if (*abort_v || !find_tile(args, n_groups, n_tiles_n, tile_prefix, ti, t)) go = 0;
        if (go) {
          const int row_tile = (t.row0 + t.mt * BM) / BM;
          const uint8_t* sfa = args.sfa + (size_t)row_tile * kgroups * 512;
          const uint8_t* sfb = args.sfb + ((size_t)t.wslot * n_tiles_n + t.nt) * kgroups * 512;
          for (int kb = 0; kb < kblocks; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_v, args.status, 11)) {
              go = 0;
              break;
            }
            uint8_t* sA = tiles + stage * TILE_BYTES;
            uint8_t* sB = sA + A_BYTES;
            uint64_t* fb = &full_bar[stage];
            const bool with_sf = (kb & 3) == 0;
            mbar_expect_tx(fb, TILE_BYTES + (with_sf ? SF_BYTES : 0));
            tma_load_2d(sA, &tmA, fb, kb * BK, t.row0 + t.mt * BM);
            tma_load_3d(sB, &tmB, fb, kb * BK, t.nt * BN, t.wslot);
            if (with_sf) {
              uint8_t* sS = sf_tiles + stage * SF_BYTES;
              bulk_load(sS, sfa + (size_t)(kb >> 2) * 512, 512, fb);
              bulk_load(sS + 512, sfb + (size_t)(kb >> 2) * 512, 512, fb);
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
    // ------------------------------------------------------------ scale copies + MMA issue
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local = 0;
      uint32_t sf_buf = 0;  // two sets of scale columns: the copy for k-group g+1 never races the MMAs of g
      Tile t;
      for (int ti = blockIdx.x; ti < total_tiles && !*abort_v; ti += gridDim.x, ++local) {
        if (!find_tile(args, n_groups, n_tiles_n, tile_prefix, ti, t)) break;
        const int buf = local & 1;
        if (!mbar_wait(&acc_empty[buf], acc_phase[buf] ^ 1u, abort_v, args.status, 12)) break;
        acc_phase[buf] ^= 1u;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        bool failed = false;
        uint32_t sfa_col = 0, sfb_col = 0;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_v, args.status, 13)) {
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(tiles + stage * TILE_BYTES);
          const uint32_t sB = sA + A_BYTES;
          if ((kb & 3) == 0) {
            const uint32_t sS = smem_u32(sf_tiles + stage * SF_BYTES);
            sfa_col = tmem_base + kSfCol + sf_buf * 8;
            sfb_col = sfa_col + 4;
            tmem_cp_sf(sfa_col, make_desc_sf(sS));
            tmem_cp_sf(sfb_col, make_desc_sf(sS + 512));
            sf_buf ^= 1u;
          }
          const uint32_t id = (uint32_t)(kb & 3);
          const uint32_t idesc = make_idesc_scaled(BN, BM, id, id);
          const uint64_t da = make_desc_sw128(sA), db = make_desc_sw128(sB);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_fp8_scaled(tmem_d, da + (uint64_t)(k * (UMMA_K >> 4)), db + (uint64_t)(k * (UMMA_K >> 4)), idesc, sfa_col,
                            sfb_col, (kb | k) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);  // frees the stage (tiles and scale chunks) once read
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (failed) break;
        umma_commit(&acc_full[buf]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;      // TMEM lanes [32*quarter, +32)
    const int half = (warp - 2) >> 2;  // columns [64*half, +64) of the tile
    uint4* stg = stage_tiles + (warp - 2) * (kStageWarpBytes / 16);
    uint32_t acc_phase[2] = {0, 0};
    int local = 0;
    Tile t;
    char* out0 = reinterpret_cast<char*>(args.out);
    for (int ti = blockIdx.x; ti < total_tiles && !*abort_v; ti += gridDim.x, ++local) {
      if (!find_tile(args, n_groups, n_tiles_n, tile_prefix, ti, t)) break;
      const int buf = local & 1;
      if (!mbar_wait(&acc_full[buf], acc_phase[buf], abort_v, args.status, 14)) break;
      acc_phase[buf] ^= 1u;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * 64);
      const int row_in_group = t.mt * BM + quarter * 32 + lane;
      const size_t row = (size_t)t.row0 + row_in_group;
      char* orow = nullptr;
      if (row_in_group < t.rows && row < (size_t)args.row_capacity) {
        if (args.meta != nullptr) {
          const int2 mt = args.meta[row];
          char* base = args.out_ptrs ? reinterpret_cast<char*>(args.out_ptrs[mt.x]) : out0;
          orow = base + (size_t)mt.y * args.N * 2;
        } else {
          orow = out0 + row * (size_t)args.N * 2;
        }
      }
      uint32_t v0[32], v1[32];
      tmem_ld32(taddr, v0);
      tmem_ld32(taddr + 32, v1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);  // the values are in registers: the buffer is free
      uint4 p0[4], p1[4];
      pack_row(v0, p0);
      pack_row(v1, p1);
      __syncwarp();
      wide_store_half(stg, lane, p0, 0);
      wide_store_half(stg, lane, p1, 1);
      __syncwarp();
      wide_flush(stg, lane, orow, (t.nt * BN + half * 64) * 2);
    }
  }

  // ------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_v && threadIdx.x == 0) {
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);  // issued copies land before smem is released
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ================================================================ CTA-pair variant (cta_group::2)
// A thread-block cluster of two SMs computes a 256 x 128 tile: each CTA stages its own 128 rows of A, its
// own 64 of the 128 weight rows (B) and the scale chunks it needs (its rows' SFA chunk and the whole SFB
// chunk), so per MMA a CTA reads 6 KB of shared memory instead of 8 KB and the tensor pipe is no longer fed at
// the shared-memory limit.  Every load is a plain TMA load (no multicast) that completes on the barrier of
// the pair's even CTA; that CTA issues the scale copies and the MMAs for both.
namespace pair {

// kBN = 128: two accumulator buffers (epilogue overlaps the next tile).  kBN = 256: one 256-column accumulator
// (the scale factors need the rest of tensor memory), twice the MMA work per TMA load and per barrier round.
template <int kBN>
struct Geo {
  static constexpr int B_HALF = kBN / 2;                     // weight rows staged per CTA
  static constexpr int A_BYTES = BM * BK, B_BYTES = B_HALF * BK, TILE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SF_BYTES = 512 + 512 * (kBN / 128);   // this CTA's SFA chunk + the SFB chunks of the whole tile
  static constexpr int STAGES = kBN == 128 ? 6 : 5;
  static constexpr int ACC_BUFS = kBN == 128 ? 2 : 1;
  static constexpr size_t SMEM = STAGES * TILE_BYTES + STAGES * 2048 + 1024 + kCtrlBytes + 8 * kStageWarpBytes;
};
constexpr int TILE_M = 2 * BM;
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;               // clears the CTA-rank bit of a shared::cluster address

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
__device__ __forceinline__ void tma_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & kPeerBitMask), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & kPeerBitMask), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void commit2(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tmem_cp_sf2(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma2(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t sfa,
                                      uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}

template <int kBN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_fp8_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                             const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                             Fp8GemmArgs args) {
  using G = Geo<kBN>;
  constexpr int STAGES = G::STAGES, TILE_BYTES = G::TILE_BYTES, A_BYTES = G::A_BYTES, B_HALF = G::B_HALF;
  constexpr int SF_BYTES = 2048;   // slot size; G::SF_BYTES of it are used
  constexpr int ACC_BUFS = G::ACC_BUFS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles = smem;
  uint8_t* sf_tiles = smem + STAGES * TILE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sf_tiles + STAGES * SF_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  int* tile_prefix = abort_flag + 1;
  uint4* stage_tiles = reinterpret_cast<uint4*>(sf_tiles + STAGES * SF_BYTES + kCtrlBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta_rank = (int)cluster_ctarank();
  const int tile_first = blockIdx.x / 2, tile_stride = gridDim.x / 2;
  int n_groups = args.totals[1];
  if (n_groups > args.n_groups_cap) n_groups = args.n_groups_cap;
  const int n_tiles_n = args.N / kBN;
  const int n128 = args.N / 128;
  const int kblocks = args.K / BK;
  const int kgroups = (kblocks + 3) / 4;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 16);   // 8 epilogue warps of each CTA
    }
    *abort_flag = 0;
    int acc = 0;
    tile_prefix[0] = 0;
    for (int g = 0; g < n_groups; ++g) {
      acc += ceil_div(args.group_rows[g], TILE_M) * n_tiles_n;
      tile_prefix[g + 1] = acc;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc2(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = tile_prefix[n_groups];
  volatile int* abort_v = abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    int stage = 0;
    uint32_t phase = 0;
    Tile t;
    for (int ti = tile_first; ti < total_tiles; ti += tile_stride) {
      int go = 1;
      if (lane == 0) {
        if (*abort_v || !find_tile(args, n_groups, n_tiles_n, tile_prefix, ti, t)) go = 0;
        if (go) {
          const int row_first = t.row0 + t.mt * TILE_M + cta_rank * BM;
          const int sfa_chunk = (row_first / BM) * kgroups;
          const int sfb_chunk = (t.wslot * n128 + t.nt * (kBN / 128)) * kgroups;
          for (int kb = 0; kb < kblocks; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_v, args.status, 21)) {
              go = 0;
              break;
            }
            uint8_t* sA = tiles + stage * TILE_BYTES;
            uint8_t* sB = sA + A_BYTES;
            uint64_t* fb = &full_bar[stage];
            const bool with_sf = (kb & 3) == 0;
            if (cta_rank == 0) mbar_expect_tx(fb, 2 * (TILE_BYTES + (with_sf ? G::SF_BYTES : 0)));
            tma_2d(sA, &tmA, fb, kb * BK, row_first);
            tma_3d(sB, &tmB, fb, kb * BK, t.nt * kBN + cta_rank * B_HALF, t.wslot);
            if (with_sf) {
              uint8_t* sS = sf_tiles + stage * SF_BYTES;
              tma_2d(sS, &tmSFA, fb, 0, sfa_chunk + (kb >> 2));
#pragma unroll
              for (int j = 0; j < kBN / 128; ++j)
                tma_2d(sS + 512 + 512 * j, &tmSFB, fb, 0, sfb_chunk + j * kgroups + (kb >> 2));
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
    // ------------------------------------------------------------ scale copies + MMA issue (even CTA only)
    if (lane == 0 && cta_rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local = 0;
      uint32_t sf_buf = 0;
      Tile t;
      for (int ti = tile_first; ti < total_tiles && !*abort_v; ti += tile_stride, ++local) {
        if (!find_tile(args, n_groups, n_tiles_n, tile_prefix, ti, t)) break;
        const int buf = ACC_BUFS == 2 ? (local & 1) : 0;
        if (!mbar_wait(&acc_empty[buf], acc_phase[buf] ^ 1u, abort_v, args.status, 22)) break;
        acc_phase[buf] ^= 1u;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * 128);
        bool failed = false;
        uint32_t sfa_col = 0, sfb_col = 0;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_v, args.status, 23)) {
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(tiles + stage * TILE_BYTES);
          const uint32_t sB = sA + A_BYTES;
          if ((kb & 3) == 0) {
            const uint32_t sS = smem_u32(sf_tiles + stage * SF_BYTES);
            sfa_col = tmem_base + kSfCol + sf_buf * 16;
            sfb_col = sfa_col + 4;
            tmem_cp_sf2(sfa_col, make_desc_sf(sS));
#pragma unroll
            for (int j = 0; j < kBN / 128; ++j) tmem_cp_sf2(sfb_col + 4 * j, make_desc_sf(sS + 512 + 512 * j));
            sf_buf ^= 1u;
          }
          const uint32_t id = (uint32_t)(kb & 3);
          const uint32_t idesc = make_idesc_scaled(kBN, TILE_M, id, id);
          const uint64_t da = make_desc_sw128(sA), db = make_desc_sw128(sB);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma2(tmem_d, da + (uint64_t)(k * (UMMA_K >> 4)), db + (uint64_t)(k * (UMMA_K >> 4)), idesc, sfa_col, sfb_col,
                  (kb | k) ? 1u : 0u);
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          commit2(eb);
          commit2(map_to_cta(eb, 1));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (failed) break;
        const uint32_t ab = smem_u32(&acc_full[buf]);
        commit2(ab);
        commit2(map_to_cta(ab, 1));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9 of both CTAs)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    uint4* stg = stage_tiles + (warp - 2) * (kStageWarpBytes / 16);
    uint32_t acc_phase[2] = {0, 0};
    int local = 0;
    Tile t;
    char* out0 = reinterpret_cast<char*>(args.out);
    for (int ti = tile_first; ti < total_tiles && !*abort_v; ti += tile_stride, ++local) {
      if (!find_tile(args, n_groups, n_tiles_n, tile_prefix, ti, t)) break;
      const int buf = ACC_BUFS == 2 ? (local & 1) : 0;
      if (!mbar_wait(&acc_full[buf], acc_phase[buf], abort_v, args.status, 24)) break;
      acc_phase[buf] ^= 1u;
      tc_fence_after();
      constexpr int COLS_PER_WARP = kBN / 2;                      // 64 or 128 columns per warp
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * 128 + half * COLS_PER_WARP);
      const int row_in_group = t.mt * TILE_M + cta_rank * BM + quarter * 32 + lane;
      const size_t row = (size_t)t.row0 + row_in_group;
      char* orow = nullptr;
      if (row_in_group < t.rows && row < (size_t)args.row_capacity) {
        if (args.meta != nullptr) {
          const int2 mt = args.meta[row];
          char* base = args.out_ptrs ? reinterpret_cast<char*>(args.out_ptrs[mt.x]) : out0;
          orow = base + (size_t)mt.y * args.N * 2;
        } else {
          orow = out0 + row * (size_t)args.N * 2;
        }
      }
      // read this warp's whole share of the accumulator into registers first and hand the buffer back at once:
      // with a single accumulator the next tile's MMAs wait for exactly this read
      uint32_t v[COLS_PER_WARP / 32][32];
#pragma unroll
      for (int c = 0; c < COLS_PER_WARP / 32; ++c) tmem_ld32(taddr + c * 32, v[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
#pragma unroll
      for (int pairc = 0; pairc < COLS_PER_WARP / 64; ++pairc) {
        uint4 p0[4], p1[4];
        pack_row(v[2 * pairc], p0);
        pack_row(v[2 * pairc + 1], p1);
        __syncwarp();
        wide_store_half(stg, lane, p0, 0);
        wide_store_half(stg, lane, p1, 1);
        __syncwarp();
        wide_flush(stg, lane, orow, (t.nt * kBN + half * COLS_PER_WARP + pairc * 64) * 2);
      }
    }
  }

  __syncthreads();
  if (*abort_v && threadIdx.x == 0) {
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

static_assert(Geo<128>::SMEM <= 232448 && Geo<256>::SMEM <= 232448, "shared memory budget exceeded");

}  // namespace pair

constexpr size_t kSmemBytes = STAGES * TILE_BYTES + STAGES * SF_BYTES + 1024 + kCtrlBytes + 8 * kStageWarpBytes;
static_assert(kSmemBytes <= 232448, "shared memory budget exceeded");

// ---------------------------------------------------------------- quantisers
// Power-of-two scale of a block with absolute maximum `amax`: the smallest 2^e with amax / 2^e <= 448.
__device__ __forceinline__ int scale_exponent(float amax) {
  if (!(amax > 0.f)) return -126;
  int ex;
  const float m = frexpf(amax * (1.f / 448.f), &ex);  // amax/448 = m * 2^ex, m in [0.5, 1)
  int e = (m == 0.5f) ? ex - 1 : ex;
  return max(-126, min(126, e));
}
__device__ __forceinline__ float exp2_int(int e) { return __int_as_float((e + 127) << 23); }  // e in [-126, 127]
__device__ __forceinline__ int chunk_byte(int r_in_128, int kb) { return (r_in_128 & 31) * 16 + (r_in_128 >> 5) * 4 + (kb & 3); }

// Is `row` inside one of the groups?  The whole warp calls this with the same row.
__device__ __forceinline__ bool row_is_real(const RowGroups& g, int row, int lane) {
  if (g.group_off == nullptr) return true;
  if (row >= g.totals[0]) return false;
  int n = g.totals[1];
  if (n > g.n_groups_cap) n = g.n_groups_cap;
  for (int base = 0; base < n; base += 32) {
    const int i = base + lane;
    const bool in = i < n && row >= g.group_off[i] && row < g.group_off[i] + g.group_rows[i];
    if (__ballot_sync(0xffffffffu, in)) return true;
  }
  return false;
}

// One warp per row; per 128-wide block each lane handles 4 consecutive values.
__global__ void __launch_bounds__(256) quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                            uint8_t* __restrict__ sfa, int rows, int K, RowGroups groups) {
  const int warp = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (warp >= rows || !row_is_real(groups, warp, lane)) return;
  const int kblocks = K / 128, kgroups = (kblocks + 3) / 4;
  const __nv_bfloat16* xr = x + (size_t)warp * K;
  uint8_t* qr = q + (size_t)warp * K;
  uint8_t* chunk_row = sfa + (size_t)(warp >> 7) * kgroups * 512;
  for (int kb = 0; kb < kblocks; ++kb) {
    const uint2 raw = *reinterpret_cast<const uint2*>(xr + kb * 128 + lane * 4);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const int e = scale_exponent(amax);
    const float inv = exp2_int(-e);
    const unsigned lo = __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv, a.y * inv), __NV_SATFINITE, __NV_E4M3);
    const unsigned hi = __nv_cvt_float2_to_fp8x2(make_float2(b.x * inv, b.y * inv), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(qr + kb * 128 + lane * 4) = (lo & 0xffffu) | (hi << 16);
    if (lane == 0) chunk_row[(size_t)(kb >> 2) * 512 + chunk_byte(warp & 127, kb)] = (uint8_t)(e + 127);
  }
  // k-blocks of a partial last group keep the neutral exponent
  if (lane == 0)
    for (int kb = kblocks; kb < kgroups * 4; ++kb) chunk_row[(size_t)(kb >> 2) * 512 + chunk_byte(warp & 127, kb)] = 127;
}

// One warp per routed unit.  A 128-wide block is held by 16 lanes (8 values each); the block maximum is a
// 4-step shuffle inside the half-warp.  Stores go to the destination rank's buffers (peer memory).
__global__ void __launch_bounds__(256) dispatch_fp8_kernel(DispatchFp8Args a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const int u = blockIdx.x * wpb + warp;
  if (u >= a.num_units) return;
  const int dst = a.unit_dst[u], row = a.unit_row[u];
  if (dst < 0 || row >= a.row_capacity) return;
  const int vec_per_row = a.H / 8;
  const int kgroups = (a.H / 128 + 3) / 4;
  const uint4* src = reinterpret_cast<const uint4*>(a.rows) + (size_t)(u / a.topk) * vec_per_row;
  uint8_t* qrow = a.xq_ptrs[dst] + (size_t)row * a.H;
  uint8_t* chunk_row = a.sfx_ptrs[dst] + (size_t)(row >> 7) * kgroups * 512;
  for (int v = lane; v < vec_per_row + (32 - vec_per_row % 32) % 32; v += 32) {
    const bool have = v < vec_per_row;
    const uint4 raw = have ? src[v] : make_uint4(0, 0, 0, 0);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float f[8];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 p = __bfloat1622float2(h[j]);
      f[2 * j] = p.x;
      f[2 * j + 1] = p.y;
      amax = fmaxf(amax, fmaxf(fabsf(p.x), fabsf(p.y)));
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (!have) continue;
    const int e = scale_exponent(amax);
    const float inv = exp2_int(-e);
    uint32_t out[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const unsigned lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * j] * inv, f[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
      const unsigned hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * j + 2] * inv, f[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
      out[j] = (lo & 0xffffu) | (hi << 16);
    }
    *reinterpret_cast<uint2*>(qrow + (size_t)v * 8) = make_uint2(out[0], out[1]);
    const int kb = v >> 4;
    if ((lane & 15) == 0) chunk_row[(size_t)(kb >> 2) * 512 + chunk_byte(row & 127, kb)] = (uint8_t)(e + 127);
  }
  if (lane == 0 && a.meta_ptrs != nullptr) a.meta_ptrs[dst][row] = make_int2(a.me, a.unit_pos[u]);
}

// SwiGLU + quantisation in one pass: h [rows, 2F] (gate columns, then up columns) ->
// act = silu(gate) * up as e4m3 [rows, F] with 1 x 128 scales (and, optionally, as bf16 too).
__global__ void __launch_bounds__(256) swiglu_quantize_kernel(const __nv_bfloat16* __restrict__ h, uint8_t* __restrict__ q,
                                                              uint8_t* __restrict__ sfa, __nv_bfloat16* __restrict__ act,
                                                              int rows, int F, RowGroups groups) {
  const int warp = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (warp >= rows || !row_is_real(groups, warp, lane)) return;
  const int kblocks = F / 128, kgroups = (kblocks + 3) / 4;
  const __nv_bfloat16* hr = h + (size_t)warp * 2 * F;
  uint8_t* qr = q + (size_t)warp * F;
  uint8_t* chunk_row = sfa + (size_t)(warp >> 7) * kgroups * 512;
  for (int kb = 0; kb < kblocks; ++kb) {
    const uint2 graw = *reinterpret_cast<const uint2*>(hr + kb * 128 + lane * 4);
    const uint2 uraw = *reinterpret_cast<const uint2*>(hr + F + kb * 128 + lane * 4);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    float v[4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float2 g = __bfloat1622float2(gh[j]), u = __bfloat1622float2(uh[j]);
      v[2 * j] = g.x * __fdividef(1.f, 1.f + __expf(-g.x)) * u.x;
      v[2 * j + 1] = g.y * __fdividef(1.f, 1.f + __expf(-g.y)) * u.y;
    }
    if (act != nullptr) {
      uint2 o;
      o.x = pack_bf16(v[0], v[1]);
      o.y = pack_bf16(v[2], v[3]);
      *reinterpret_cast<uint2*>(act + (size_t)warp * F + kb * 128 + lane * 4) = o;
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const int e = scale_exponent(amax);
    const float inv = exp2_int(-e);
    const unsigned lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3);
    const unsigned hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(qr + kb * 128 + lane * 4) = (lo & 0xffffu) | (hi << 16);
    if (lane == 0) chunk_row[(size_t)(kb >> 2) * 512 + chunk_byte(warp & 127, kb)] = (uint8_t)(e + 127);
  }
}

// One CTA per (k-block, n-block, slot): 128 x 128 values, 256 threads, 64 values each.
__global__ void __launch_bounds__(256) quantize_weights_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                                                               uint8_t* __restrict__ sfb, int N, int K) {
  const int kb = blockIdx.x, nb = blockIdx.y, slot = blockIdx.z;
  const int kblocks = K / 128, kgroups = (kblocks + 3) / 4, n_tiles = N / 128;
  const size_t base = ((size_t)slot * N + (size_t)nb * 128) * K + (size_t)kb * 128;
  // thread t: row t/2 of the block, 64 consecutive values starting at (t%2)*64
  const int r = threadIdx.x >> 1, c0 = (threadIdx.x & 1) * 64;
  const uint4* src = reinterpret_cast<const uint4*>(w + base + (size_t)r * K + c0);
  uint4 v[8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] = src[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const int e = scale_exponent(amax);
  const float inv = exp2_int(-e);
  uint8_t* dst = q + base + (size_t)r * K + c0;
#pragma unroll
  for (int i = 0; i < 8; i += 2) {
    uint32_t out[4];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i + half]);
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const float2 f0 = __bfloat1622float2(h[j]), f1 = __bfloat1622float2(h[j + 1]);
        const unsigned lo = __nv_cvt_float2_to_fp8x2(make_float2(f0.x * inv, f0.y * inv), __NV_SATFINITE, __NV_E4M3);
        const unsigned hi = __nv_cvt_float2_to_fp8x2(make_float2(f1.x * inv, f1.y * inv), __NV_SATFINITE, __NV_E4M3);
        out[half * 2 + j / 2] = (lo & 0xffffu) | (hi << 16);
      }
    }
    *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(out[0], out[1], out[2], out[3]);
  }
  uint8_t* chunk = sfb + (((size_t)slot * n_tiles + nb) * kgroups + (kb >> 2)) * 512;
  if (threadIdx.x < 128) chunk[chunk_byte(threadIdx.x, kb)] = (uint8_t)(e + 127);
  if (kb == kblocks - 1 && threadIdx.x < 128)
    for (int k2 = kblocks; k2 < kgroups * 4; ++k2) chunk[chunk_byte(threadIdx.x, k2)] = 127;
}

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

bool make_tmap_fp8_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols};
  cuuint32_t box[2] = {128, 128};
  cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool make_tmap_fp8_3d(CUtensorMap* out, const void* base, uint64_t slots, uint64_t rows, uint64_t cols,
                      uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[3] = {cols, rows, slots};
  cuuint64_t strides[2] = {cols, rows * cols};
  cuuint32_t box[3] = {128, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_tmap_sf(CUtensorMap* out, const void* base, uint64_t chunks) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || chunks == 0) return false;
  cuuint64_t dims[2] = {128, chunks};          // one 512-byte chunk = 128 x int32
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, 1};
  cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

cudaError_t launch_grouped_gemm_fp8_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmSFA,
                                         const CUtensorMap& tmSFB, const Fp8GemmArgs& args, int num_sms,
                                         cudaStream_t stream) {
  if (args.n_groups_cap > MAX_GROUPS || args.N % BN != 0 || args.K % BK != 0 || args.K <= 0) return cudaErrorInvalidValue;
  const bool wide = args.N % 256 == 0;   // 256-column tiles when the width allows it
  static bool configured[kMaxTrackedDevices] = {};
  int dev;
  if (device_needs_setup(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(pair::grouped_gemm_fp8_pair_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)pair::Geo<128>::SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(pair::grouped_gemm_fp8_pair_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)pair::Geo<256>::SMEM);
    if (e != cudaSuccess) return e;
    device_setup_done(configured, dev);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(num_sms / 2 * 2));
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = wide ? pair::Geo<256>::SMEM : pair::Geo<128>::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (wide) return cudaLaunchKernelEx(&cfg, pair::grouped_gemm_fp8_pair_kernel<256>, tmA, tmB, tmSFA, tmSFB, args);
  return cudaLaunchKernelEx(&cfg, pair::grouped_gemm_fp8_pair_kernel<128>, tmA, tmB, tmSFA, tmSFB, args);
}

cudaError_t launch_grouped_gemm_fp8(const CUtensorMap& tmA, const CUtensorMap& tmB, const Fp8GemmArgs& args,
                                    int num_sms, cudaStream_t stream) {
  if (args.n_groups_cap > MAX_GROUPS || args.N % BN != 0 || args.K % BK != 0 || args.K <= 0) return cudaErrorInvalidValue;
  static bool configured[kMaxTrackedDevices] = {};
  int dev;
  if (device_needs_setup(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemBytes);
    if (e != cudaSuccess) return e;
    device_setup_done(configured, dev);
  }
  grouped_gemm_fp8_kernel<<<num_sms, NUM_THREADS, kSmemBytes, stream>>>(tmA, tmB, args);
  return cudaGetLastError();
}

cudaError_t launch_quantize_rows(const void* x, uint8_t* q, uint8_t* sfa, int rows, int K, const RowGroups* groups,
                                 cudaStream_t stream) {
  if (rows % 128 != 0 || K % 128 != 0) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  const int blocks = (rows + 7) / 8;
  quantize_rows_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), q, sfa, rows, K,
                                                   groups ? *groups : RowGroups{nullptr, nullptr, nullptr, 0});
  return cudaGetLastError();
}

cudaError_t launch_dispatch_fp8(const DispatchFp8Args& a, cudaStream_t stream) {
  if (a.H % 128 != 0) return cudaErrorInvalidValue;
  if (a.num_units <= 0) return cudaSuccess;
  const int wpb = 8;
  dispatch_fp8_kernel<<<(a.num_units + wpb - 1) / wpb, wpb * 32, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_swiglu_quantize(const void* h, uint8_t* q, uint8_t* sfa, void* act, int rows, int F,
                                   const RowGroups* groups, cudaStream_t stream) {
  if (rows % 128 != 0 || F % 128 != 0) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  const int blocks = (rows + 7) / 8;
  swiglu_quantize_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(h), q, sfa,
                                                     reinterpret_cast<__nv_bfloat16*>(act), rows, F,
                                                     groups ? *groups : RowGroups{nullptr, nullptr, nullptr, 0});
  return cudaGetLastError();
}

cudaError_t launch_quantize_weights(const void* w, uint8_t* q, uint8_t* sfb, int slots, int N, int K,
                                    cudaStream_t stream) {
  if (N % 128 != 0 || K % 128 != 0) return cudaErrorInvalidValue;
  dim3 grid(K / 128, N / 128, slots);
  quantize_weights_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(w), q, sfb, N, K);
  return cudaGetLastError();
}

}  // namespace epb
