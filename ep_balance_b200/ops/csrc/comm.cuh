// Device side of the item-driven transport described at CommArgs (route.h): one warp per item,
// callable from a stand-alone kernel (route.cu) and from the spare warps of the grouped GEMM kernel
// (grouped_gemm.cu).
//
// Copy engine: every warp owns a small ring of shared-memory slots.  A row (or weight chunk) moves in
// segments: one lane issues a bulk async load (global -> shared, completion on the slot's mbarrier) and,
// once a segment has landed, a bulk async store (shared -> global, possibly a peer's memory).  Several
// segments per warp are in flight with no register traffic, so two warps beside a running GEMM keep
// enough bytes outstanding to cover memory and NVLink latency.  No load names a cluster multicast;
// sources and destinations may be another GPU's memory.
//
// Nothing here waits on another CTA or rank, so a warp running it always makes progress; only the
// consumers of its signals wait, and those waits are bounded.  The waits on the warp's own copies are
// bounded too.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"
#include "route.h"

namespace epb {

constexpr int kCommSlots = 4;          // ring slots per warp
constexpr int kCommSlotBytes = 4096;   // one segment
constexpr int kCommWarpBytes = kCommSlots * kCommSlotBytes;   // ring bytes per warp
constexpr int kCommCtrlBytes = 192;    // per warp: kCommSlots mbarriers + kCommSlots slot records

struct CommSlot {
  void* dst;       // where the segment goes
  int bytes;
  int pad;
};
static_assert(kCommSlots * 8 + kCommSlots * sizeof(CommSlot) <= kCommCtrlBytes, "per-warp control block too small");

__device__ __forceinline__ void red_release_gpu_add(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t comm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void comm_bar_init(uint64_t* bar) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(comm_smem(bar)) : "memory");
}
__device__ __forceinline__ void comm_bar_expect(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(comm_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool comm_bar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(comm_smem(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void comm_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(comm_smem(smem_dst)), "l"(gsrc), "r"(bytes), "r"(comm_smem(bar))
               : "memory");
}
__device__ __forceinline__ void comm_bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(comm_smem(smem_src)), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// The per-warp copy pipeline.  `smem` is the warp's private region: kCommWarpBytes of ring (16-byte
// aligned) followed by kCommCtrlBytes of control data.  All 32 lanes call every member together.
struct CommPipe {
  static constexpr int kSeg = kCommSlotBytes;  // bytes of one segment
  uint8_t* ring;
  uint64_t* bars;
  CommSlot* slots;
  unsigned pushed, popped;
  int lane;
  bool failed;
  int* status;

  __device__ __forceinline__ void init(uint8_t* smem, int* status_word) {
    ring = smem;
    bars = reinterpret_cast<uint64_t*>(smem + kCommWarpBytes);
    slots = reinterpret_cast<CommSlot*>(bars + kCommSlots);
    pushed = popped = 0u;
    lane = threadIdx.x & 31;
    failed = false;
    status = status_word;
    if (lane == 0) {
      for (int s = 0; s < kCommSlots; ++s) comm_bar_init(&bars[s]);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
  }

  // Oldest segment in flight: wait for its load, store it.
  __device__ __forceinline__ void pop() {
    const int s = (int)(popped % kCommSlots);
    const uint32_t parity = (popped / kCommSlots) & 1u;
    if (!failed) {
      unsigned long long t0 = 0;
      for (unsigned spin = 0; !comm_bar_try(&bars[s], parity); ++spin) {
        if ((spin & 1023u) == 1023u) {
          unsigned long long now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > kWaitBudgetNs) {
            failed = true;
            break;
          }
        }
      }
      failed = __any_sync(0xffffffffu, failed);
      if (failed && lane == 0) set_status(status, kStatusPipeTimeout, 8, (int)blockIdx.x);
    }
    const CommSlot rec = slots[s];
    uint8_t* seg = ring + (size_t)s * kCommSlotBytes;
    __syncwarp();
    if (lane == 0 && !failed) comm_bulk_store(rec.dst, seg, (uint32_t)rec.bytes);
    ++popped;
  }

  // Start moving `bytes` (<= kSeg, multiple of 16) from `src` to `dst`.
  __device__ __forceinline__ void push(const void* src, void* dst, int bytes) {
    if (pushed - popped >= (unsigned)(kCommSlots - 1)) pop();
    const int s = (int)(pushed % kCommSlots);
    if (lane == 0 && !failed) {
      // every store but the most recent one has finished reading its slot; slot s was stored two pops ago
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      slots[s] = CommSlot{dst, bytes, 0};
      uint8_t* seg = ring + (size_t)s * kCommSlotBytes;
      comm_bar_expect(&bars[s], (uint32_t)bytes);
      comm_bulk_load(seg, src, (uint32_t)bytes, &bars[s]);
    }
    __syncwarp();
    ++pushed;
  }

  // Finish everything in flight; on return the stores are complete and fenced for a following release.
  __device__ __forceinline__ void drain() {
    while (popped != pushed) pop();
    if (lane == 0) {
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async;" ::: "memory");
    }
    __syncwarp();
  }
};

// The warp sends rows [row0, row0 + nrow) (nrow <= 32) of peer buffer `dbuf`; lane i holds the unit of
// row row0 + i in `my_u`.  Forward also stores {source rank, unit} and the unit's gate weight beside the row.
__device__ __forceinline__ void comm_send_rows(const CommArgs& a, CommPipe& pipe, int my_u, int nrow, int row0,
                                               uint8_t* dbuf, int2* dmeta, float* drowp, int lane) {
  constexpr unsigned kAll = 0xffffffffu;
  constexpr int kSeg = CommPipe::kSeg;
  const int row_bytes = a.H * 2;
  if (lane < nrow) {
    if (dmeta != nullptr) dmeta[row0 + lane] = make_int2(a.me, my_u);
    if (drowp != nullptr) drowp[row0 + lane] = a.unit_prob[my_u];
  }
  for (int i = 0; i < nrow; ++i) {
    const int u = __shfl_sync(kAll, my_u, i);
    const uint8_t* src = reinterpret_cast<const uint8_t*>(a.rows) + (size_t)(u / a.topk) * row_bytes;
    uint8_t* dst = dbuf + (size_t)(row0 + i) * row_bytes;
    for (int off = 0; off < row_bytes; off += kSeg) pipe.push(src + off, dst + off, min(kSeg, row_bytes - off));
  }
}

// Warp `worker` of `n_workers` takes items worker, worker + n_workers, ... of each item list.
// Called by whole warps (all 32 lanes active); `smem` = the warp's kCommWarpBytes + kCommCtrlBytes.
__device__ inline void comm_run(const CommArgs& a, int worker, int n_workers, uint8_t* smem, int* status) {
  constexpr unsigned kAll = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  CommPipe pipe;
  pipe.init(smem, status);

  // ---------------------------------------------------------------- replica weights (peer loads)
  if (a.do_pull && a.w_slots > a.home_cap) {
    constexpr int kSeg = CommPipe::kSeg;
    const int rs = a.w_slots - a.home_cap;
    const int c1 = (int)pull_chunks(a.w1_elems), c2 = (int)pull_chunks(a.w2_elems);
    const int n_items = rs * (c1 + c2);
    for (int it = worker; it < n_items; it += n_workers) {
      // every slot's w1 first (the first GEMM waits for it), then w2; slot-major inside a tensor
      const int j = it < rs * c1 ? 0 : 1;
      const int rem = j ? it - rs * c1 : it;
      const int cj = j ? c2 : c1;
      const int s = rem / cj, c = rem - s * cj;
      int e = -1;
      for (int g0 = 0; g0 < a.n_groups_cap && e < 0; g0 += 32) {
        const int g = g0 + lane;
        const int ge = (g < a.n_groups_cap && a.group_wslot[g] == a.home_cap + s) ? a.group_expert[g] : -1;
        const unsigned m = __ballot_sync(kAll, ge >= 0);
        if (m) e = __shfl_sync(kAll, ge, __ffs(m) - 1);
      }
      if (e >= 0 && a.main_rank[e] != a.me) {
        const size_t slot_bytes = (j ? a.w2_elems : a.w1_elems) * 2;
        void* const* ptrs = j ? a.w2_ptrs : a.w1_ptrs;
        const size_t first = (size_t)c * kPullChunkBytes;
        const int n = (int)(slot_bytes - first < (size_t)kPullChunkBytes ? slot_bytes - first : (size_t)kPullChunkBytes);
        const uint8_t* src = reinterpret_cast<const uint8_t*>(ptrs[a.main_rank[e]]) + (size_t)a.home_index[e] * slot_bytes + first;
        uint8_t* dst = reinterpret_cast<uint8_t*>(ptrs[a.me]) + (size_t)(a.home_cap + s) * slot_bytes + first;
        for (int off = 0; off < n; off += kSeg) pipe.push(src + off, dst + off, min(kSeg, n - off));
        pipe.drain();
      }
      __threadfence();
      __syncwarp();
      if (lane == 0) red_release_gpu_add(a.pull_cnt + (size_t)j * rs + s, 1u);
    }
  }

  // ---------------------------------------------------------------- token rows (peer stores)
  if (a.do_dispatch) {
    int max_tiles = 0;
    for (int h = lane; h < a.R; h += 32) max_tiles = max(max_tiles, a.tiles_of[h]);
    for (int off = 16; off > 0; off >>= 1) max_tiles = max(max_tiles, __shfl_xor_sync(kAll, max_tiles, off));
    const int bpt = a.tile_rows / a.block_rows;
    const int n_items = max_tiles * bpt * a.R;
    for (int it = worker; it < n_items; it += n_workers) {
      const int b = it / a.R, k = it - b * a.R;
      int dst = a.me + k;
      if (dst >= a.R) dst -= a.R;
      if (b >= a.tiles_of[dst] * bpt) continue;
      const int r0 = b * a.block_rows, r1 = r0 + a.block_rows;
      uint8_t* dbuf = reinterpret_cast<uint8_t*>(a.buf_ptrs[dst]);
      int2* dmeta = a.meta_ptrs != nullptr ? a.meta_ptrs[dst] : nullptr;
      float* drowp = (a.rowp_ptrs != nullptr && a.unit_prob != nullptr) ? a.rowp_ptrs[dst] : nullptr;
      for (int e0 = 0; e0 < a.E; e0 += 32) {
        const int e = e0 + lane;
        int base = -1, cnt = 0;
        if (e < a.E) {
          base = a.row_base[(size_t)e * a.R + dst];
          cnt = a.q_me[(size_t)e * a.R + dst];
        }
        const int lo = max(base, r0), hi = min(base + cnt, r1);
        unsigned m = __ballot_sync(kAll, base >= 0 && lo < hi);
        while (m) {
          const int sl = __ffs(m) - 1;
          m &= m - 1;
          const int slo = __shfl_sync(kAll, lo, sl), shi = __shfl_sync(kAll, hi, sl), sbase = __shfl_sync(kAll, base, sl);
          const int se = e0 + sl;
          int pos = a.exp_prefix[se] + a.send_off[(size_t)se * a.R + dst] + (slo - sbase);
          for (int row0 = slo; row0 < shi; row0 += 32) {
            const int nrow = min(32, shi - row0);
            const int my_u = lane < nrow ? a.sorted_units[pos + lane] : 0;
            comm_send_rows(a, pipe, my_u, nrow, row0, dbuf, dmeta, drowp, lane);
            pos += nrow;
          }
        }
      }
      // the block's copies are complete; every lane's plain stores are fenced; one lane publishes the block
      pipe.drain();
      __threadfence_system();
      __syncwarp();
      if (lane == 0) red_release_sys_add(a.arrive_ptrs[dst] + a.arrive_off + r0 / a.tile_rows, 1u);
    }
  }

  // ---------------------------------------------------------------- this rank's padding rows
  if (a.do_pad) {
    const int vec_per_row = a.H / 8;
    const int sub = a.tile_rows / 32;  // a group's padding is shorter than one tile
    const int n_items = a.n_groups_cap * sub;
    uint4* buf = reinterpret_cast<uint4*>(a.local_buf);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int it = worker; it < n_items; it += n_workers) {
      const int g = it / sub, s = it - g * sub;
      const int end = min(a.group_off[g + 1], a.row_capacity);
      const int lo = min(a.group_off[g] + a.group_rows[g] + 32 * s, end), hi = min(lo + 32, end);
      const size_t first = (size_t)lo * vec_per_row, last = (size_t)hi * vec_per_row;
      for (size_t i = first + lane; i < last; i += 32) buf[i] = zero;
      if (a.local_meta != nullptr && lo + lane < hi) a.local_meta[lo + lane] = make_int2(-1, -1);
    }
  }
  pipe.drain();
}

}  // namespace epb
