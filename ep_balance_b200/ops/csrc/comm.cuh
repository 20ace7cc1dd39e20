// Device side of the item-driven transport described at CommArgs (route.h): one warp per item,
// callable from a stand-alone kernel (route.cu) and from the spare warps of the grouped GEMM kernel
// (grouped_gemm.cu).
//
// Copy engine: every warp owns a small ring of shared-memory slots.  A row (or weight chunk) moves in
// segments: a lane issues a bulk async load (global -> shared, completion on the slot's mbarrier) and,
// once the segment has landed, a bulk async store (shared -> global, possibly a peer's memory); several
// lanes do so side by side, each for its own segment.  The segments in flight cost no register traffic, so
// two warps beside a running GEMM keep enough bytes outstanding to cover memory and NVLink latency.  No
// load names a cluster multicast; sources and destinations may be another GPU's memory.
//
// Nothing here waits on another CTA or rank, so a warp running it always makes progress; only the
// consumers of its signals wait, and those waits are bounded.  The waits on the warp's own copies are
// bounded too.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"
#include "route.h"

namespace epb {

constexpr int kCommSlotBytes = 4096;   // one segment
constexpr int kCommCtrlBytes = 192;    // per warp: up to 8 mbarriers
// Shared memory of one transport warp with a ring of kSlots segments (kSlots / 2 loads in flight).
template <int kSlots>
constexpr int comm_warp_bytes() { return kSlots * kCommSlotBytes + kCommCtrlBytes; }

static_assert(8 * 8 <= kCommCtrlBytes, "per-warp control block too small");

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

// The per-warp copy pipeline.  `smem` is the warp's private region: kSlots segments of ring (16-byte
// aligned) followed by kCommCtrlBytes of control data.  All 32 lanes call every member together.
//
// The ring is two halves of kBatch = kSlots / 2 segments.  A push moves one BATCH: lane l < kBatch gives its own
// segment (source, destination, bytes) and issues its own bulk load into slot l of the current half, then the
// lanes complete the previous batch (each waits on its slot's mbarrier and issues its own bulk store).  So one
// instruction issues kBatch copies -- the issuing lanes' instruction latency (mbarrier operations, bulk-copy
// issue), not the copy engine, was what bounded a warp that moved one segment per instruction -- and the loads
// of a batch are in flight while the previous batch is stored.  Bulk groups are per thread: every lane commits
// one group per batch (an empty one when it had nothing to store), so "all but the newest group have been
// read" means for each lane that its slot in the half it is about to reuse is free.
template <int kCommSlots>
struct CommPipe {
  static_assert(kCommSlots >= 4 && kCommSlots <= 8 && kCommSlots % 2 == 0, "ring of 4, 6 or 8 slots");
  static constexpr int kCommWarpBytes = kCommSlots * kCommSlotBytes;
  static constexpr int kBatch = kCommSlots / 2;  // segments per push; lanes [0, kBatch) own one each
  static constexpr int kSeg = kCommSlotBytes;    // bytes of one segment
  uint8_t* ring;
  uint64_t* bars;
  unsigned batches;        // batches pushed
  unsigned uses[2];        // this lane's loads issued into its slot of half 0 / 1 (mbarrier phase)
  void* pend_dst;          // this lane's segment of the batch whose loads are in flight
  int pend_bytes, pend_slot;
  uint32_t pend_parity;
  int lane;
  bool failed;
  int* status;
  // optional profiling (null: off): ns spent by lane 0 waiting for loads, for stores' reads, and draining
  unsigned long long* prof;
  unsigned long long t_load, t_read, t_drain, n_seg;

  __device__ __forceinline__ void init(uint8_t* smem, int* status_word, unsigned long long* prof_out = nullptr) {
    prof = prof_out;
    t_load = t_read = t_drain = n_seg = 0ull;
    ring = smem;
    bars = reinterpret_cast<uint64_t*>(smem + kCommWarpBytes);
    batches = 0u;
    uses[0] = uses[1] = 0u;
    pend_dst = nullptr;
    pend_bytes = 0;
    pend_slot = 0;
    pend_parity = 0u;
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

  // Complete the batch in flight: every lane waits for its own load and stores its segment.
  __device__ __forceinline__ void flush() {
    const unsigned long long p0 = prof ? globaltimer_ns() : 0ull;
    if (!failed) {
      bool ok = pend_bytes == 0;
      unsigned long long t0 = 0;
      for (unsigned spin = 0;; ++spin) {
        if (!ok) ok = comm_bar_try(&bars[pend_slot], pend_parity);
        if (__all_sync(0xffffffffu, ok)) break;
        if ((spin & 1023u) == 1023u) {
          unsigned long long now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > kWaitBudgetNs) failed = true;
        }
        if (__any_sync(0xffffffffu, failed)) {
          failed = true;
          break;
        }
      }
      if (failed && lane == 0) set_status(status, kStatusPipeTimeout, 8, (int)blockIdx.x);
    }
    if (prof) t_load += globaltimer_ns() - p0;
    if (lane < kBatch && batches > 0u) {
      if (pend_bytes > 0 && !failed) {
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                     ::"l"(pend_dst), "r"(comm_smem(ring + (size_t)pend_slot * kCommSlotBytes)), "r"((uint32_t)pend_bytes)
                     : "memory");
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");  // one group per lane and batch, possibly empty
    }
    pend_bytes = 0;
    __syncwarp();
  }

  // Start moving one batch: lane l < kBatch moves `bytes` (<= kSeg, multiple of 16; 0: nothing) from `src` to `dst`.
  // The arguments of the other lanes are ignored.
  __device__ __forceinline__ void push(const void* src, void* dst, int bytes) {
    const int h = (int)(batches & 1u);
    const int s = h * kBatch + lane;
    if (lane >= kBatch) bytes = 0;
    if (lane < kBatch && !failed) {
      // this lane's slot of half h was last read by the store of two batches ago, which is the newest group it has
      // committed (the previous batch's store is issued by the flush below)
      const unsigned long long p1 = prof ? globaltimer_ns() : 0ull;
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      if (bytes > 0) {
        comm_bar_expect(&bars[s], (uint32_t)bytes);
        comm_bulk_load(ring + (size_t)s * kCommSlotBytes, src, (uint32_t)bytes, &bars[s]);
      }
      if (prof) t_read += globaltimer_ns() - p1;
    }
    __syncwarp();
    if (prof) n_seg += (unsigned long long)__popc(__ballot_sync(0xffffffffu, bytes > 0));
    flush();  // the previous batch: its loads have been in flight for one batch
    pend_dst = dst;
    pend_bytes = bytes;
    pend_slot = s;
    pend_parity = uses[h] & 1u;
    if (bytes > 0) ++uses[h];
    ++batches;
  }

  // Finish everything in flight; on return the stores are complete and fenced for a following release.
  __device__ __forceinline__ void drain() {
    const unsigned long long p2 = prof ? globaltimer_ns() : 0ull;
    flush();
    if (lane < kBatch) {
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async;" ::: "memory");
    }
    __syncwarp();
    if (prof) t_drain += globaltimer_ns() - p2;
  }
  // add this warp's counters to prof[0..3] = {load waits, read waits, drains (incl. their load waits), batches x lanes}
  __device__ __forceinline__ void report() {
    if (prof != nullptr && lane == 0) {
      atomicAdd(prof, t_load);
      atomicAdd(prof + 1, t_read);
      atomicAdd(prof + 2, t_drain);
      atomicAdd(prof + 3, n_seg);
    }
  }
};

// The warp sends rows [row0, row0 + nrow) (nrow <= 32) of peer buffer `dbuf`; lane i holds the unit of
// row row0 + i in `my_u` and that unit's position in this rank's sorted order in `my_pos`.  Forward also stores
// {source rank, position} (where the host returns the row) and the unit's gate weight beside the row.
template <int kSlots>
__device__ __forceinline__ void comm_send_rows(const CommArgs& a, CommPipe<kSlots>& pipe, int my_u, int my_pos, int nrow, int row0,
                                               uint8_t* dbuf, int2* dmeta, float* drowp, int lane) {
  constexpr unsigned kAll = 0xffffffffu;
  constexpr int kSeg = CommPipe<kSlots>::kSeg, kBatch = CommPipe<kSlots>::kBatch;
  const int row_bytes = a.H * 2;
  if (lane < nrow) {
    if (dmeta != nullptr) dmeta[row0 + lane] = make_int2(a.me, my_pos);
    if (drowp != nullptr) drowp[row0 + lane] = a.unit_prob[my_u];
  }
  // (row, segment) pairs in order, kBatch of them per push: lane l takes pair first + l
  const int segs = (row_bytes + kSeg - 1) / kSeg;
  const int total = nrow * segs;
  for (int first = 0; first < total; first += kBatch) {
    const int idx = first + (lane < kBatch ? lane : 0);
    const int i = idx / segs, sg = idx - i * segs;
    const int u = __shfl_sync(kAll, my_u, i < nrow ? i : 0);
    const bool have = lane < kBatch && idx < total;
    const int off = sg * kSeg;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(a.rows) + (size_t)(u / a.topk) * row_bytes + off;
    uint8_t* dst = dbuf + (size_t)(row0 + i) * row_bytes + off;
    pipe.push(src, dst, have ? min(kSeg, row_bytes - off) : 0);
  }
}

// Replica weights (peer loads): the worker's share of the 32 KB chunks of every replica slot.
template <int kSlots>
__device__ inline void comm_pull(const CommArgs& a, CommPipe<kSlots>& pipe, int worker, int n_workers) {
  constexpr unsigned kAll = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  {
    constexpr int kSeg = CommPipe<kSlots>::kSeg;
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
        constexpr int kBatch = CommPipe<kSlots>::kBatch;
        for (int off0 = 0; off0 < n; off0 += kSeg * kBatch) {
          const int off = off0 + (lane < kBatch ? lane : 0) * kSeg;
          pipe.push(src + off, dst + off, off < n ? min(kSeg, n - off) : 0);
        }
        pipe.drain();
      }
      __threadfence();
      __syncwarp();
      if (lane == 0) red_release_gpu_add(a.pull_cnt + (size_t)j * rs + s, 1u);
    }
  }
}

// Token rows (peer stores): the warp draws blocks from the shared ticket counter, at most max_items of them.
template <int kSlots>
__device__ inline void comm_dispatch(const CommArgs& a, CommPipe<kSlots>& pipe, int max_items) {
  constexpr unsigned kAll = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  {
    int max_tiles = 0;
    for (int h = lane; h < a.R; h += 32) max_tiles = max(max_tiles, a.tiles_of[h]);
    for (int off = 16; off > 0; off >>= 1) max_tiles = max(max_tiles, __shfl_xor_sync(kAll, max_tiles, off));
    const int bpt = a.tile_rows / a.block_rows;
    const int n_items = max_tiles * bpt * a.R;
    for (int done = 0; done < max_items; ++done) {
      unsigned drawn = 0;
      if (lane == 0) drawn = atomicAdd(a.ticket, 1u);
      const int it = (int)__shfl_sync(kAll, drawn, 0);
      if (it >= n_items) break;
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
            comm_send_rows(a, pipe, my_u, pos + lane, nrow, row0, dbuf, dmeta, drowp, lane);
            pos += nrow;
          }
        }
      }
      // the block's copies are complete; the release orders them, and the lanes' plain stores (ordered before it
      // by the warp barrier), before the counter update that publishes the block
      pipe.drain();
      if (dmeta != nullptr || drowp != nullptr) __threadfence_system();  // every lane fences its own plain stores
      __syncwarp();
      if (lane == 0) red_release_sys_add(a.arrive_ptrs[dst] + a.arrive_off + r0 / a.tile_rows, 1u);
    }
  }
}

// This rank's padding rows.
__device__ inline void comm_pad(const CommArgs& a, int worker, int n_workers) {
  const int lane = threadIdx.x & 31;
  {
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
}

// Warp `worker` of `n_workers` takes chunks worker, worker + n_workers, ... of the replica weights and of the
// padding rows; blocks of token rows are drawn from the ticket counter.
// Called by whole warps (all 32 lanes active); `smem` = the warp's comm_warp_bytes<kSlots>().
// Order: the worker's first block of token rows (so that the consumer's first tiles complete early), then its
// share of the replica weights, then the remaining blocks, then its share of the padding rows.
template <int kSlots>
__device__ inline void comm_run(const CommArgs& a, int worker, int n_workers, uint8_t* smem, int* status,
                                unsigned long long* prof = nullptr) {
  CommPipe<kSlots> pipe;
  pipe.init(smem, status, prof);
  if (a.do_dispatch) comm_dispatch(a, pipe, 1);
  if (a.do_pull && a.w_slots > a.home_cap) comm_pull(a, pipe, worker, n_workers);
  if (a.do_dispatch) comm_dispatch(a, pipe, 0x7fffffff);
  if (a.do_pad) comm_pad(a, worker, n_workers);
  pipe.drain();
  pipe.report();
}


}  // namespace epb
