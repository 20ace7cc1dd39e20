// On-device plan solver: one cooperative launch computes placement x, routing quota q and
// the per-rank routing tables, with no host decision and no q memset.
//
// Semantics (must equal solver/device_semantics.py element for element; they restate the
// reference's CUDA path, eplb/cuda_solve.py:36-68 and eplb/csrc/fast_solver.cu:34-643):
//   phase 0  per domain: demand T[d,e], gate + benefit, stable descending order, greedy admission
//   phase 1  per (src, e): even split over active hosts in ascending rank id
//   phase 2  per domain: bounded greedy repair (busiest rank -> best (expert, target))
//   phase 3  routing tables for the calling rank (slot layout, destination row bases)
// The reference spends a sort + ~10 torch kernels + 3 launches and R*E blocks on this; here phases are
// separated by a bounded grid barrier inside one launch, one CTA per domain.  On the common path (<= 64
// ranks, the domain's quota columns fit in shared memory) a CTA routes exactly its own domain's columns
// straight into the shared-memory state the repair loop works on, so phases 1 and 2 need no barrier and no
// cache fill between them; walks that cannot change anything (no free slot left, nothing movable) stop early.
#include "solver.h"

#include <cooperative_groups.h>

#include "common.cuh"

namespace epb {
namespace {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

struct Cand {
  int delta, load, cost, expert, target;
};
__device__ __forceinline__ Cand no_cand() { return Cand{0, INT_MAX, INT_MAX, INT_MAX, INT_MAX}; }
__device__ __forceinline__ bool better(const Cand& a, const Cand& b) {
  if (a.delta != b.delta) return a.delta > b.delta;
  if (a.load != b.load) return a.load < b.load;
  if (a.cost != b.cost) return a.cost < b.cost;
  if (a.expert != b.expert) return a.expert < b.expert;
  return a.target < b.target;
}
__device__ __forceinline__ Cand warp_best(Cand v) {
  for (int off = kWarp / 2; off > 0; off >>= 1) {
    Cand o{__shfl_down_sync(kFull, v.delta, off), __shfl_down_sync(kFull, v.load, off),
           __shfl_down_sync(kFull, v.cost, off), __shfl_down_sync(kFull, v.expert, off),
           __shfl_down_sync(kFull, v.target, off)};
    if (better(o, v)) v = o;
  }
  return v;
}

__device__ __forceinline__ int safe_move(int have, int there, int left, int u_min) {
  int upper = min(have, left);
  if (upper <= 0) return 0;
  if (upper == have && there + upper >= u_min) return upper;
  int cap = min(upper, max(have - u_min, 0));
  return cap >= (there > 0 ? 1 : u_min) ? cap : 0;
}

// Bounded grid barrier on a monotonically increasing arrival counter.  All CTAs of the launch
// are co-resident (cooperative launch).  Returns false when the wait ran out.
__device__ bool grid_barrier(const SolverParams& p, int site) {
  __shared__ int ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    ok = 1;
    if (gridDim.x > 1) {
      __threadfence();
      unsigned old = atomicAdd(p.sync, 1u);
      unsigned target = (old / gridDim.x + 1u) * gridDim.x;
      if (!wait_ge<false>(p.sync, target, kWaitBudgetNs)) {
        set_status(p.status, kStatusBarrierTimeout, site);
        ok = 0;
      }
      __threadfence();
    }
  }
  __syncthreads();
  return ok != 0;
}

struct Smem {
  long long* prio;  // [E]
  int* order;       // [E]
  int* dom_ranks;   // [R] ranks of the domain being processed, ascending
  int* local_idx;   // [R] rank -> index in dom_ranks or -1
  int* load;        // [R] by domain-local index
  int* slot;        // [R]
  int* stuck;       // [R]
  Cand* wcand;      // [32]
  int* erl_c;       // [E * n] cached erl[e, domain rank] of the domain being repaired (or null)
  signed char* x_c; // [E * n] cached x[e, domain rank]
  int* q_c;         // [R * E * n] cached q[s, e, domain rank] (or unused)
};

__host__ __device__ inline int pow2_at_least(int n) {
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}

__device__ Smem carve(unsigned char* base, int R, int E) {
  Smem s;
  const int P = pow2_at_least(E) < 32 ? 32 : pow2_at_least(E);  // the candidate sort works on a power-of-two array
  s.prio = reinterpret_cast<long long*>(base);
  base += sizeof(long long) * P;
  s.order = reinterpret_cast<int*>(base);
  base += sizeof(int) * P;
  s.dom_ranks = reinterpret_cast<int*>(base);
  base += sizeof(int) * R;
  s.local_idx = reinterpret_cast<int*>(base);
  base += sizeof(int) * R;
  s.load = reinterpret_cast<int*>(base);
  base += sizeof(int) * R;
  s.slot = reinterpret_cast<int*>(base);
  base += sizeof(int) * R;
  s.stuck = reinterpret_cast<int*>(base);
  base += sizeof(int) * R;
  s.wcand = reinterpret_cast<Cand*>(base);
  base += sizeof(Cand) * 32;
  s.erl_c = reinterpret_cast<int*>(base);
  s.x_c = reinterpret_cast<signed char*>(base + sizeof(int) * (size_t)E * R);
  s.q_c = reinterpret_cast<int*>(base + (((size_t)E * R * 5 + 15) / 16) * 16);
  return s;
}

// Ranks of domain d in ascending id (s.dom_ranks) and every rank's index in that list or -1 (s.local_idx).
// One warp compacts 32 ranks per step with a ballot; the loads of a step are one coalesced request.
__device__ int collect_domain(const SolverParams& p, Smem& s, int d) {
  __shared__ int n_sh;
  __syncthreads();
  if (threadIdx.x < kWarp) {
    const int lane = threadIdx.x;
    int n = 0;
    for (int base = 0; base < p.R; base += kWarp) {
      const int r = base + lane;
      const bool in = r < p.R && p.dom[r] == d;
      const unsigned m = __ballot_sync(kFull, in);
      if (r < p.R) s.local_idx[r] = in ? n + __popc(m & ((1u << lane) - 1u)) : -1;
      if (in) s.dom_ranks[n + __popc(m & ((1u << lane) - 1u))] = r;
      n += __popc(m);
    }
    if (lane == 0) n_sh = n;
  }
  __syncthreads();
  return n_sh;
}

// ------------------------------------------------------------------ phase 0
__device__ void phase0_domain(const SolverParams& p, Smem& s, int d) {
  __shared__ int n_valid;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int R = p.R, E = p.E;
  const int n = collect_domain(p, s, d);
  if (n == 0) return;
  // With the cache region available the domain's placement columns live in shared memory while
  // candidates are admitted (one global round trip per candidate otherwise) and are stored once.
  signed char* xc = p.cache_stage2 ? s.x_c : nullptr;
  if (tid == 0) n_valid = 0;
  for (int i = tid; i < n; i += nt) s.slot[i] = 0;
  __syncthreads();
  // owners: x[e, r] = (main(e) == r) for this domain's columns; slots used by owners
  for (int idx = tid; idx < E * n; idx += nt) {
    int e = idx / n, i = idx - e * n;
    int r = s.dom_ranks[i];
    bool own = p.main_rank[e] == r;
    if (xc) xc[idx] = own ? 1 : 0;
    else p.x[(size_t)e * R + r] = own ? 1 : 0;
    if (own) atomicAdd(&s.slot[i], 1);
  }
  // gate and benefit
  for (int e = tid; e < E; e += nt) {
    long long T = 0;
    const int owner = __ldg(p.main_rank + e);
    const long long wb = __ldg(p.weight_bytes + e);
    for (int i = 0; i < n; ++i) T += __ldg(p.omega + (size_t)s.dom_ranks[i] * E + e);
    long long rhs = 2 * T * p.s_tok;
    bool valid = p.allow_cross && __ldg(p.dom + owner) != d && T > 0 && wb < rhs;
    s.prio[e] = valid ? rhs - wb : -1;
    if (valid) atomicAdd(&n_valid, 1);
  }
  __syncthreads();
  const int nv = n_valid;
  if (nv > 0) {
    // Descending benefit, ties by ascending expert id (what a stable descending sort of the row gives).  The
    // (benefit, id) pairs are distinct, so any comparison sort yields this one order: a bitonic sort,
    // O(E log^2 E / threads) instead of counting all pairs.  Invalid entries (-1) and the padding (-2) sink
    // to the end.
    const int P = max(pow2_at_least(E), kWarp);
    if (P <= nt) {
      // one element per thread, kept in registers: exchanges at distance < 32 are warp shuffles, only the
      // longer ones go through shared memory (10 of the 45 steps at 512 experts)
      long long mp = tid < E ? s.prio[tid] : -2;
      int me = tid;
      __syncthreads();
      for (int k = 2; k <= P; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
          long long op;
          int oe;
          if (j >= kWarp) {
            if (tid < P) {
              s.prio[tid] = mp;
              s.order[tid] = me;
            }
            __syncthreads();
            op = tid < P ? s.prio[tid ^ j] : -2;
            oe = tid < P ? s.order[tid ^ j] : tid;
            __syncthreads();
          } else {
            op = __shfl_xor_sync(kFull, mp, j);
            oe = __shfl_xor_sync(kFull, me, j);
          }
          const bool mine_first = mp > op || (mp == op && me < oe);  // does my element precede the partner's?
          const bool keep_first = ((tid & j) == 0) == ((tid & k) == 0);
          if (mine_first != keep_first) {
            mp = op;
            me = oe;
          }
        }
      }
      if (tid < P) s.order[tid] = me;
      __syncthreads();
    } else {
      for (int i = tid; i < P; i += nt) {
        s.order[i] = i;
        if (i >= E) s.prio[i] = -2;
      }
      __syncthreads();
      for (int k = 2; k <= P; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
          for (int t = tid; t < P / 2; t += nt) {
            const int lo = ((t & ~(j - 1)) << 1) | (t & (j - 1)), hi = lo | j;
            const long long pl = s.prio[lo], ph = s.prio[hi];
            const int el = s.order[lo], eh = s.order[hi];
            const bool lo_first = pl > ph || (pl == ph && el < eh);   // does `lo` precede `hi` in the wanted order?
            const bool ascending_block = (lo & k) == 0;               // blocks alternate direction
            if (lo_first != ascending_block) {
              s.prio[lo] = ph;
              s.prio[hi] = pl;
              s.order[lo] = eh;
              s.order[hi] = el;
            }
          }
          __syncthreads();
        }
      }
    }
    if (tid < kWarp) {
      const int lane = tid;
      // free slots left in the domain: once they are used up no later candidate can be admitted, so the walk stops
      int free_left = 0;
      for (int i = lane; i < n; i += kWarp) free_left += max(p.n_slot - s.slot[i], 0);
      for (int off = kWarp / 2; off > 0; off >>= 1) free_left += __shfl_xor_sync(kFull, free_left, off);
      for (int c = 0; c < nv && free_left > 0; ++c) {
        const int e = s.order[c];
        bool present = false;
        long long key = LLONG_MAX;  // (slots used, domain-local index) of the best free rank
        for (int i = lane; i < n; i += kWarp) {
          const bool here = xc ? xc[e * n + i] != 0 : p.x[(size_t)e * R + s.dom_ranks[i]] != 0;
          if (here) present = true;
          int used = s.slot[i];
          if (used < p.n_slot) key = min(key, ((long long)used << 32) | (unsigned)i);
        }
        const unsigned any = __ballot_sync(kFull, present);
        for (int off = kWarp / 2; off > 0; off >>= 1) key = min(key, __shfl_xor_sync(kFull, key, off));
        if (any == 0 && key != LLONG_MAX) {  // the same decision on every lane
          if (lane == 0) {
            int i = (int)(key & 0xffffffffll);
            if (xc) xc[e * n + i] = 1;
            else p.x[(size_t)e * R + s.dom_ranks[i]] = 1;
            s.slot[i] += 1;
          }
          --free_left;
        }
        __syncwarp(kFull);
      }
    }
  }
  __syncthreads();
  if (xc)
    for (int idx = tid; idx < E * n; idx += nt) {
      int e = idx / n, i = idx - e * n;
      p.x[(size_t)e * R + s.dom_ranks[i]] = xc[idx];
    }
  for (int i = tid; i < n; i += nt) p.slot_used[s.dom_ranks[i]] = s.slot[i];
}

// ------------------------------------------------------------------ phase 1
// Units a destination gets from one (src, e) pair under the even split: `act` is the set of active
// hosts (bit per rank), `dst` one of them.
__device__ __forceinline__ int even_share(int need, unsigned long long act, int dst, int u_min) {
  const int count = __popcll(act);
  if (need <= 0 || count == 0) return 0;
  int n = count;
  if (u_min > 1 && need >= u_min) n = min(count, need / u_min);
  else if (need < u_min) n = 1;
  const int pos = __popcll(act & ((1ull << dst) - 1ull));
  return pos < n ? need / n + (pos < need % n ? 1 : 0) : 0;
}

// R <= 64: one thread per (src, e) pair writes its row of q, one thread per (e, dst) pair sums
// erl; host sets are 64-bit masks held in shared memory.  Every pair is independent, so the whole
// grid works on them at once instead of one warp walking an expert's sources serially.
__device__ void phase1_routing_masks(const SolverParams& p, Smem& s) {
  __shared__ unsigned long long dom_mask[64];
  const int R = p.R, E = p.E, u_min = p.u_min;
  const int tid = threadIdx.x, nt = blockDim.x;
  unsigned long long* host = reinterpret_cast<unsigned long long*>(s.prio);  // [E]
  __syncthreads();
  for (int e = tid; e < E; e += nt) {
    unsigned long long m = 0;
    for (int dst = 0; dst < R; ++dst) m |= (unsigned long long)(p.x[(size_t)e * R + dst] != 0) << dst;
    host[e] = m;
  }
  for (int r = tid; r < R; r += nt) {
    unsigned long long m = 0;
    const int dr = p.dom[r];
    for (int o = 0; o < R; ++o) m |= (unsigned long long)(p.dom[o] == dr) << o;
    dom_mask[r] = m;
  }
  __syncthreads();
  const int gtid = blockIdx.x * nt + tid, gthreads = gridDim.x * nt;
  for (int pair = gtid; pair < R * E; pair += gthreads) {
    const int src = pair / E, e = pair - src * E;
    const int need = p.omega[pair];
    const unsigned long long loc = host[e] & dom_mask[src];
    const unsigned long long act = loc ? loc : host[e];
    int* qrow = p.q + (size_t)pair * R;
    for (int dst = 0; dst < R; ++dst) qrow[dst] = ((act >> dst) & 1ull) ? even_share(need, act, dst, u_min) : 0;
  }
  for (int cell = gtid; cell < E * R; cell += gthreads) {
    const int e = cell / R, dst = cell - e * R;
    int acc = 0;
    if ((host[e] >> dst) & 1ull) {
      for (int src = 0; src < R; ++src) {
        const unsigned long long loc = host[e] & dom_mask[src];
        const unsigned long long act = loc ? loc : host[e];
        if ((act >> dst) & 1ull) acc += even_share(p.omega[(size_t)src * E + e], act, dst, u_min);
      }
    }
    p.erl[cell] = acc;
  }
}

// One CTA computes exactly the quota columns of ITS domain's ranks (all sources, all experts), straight
// into the shared-memory caches that the repair loop works on, and stores them to global memory on the
// way.  The repair loop then needs neither a grid barrier after routing nor a cache fill.
// Requires R <= 64 and the quota cache (s.q_c, s.erl_c) of this domain to fit.
__device__ void phase1_domain(const SolverParams& p, Smem& s, int d) {
  __shared__ unsigned long long dom_mask[64];
  const int R = p.R, E = p.E, u_min = p.u_min;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int n = collect_domain(p, s, d);
  if (n == 0) return;
  unsigned long long* host = reinterpret_cast<unsigned long long*>(s.prio);  // [E]
  for (int e = tid; e < E; e += nt) {
    unsigned long long m = 0;
    for (int dst = 0; dst < R; ++dst) m |= (unsigned long long)(p.x[(size_t)e * R + dst] != 0) << dst;
    host[e] = m;
  }
  for (int r = tid; r < R; r += nt) {
    unsigned long long m = 0;
    const int dr = p.dom[r];
    for (int o = 0; o < R; ++o) m |= (unsigned long long)(p.dom[o] == dr) << o;
    dom_mask[r] = m;
  }
  __syncthreads();
  // the loads of the next pair are issued before the stores of the current one (the compiler cannot reorder them
  // itself: q and omega might alias for all it knows)
  int need_next = tid < R * E ? __ldg(p.omega + tid) : 0;
  for (int pair = tid; pair < R * E; pair += nt) {
    const int src = pair / E, e = pair - src * E;
    const int need = need_next;
    if (pair + nt < R * E) need_next = __ldg(p.omega + pair + nt);
    const unsigned long long loc = host[e] & dom_mask[src];
    const unsigned long long act = loc ? loc : host[e];
    // the even split of even_share(), with its divisions done once per pair instead of once per destination
    const int count = __popcll(act);
    int takers = count;
    if (u_min > 1 && need >= u_min) takers = min(count, need / u_min);
    else if (need < u_min) takers = 1;
    const bool any = need > 0 && count > 0;
    const int base = any ? need / takers : 0, extra = any ? need - base * takers : 0;
    int* qrow = p.q + (size_t)pair * R;
    int* crow = s.q_c + (size_t)pair * n;
    for (int i = 0; i < n; ++i) {
      const int dst = s.dom_ranks[i];
      int v = 0;
      if (any && ((act >> dst) & 1ull)) {
        const int pos = __popcll(act & ((1ull << dst) - 1ull));
        if (pos < takers) v = base + (pos < extra ? 1 : 0);
      }
      qrow[dst] = v;
      crow[i] = v;
    }
  }
  __syncthreads();
  for (int cell = tid; cell < E * n; cell += nt) {
    const int e = cell / n, i = cell - e * n;
    int acc = 0;
    for (int src = 0; src < R; ++src) acc += s.q_c[((size_t)src * E + e) * n + i];
    s.erl_c[cell] = acc;
    p.erl[(size_t)e * R + s.dom_ranks[i]] = acc;
    s.x_c[cell] = (signed char)((host[e] >> s.dom_ranks[i]) & 1ull);
  }
  __syncthreads();
}

__device__ void phase1_routing(const SolverParams& p) {
  const int R = p.R, E = p.E, u_min = p.u_min;
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int gwarp = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int total_warps = gridDim.x * warps_per_block;
  const unsigned lt = (1u << lane) - 1u;
  for (int e = gwarp; e < E; e += total_warps) {
    int* erl = p.erl + (size_t)e * R;
    const signed char* xe = p.x + (size_t)e * R;
    for (int dst = lane; dst < R; dst += kWarp) erl[dst] = 0;
    __syncwarp(kFull);
    for (int src = 0; src < R; ++src) {
      const int need = p.omega[(size_t)src * E + e];
      const int dsrc = p.dom[src];
      int cnt_all = 0, cnt_loc = 0;
      for (int base = 0; base < R; base += kWarp) {
        int dst = base + lane;
        bool h = dst < R && xe[dst] != 0;
        bool loc = h && p.dom[dst] == dsrc;
        cnt_all += __popc(__ballot_sync(kFull, h));
        cnt_loc += __popc(__ballot_sync(kFull, loc));
      }
      const bool has_local = cnt_loc > 0;
      const int count = has_local ? cnt_loc : cnt_all;
      int n = count;
      if (u_min > 1 && need >= u_min) n = min(count, need / u_min);
      else if (need < u_min) n = 1;
      int seen = 0;
      int* qrow = p.q + ((size_t)src * E + e) * R;
      for (int base = 0; base < R; base += kWarp) {
        int dst = base + lane;
        bool h = dst < R && xe[dst] != 0;
        bool act = h && (!has_local || p.dom[dst] == dsrc);
        unsigned m = __ballot_sync(kFull, act);
        int pos = seen + __popc(m & lt);
        int give = 0;
        if (act && need > 0 && count > 0 && pos < n) give = need / n + (pos < need % n ? 1 : 0);
        if (dst < R) {
          qrow[dst] = give;
          if (give) erl[dst] += give;
        }
        seen += __popc(m);
      }
    }
  }
}

// ------------------------------------------------------------------ phase 2
struct ProbeState {
  bool on;
  int patience;
};

// prefilled: phase1_domain of this CTA has just left this domain's q / erl / x columns in the caches.
__device__ void stage2_domain(const SolverParams& p, Smem& s, int d, int iters, ProbeState probe, bool fresh,
                              bool prefilled = false) {
  __shared__ int busy_idx, busy_rank, busy_load, finished, sel_idx, apply_move;
  __shared__ int best_theta, stagnant;
  __shared__ Cand best_sh;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
  const int R = p.R, E = p.E, u_min = p.u_min;
  const int n = collect_domain(p, s, d);
  if (n == 0) return;
  if (fresh) {
    // first repair pass after routing: this domain's rank loads are column sums of erl
    const int lane_ = tid & 31, warp_ = tid >> 5, nwarps_ = nt >> 5;
    for (int i = warp_; i < n; i += nwarps_) {
      const int r = s.dom_ranks[i];
      int acc = 0;
      for (int e = lane_; e < E; e += kWarp) acc += prefilled ? s.erl_c[e * n + i] : p.erl[(size_t)e * R + r];
      for (int off = kWarp / 2; off > 0; off >>= 1) acc += __shfl_down_sync(kFull, acc, off);
      if (lane_ == 0) {
        s.load[i] = acc;
        s.slot[i] = p.slot_used[r];
        s.stuck[i] = 0;
      }
    }
  } else {
    for (int i = tid; i < n; i += nt) {
      int r = s.dom_ranks[i];
      s.load[i] = p.rank_load[r];
      s.slot[i] = p.slot_used[r];
      s.stuck[i] = probe.on ? p.stuck[r] : 0;
    }
  }
  // The repair loop re-reads erl[e, r] and x[e, r] of this domain's ranks on every iteration;
  // keep them in shared memory (when they fit) so an iteration costs no global round trips
  // beyond the quota move itself.  Global copies are kept up to date for the later phases.
  const bool cached = p.cache_stage2 != 0;
  const bool qcached = p.cache_q != 0 && u_min == 1;  // the quota columns of this domain's ranks too
  if (qcached && !prefilled) {
    for (int idx = tid; idx < R * E * n; idx += nt) {
      const int se = idx / n, i = idx - se * n;
      s.q_c[idx] = p.q[(size_t)se * R + s.dom_ranks[i]];
    }
  }
  if (cached && !prefilled) {
    for (int idx = tid; idx < E * n; idx += nt) {
      const int e = idx / n, i = idx - e * n;
      const int r = s.dom_ranks[i];
      s.erl_c[idx] = p.erl[(size_t)e * R + r];
      s.x_c[idx] = p.x[(size_t)e * R + r];
    }
  }
  __syncthreads();

  // A move needs a target that already hosts the expert or has a free slot.  When no rank of the domain has a
  // free slot and no expert has two hosts inside the domain, no iteration can ever move anything: the loop
  // would only mark the loaded ranks stuck one by one.  Write that outcome down directly.
  if (cached && !probe.on) {
    __shared__ int movable;
    if (tid == 0) {
      movable = 0;
      for (int i = 0; i < n; ++i)
        if (s.slot[i] < p.n_slot) movable = 1;
    }
    __syncthreads();
    if (!movable) {
      for (int e = tid; e < E; e += nt) {
        int hosts = 0;
        for (int i = 0; i < n; ++i) hosts += s.x_c[e * n + i] != 0;
        if (hosts > 1) movable = 1;  // benign race: every writer stores 1
      }
    }
    __syncthreads();
    if (tid == 0 && !movable) {
      int loaded = 0;
      for (int i = 0; i < n; ++i) loaded += s.load[i] > 0;
      if (loaded > iters) movable = 1;  // the loop would stop early: let it run
    }
    __syncthreads();
    if (!movable) {
      if (tid == 0) {
        // the loop marks the ranks busiest first and stops at the first rank with no load, which stays unmarked
        for (int i = 0; i < n; ++i) s.stuck[i] = s.load[i] > 0 ? 1 : 0;
      }
      __syncthreads();
      iters = 0;
    }
  }

  for (int it = 0; it < iters; ++it) {
    if (tid == 0) {
      int bi = -1, br = -1, bl = -1, theta = -1;
      for (int i = 0; i < n; ++i) {
        int l = s.load[i];
        theta = max(theta, l);
        if (s.stuck[i] == 0 && l > bl) {  // ascending rank order: first max wins ties
          bi = i;
          br = s.dom_ranks[i];
          bl = l;
        }
      }
      bool stop = false;
      if (probe.on) {
        if (it == 0 || theta < best_theta) {
          best_theta = theta;
          stagnant = 0;
        } else {
          ++stagnant;
        }
        stop = stagnant >= probe.patience;
      }
      busy_idx = bi;
      busy_rank = br;
      busy_load = bl;
      finished = stop || br < 0 || bl <= 0;
    }
    __syncthreads();
    if (finished) break;
    const int src = busy_rank, top = busy_load;

    Cand mine = no_cand();
    for (int e = tid; e < E; e += nt) {
      const int avail = cached ? s.erl_c[e * n + busy_idx] : p.erl[(size_t)e * R + src];
      if (avail <= 0) continue;
      for (int ti = 0; ti < n; ++ti) {
        const int t = s.dom_ranks[ti], tl = s.load[ti];
        if (t == src || tl >= top) continue;
        const bool host = cached ? s.x_c[e * n + ti] != 0 : p.x[(size_t)e * R + t] != 0;
        if (!host && s.slot[ti] >= p.n_slot) continue;
        const int delta = min(avail, (top - tl) / 2);
        if (delta < u_min) continue;
        Cand c{delta, tl, p.cost[(size_t)src * R + t], e, t};
        if (better(c, mine)) mine = c;
      }
    }
    mine = warp_best(mine);
    if (lane == 0) s.wcand[warp] = mine;
    __syncthreads();
    if (warp == 0) {
      Cand c = lane < nwarps ? s.wcand[lane] : no_cand();
      c = warp_best(c);
      if (lane == 0) best_sh = c;
    }
    __syncthreads();
    const Cand best = best_sh;

    if (u_min == 1) {
      if (tid == 0) {
        sel_idx = best.delta > 0 ? s.local_idx[best.target] : -1;
        apply_move = best.delta > 0 && sel_idx >= 0;
        if (!apply_move) {
          s.stuck[busy_idx] = 1;
        } else {
          signed char* cell = p.x + (size_t)best.expert * R + best.target;
          const bool hosted = cached ? s.x_c[best.expert * n + sel_idx] != 0 : *cell != 0;
          if (!hosted) {
            *cell = 1;
            if (cached) s.x_c[best.expert * n + sel_idx] = 1;
            s.slot[sel_idx] += 1;
          }
        }
      }
      __syncthreads();
      if (apply_move) {
        if (warp == 0) {
          // prefix over source ranks: source s gives min(q_s, max(delta - sum_{s'<s} q_s', 0))
          int carry = 0;
          for (int base = 0; base < R && carry < best.delta; base += kWarp) {
            const int sr = base + lane;
            int* from = p.q + ((size_t)sr * E + best.expert) * R + src;
            int* to = p.q + ((size_t)sr * E + best.expert) * R + best.target;
            int* cfrom = qcached && sr < R ? s.q_c + ((size_t)sr * E + best.expert) * n + busy_idx : nullptr;
            int* cto = qcached && sr < R ? s.q_c + ((size_t)sr * E + best.expert) * n + sel_idx : nullptr;
            const int have = sr < R ? (cfrom ? *cfrom : *from) : 0;
            int incl = have;
            for (int off = 1; off < kWarp; off <<= 1) {
              int o = __shfl_up_sync(kFull, incl, off);
              if (lane >= off) incl += o;
            }
            const int before = carry + incl - have;
            const int mv = min(have, max(best.delta - before, 0));
            if (sr < R && mv > 0) {
              *from = have - mv;
              if (cfrom) {
                *cfrom = have - mv;
                *to = (*cto += mv);
              } else {
                *to += mv;
              }
            }
            carry += __shfl_sync(kFull, incl, kWarp - 1);
          }
        }
        if (tid == 0) {
          if (cached) {
            const int a = (s.erl_c[best.expert * n + busy_idx] -= best.delta);
            const int b = (s.erl_c[best.expert * n + sel_idx] += best.delta);
            p.erl[(size_t)best.expert * R + src] = a;
            p.erl[(size_t)best.expert * R + best.target] = b;
          } else {
            p.erl[(size_t)best.expert * R + src] -= best.delta;
            p.erl[(size_t)best.expert * R + best.target] += best.delta;
          }
          s.load[busy_idx] -= best.delta;
          s.load[sel_idx] += best.delta;
          for (int i = 0; i < n; ++i) s.stuck[i] = 0;
        }
      }
    } else if (tid == 0) {
      if (best.delta <= 0) {
        s.stuck[busy_idx] = 1;
      } else {
        const int ti = s.local_idx[best.target];
        auto qa = [&](int sr, int dst) { return p.q + ((size_t)sr * E + best.expert) * R + dst; };
        auto dry = [&](int limit) {
          int left = limit, tot = 0;
          for (int sr = 0; sr < R; ++sr) {
            int mv = safe_move(*qa(sr, src), *qa(sr, best.target), left, u_min);
            left -= mv;
            tot += mv;
          }
          return tot;
        };
        int limit = best.delta;
        int actual = dry(limit);
        if (actual < u_min) {
          limit = top - best.load - 1;
          actual = dry(limit);
        }
        if (actual < u_min) {
          s.stuck[busy_idx] = 1;
        } else {
          signed char* cell = p.x + (size_t)best.expert * R + best.target;
          if (*cell == 0) {
            *cell = 1;
            if (cached) s.x_c[best.expert * n + ti] = 1;
            s.slot[ti] += 1;
          }
          int left = limit;
          for (int sr = 0; sr < R; ++sr) {
            int have = *qa(sr, src), there = *qa(sr, best.target);
            int mv = safe_move(have, there, left, u_min);
            *qa(sr, src) = have - mv;
            *qa(sr, best.target) = there + mv;
            left -= mv;
          }
          p.erl[(size_t)best.expert * R + src] -= actual;
          p.erl[(size_t)best.expert * R + best.target] += actual;
          if (cached) {
            s.erl_c[best.expert * n + busy_idx] -= actual;
            s.erl_c[best.expert * n + ti] += actual;
          }
          s.load[busy_idx] -= actual;
          s.load[ti] += actual;
          for (int i = 0; i < n; ++i) s.stuck[i] = 0;
        }
      }
    }
    __syncthreads();
  }

  for (int i = tid; i < n; i += nt) {
    int r = s.dom_ranks[i];
    p.rank_load[r] = s.load[i];
    p.slot_used[r] = s.slot[i];
    p.stuck[r] = (unsigned char)s.stuck[i];
  }
  __syncthreads();
}

__device__ int global_theta(const SolverParams& p) {
  int th = -1;
  for (int r = 0; r < p.R; ++r) th = max(th, p.rank_load[r]);
  return th;
}
// The same maximum, by the first warp of the CTA (all 32 lanes call it); valid on every lane.
__device__ int global_theta_warp(const SolverParams& p) {
  int th = -1;
  for (int r = threadIdx.x & 31; r < p.R; r += kWarp) th = max(th, p.rank_load[r]);
  for (int off = kWarp / 2; off > 0; off >>= 1) th = max(th, __shfl_xor_sync(kFull, th, off));
  return th;
}

// ------------------------------------------------------------------ phase 3
__device__ void build_tables(const SolverParams& p, const RankTables& t, int me) {
  const int R = p.R, E = p.E;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const unsigned lt = (1u << lane) - 1u;
  if (t.send_off != nullptr && me >= 0) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      const int* qrow = p.q + ((size_t)me * E + e) * R;
      int acc = 0;
      for (int d = 0; d < R; ++d) {
        t.send_off[(size_t)e * R + d] = acc;
        acc += qrow[d];
      }
    }
  }
  // With home slots (home_index given) a rank's row blocks are ordered: the experts it owns first, then its
  // replicas, each by ascending id.  The consuming GEMM walks its tiles in row order and the senders deliver in
  // row order, so the owned groups are computed while the replica weights are still on their way.  Without home
  // slots the order is plain ascending id (the reference's physical slot order).
  const int passes = t.home_index != nullptr ? 2 : 1;
  for (int h = warp; h < R; h += nwarps) {
    int groups = 0, replicas = 0, rows = 0;  // running counts / padded row offset on rank h
    for (int pass = 0; pass < passes; ++pass) {
      for (int base = 0; base < E; base += kWarp) {
        const int e = base + lane;
        const bool hosted = e < E && p.x[(size_t)e * R + h] != 0;
        const bool is_main = hosted && p.main_rank[e] == h;
        const bool sel = hosted && (passes == 1 || is_main == (pass == 0));   // handled in this pass
        const int size = sel ? p.erl[(size_t)e * R + h] : 0;
        const int padded = round_up(size, t.row_align);
        const unsigned m = __ballot_sync(kFull, sel);
        const unsigned mr = __ballot_sync(kFull, sel && !is_main);
        const int my_group = groups + __popc(m & lt);
        const int my_rep = replicas + __popc(mr & lt);
        int incl = padded;
        for (int off = 1; off < kWarp; off <<= 1) {
          int o = __shfl_up_sync(kFull, incl, off);
          if (lane >= off) incl += o;
        }
        const int my_off = rows + incl - padded;
        int wslot = my_group;
        if (t.home_index != nullptr) wslot = is_main ? t.home_index[e < E ? e : 0] : t.home_cap + my_rep;
        if (e < E && (sel || (!hosted && pass == 0))) {
          if (t.slot_of) t.slot_of[(size_t)e * R + h] = hosted ? wslot : -1;
          if (t.row_base && me >= 0) {
            int before = 0;
            if (hosted)
              for (int s2 = 0; s2 < me; ++s2) before += p.q[((size_t)s2 * E + e) * R + h];
            t.row_base[(size_t)e * R + h] = hosted ? my_off + before : -1;
          }
          if (hosted && h == me && my_group < t.n_slot) {
            t.group_expert[my_group] = e;
            t.group_wslot[my_group] = wslot;
            t.group_off[my_group] = my_off;
            t.group_rows[my_group] = size;
          }
        }
        groups += __popc(m);
        replicas += __popc(mr);
        rows += __shfl_sync(kFull, incl, kWarp - 1);
      }
    }
    if (t.tiles_of != nullptr && lane == 0) {
      const int used = t.row_capacity > 0 && rows > t.row_capacity ? t.row_capacity : rows;
      t.tiles_of[h] = used / t.row_align;
    }
    if (h == me) {
      for (int g = groups + lane; g < t.n_slot; g += kWarp) {
        t.group_expert[g] = -1;
        t.group_wslot[g] = 0;
        t.group_off[g] = rows;
        t.group_rows[g] = 0;
      }
      if (lane == 0) {
        t.group_off[t.n_slot] = rows;
        t.totals[0] = rows;
        t.totals[1] = groups < t.n_slot ? groups : t.n_slot;
        if (t.row_capacity > 0 && rows > t.row_capacity) set_status(p.status, kStatusRowOverflow, 30, rows);
      }
    }
  }
}

// ------------------------------------------------------------------ kernels
__device__ __forceinline__ void trace_mark(const SolverParams& p, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.trace[slot] = (int64_t)globaltimer_ns();
}

__global__ void __launch_bounds__(1024) solver_kernel(SolverParams p, RankTables tables) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Smem s = carve(smem_raw, p.R, p.E);
  trace_mark(p, 0);

  // Wait (bounded) until every rank's row of omega has landed in the gather buffer.
  if (p.omega_signal != nullptr) {
    __shared__ int sig_ok;
    if (threadIdx.x == 0) {
      sig_ok = wait_ge<true>(p.omega_signal, (*p.omega_epoch) * (unsigned)p.R, kWaitBudgetNs) ? 1 : 0;
      if (!sig_ok) set_status(p.status, kStatusSignalTimeout, 10);
    }
    __syncthreads();
    if (!sig_ok) return;  // every CTA fails the same bounded wait; nobody is left at a barrier
  }

  // Every rank must belong to one of the D domains; a plan solved with an out-of-range id would leave that
  // rank's load unset.  Every CTA evaluates the same input, so all of them return together.
  {
    __shared__ int bad_rank;
    if (threadIdx.x == 0) bad_rank = -1;
    __syncthreads();
    for (int r = threadIdx.x; r < p.R; r += blockDim.x)
      if (p.dom[r] < 0 || p.dom[r] >= p.D) bad_rank = r;
    __syncthreads();
    if (bad_rank >= 0) {
      if (threadIdx.x == 0) set_status(p.status, kStatusBadArgument, 13, bad_rank);
      return;
    }
  }

  bool ok = true;
  trace_mark(p, 1);
  for (int d = blockIdx.x; d < p.D; d += gridDim.x) phase0_domain(p, s, d);
  trace_mark(p, 2);
  ok = ok && grid_barrier(p, 11);
  trace_mark(p, 3);
  // Fast path (every domain has its own CTA, <= 64 ranks, quota cache fits, plain quota floor): each CTA routes
  // exactly its own domain's columns into its caches and goes on repairing them, with no grid barrier between.
  const bool own_columns = p.cache_q && p.u_min == 1 && p.R <= 64 && (int)gridDim.x >= p.D && !p.probe;
  if (ok && !own_columns) {
    if (p.R <= 64) phase1_routing_masks(p, s);
    else phase1_routing(p);
  }
  if (!own_columns) ok = ok && grid_barrier(p, 12);

  if (ok) {
    if (own_columns) {
      if ((int)blockIdx.x < p.D) {
        phase1_domain(p, s, blockIdx.x);
        trace_mark(p, 4);
        stage2_domain(p, s, blockIdx.x, p.iters, ProbeState{false, 0}, true, true);
        trace_mark(p, 5);
      }
    } else if (!p.probe) {
      for (int d = blockIdx.x; d < p.D; d += gridDim.x) stage2_domain(p, s, d, p.iters, ProbeState{false, 0}, true);
    } else {
      // Stagnation probe: 1 repair round, then `patience` rounds, then the remainder unless the
      // global max load stopped improving.  Every CTA evaluates the same control values.
      ProbeState pr{true, p.patience};
      for (int d = blockIdx.x; d < p.D; d += gridDim.x) stage2_domain(p, s, d, 1, pr, true);
      ok = ok && grid_barrier(p, 14);
      long long best = global_theta(p);
      long long stagnant = 0, stop = 0;
      int left = p.iters - 1;
      const int probe_iters = min(p.patience, left);
      if (ok && probe_iters > 0)
        for (int d = blockIdx.x; d < p.D; d += gridDim.x) stage2_domain(p, s, d, probe_iters, pr, false);
      left -= probe_iters;
      ok = ok && grid_barrier(p, 15);
      if (ok && left > 0) {
        long long th = global_theta(p);
        if (th < best) {
          best = th;
          stagnant = 0;
        } else {
          stagnant += probe_iters;
          if (stagnant >= p.patience) stop = 1;
        }
        if (!stop)
          for (int d = blockIdx.x; d < p.D; d += gridDim.x) stage2_domain(p, s, d, left, pr, false);
      }
      if (blockIdx.x == 0 && threadIdx.x == 0 && p.control) {
        p.control[0] = best;
        p.control[1] = stagnant;
        p.control[2] = stop;
      }
    }
  }
  // No barrier before the tail: every CTA publishes its results and counts itself out; the LAST one to leave sees
  // all domains' results, so it computes theta, builds the routing tables and rewinds the barrier counters.
  __shared__ int last_out;
  __syncthreads();
  if (threadIdx.x == 0) {
    last_out = 1;
    if (gridDim.x > 1) {
      __threadfence();
      last_out = atomicAdd(p.sync + 1, 1u) == gridDim.x - 1 ? 1 : 0;
      __threadfence();
    }
  }
  __syncthreads();
  if (!last_out) return;
  if (ok && (gridDim.x == 1 || *reinterpret_cast<volatile int*>(p.status) == 0)) {
    if (threadIdx.x < kWarp) {
      const int th = global_theta_warp(p);
      if (threadIdx.x == 0) p.theta[0] = th;
    }
    if (tables.me >= 0) build_tables(p, tables, tables.me);
  }
  if (threadIdx.x == 0 && gridDim.x > 1) {
    p.sync[0] = 0;
    p.sync[1] = 0;
    __threadfence();
  }
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[6] = (int64_t)globaltimer_ns();
}

__global__ void __launch_bounds__(1024) tables_kernel(SolverParams p, RankTables tables) {
  build_tables(p, tables, tables.me);
}

size_t solver_base_smem(int R, int E) {
  const size_t P = (size_t)(pow2_at_least(E) < 32 ? 32 : pow2_at_least(E));
  return sizeof(long long) * P + sizeof(int) * P + sizeof(int) * 5 * R + sizeof(Cand) * 32 + 64;
}
size_t solver_cache_smem(int R, int E) { return (((size_t)E * R * 5 + 15) / 16) * 16; }  // erl (int) + x (byte) per (e, rank)
size_t solver_qcache_smem(int R, int E) { return (size_t)R * E * R * 4; }
constexpr size_t kCacheBudget = 200 * 1024;

int pow2_threads(int R, int E) {
  int want = E > R ? E : R;
  int t = 256;
  while (t < want && t < 1024) t <<= 1;
  return t;
}

}  // namespace

cudaError_t launch_solver(const SolverParams& p, const RankTables& tables, cudaStream_t stream) {
  int dev = 0, sms = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (err != cudaSuccess) return err;
  SolverParams pc = p;
  const size_t base = solver_base_smem(p.R, p.E);
  pc.cache_stage2 = base + solver_cache_smem(p.R, p.E) <= kCacheBudget ? 1 : 0;
  pc.cache_q = pc.cache_stage2 && base + solver_cache_smem(p.R, p.E) + solver_qcache_smem(p.R, p.E) <= kCacheBudget ? 1 : 0;
  const size_t smem = base + (pc.cache_stage2 ? solver_cache_smem(p.R, p.E) : 0) + (pc.cache_q ? solver_qcache_smem(p.R, p.E) : 0);
  // The dynamic shared-memory limit is an attribute of (kernel, device): raise it per device, only when needed.
  constexpr int kMaxDevices = 64;
  static size_t configured_smem[kMaxDevices] = {};
  const bool tracked = dev >= 0 && dev < kMaxDevices;
  const size_t have = tracked && configured_smem[dev] ? configured_smem[dev] : 48 * 1024;
  if (smem > have || (!tracked && smem > 48 * 1024)) {
    err = cudaFuncSetAttribute(solver_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    if (tracked) configured_smem[dev] = smem;
  }
  int grid = p.D < sms ? p.D : sms;
  if (grid < 1) grid = 1;
  const int threads = pow2_threads(p.R, p.E);
  RankTables tc = tables;
  void* args[] = {&pc, &tc};
  if (grid > 1) return cudaLaunchCooperativeKernel((void*)solver_kernel, dim3(grid), dim3(threads), args, smem, stream);
  solver_kernel<<<1, threads, smem, stream>>>(pc, tc);
  return cudaGetLastError();
}

cudaError_t launch_tables(const SolverParams& p, const RankTables& tables, cudaStream_t stream) {
  int threads = 32 * (p.R < 32 ? p.R : 32);
  if (threads < 32) threads = 32;
  tables_kernel<<<1, threads, 0, stream>>>(p, tables);
  return cudaGetLastError();
}

}  // namespace epb
