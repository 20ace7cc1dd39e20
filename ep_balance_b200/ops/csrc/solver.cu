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
// The best candidate of the warp under better(), on EVERY lane.  The order is lexicographic, so five warp-wide
// integer reductions (one instruction each), each over the lanes still tied on the earlier fields, replace a
// 5-step butterfly of 5-word shuffles: the repair loop's critical path is made of these.
__device__ __forceinline__ Cand warp_best(Cand v) {
  const int d = __reduce_max_sync(kFull, v.delta);
  bool in = v.delta == d;
  const int l = __reduce_min_sync(kFull, in ? v.load : INT_MAX);
  in = in && v.load == l;
  const int c = __reduce_min_sync(kFull, in ? v.cost : INT_MAX);
  in = in && v.cost == c;
  const int e = __reduce_min_sync(kFull, in ? v.expert : INT_MAX);
  in = in && v.expert == e;
  const int t = __reduce_min_sync(kFull, in ? v.target : INT_MAX);
  return Cand{d, l, c, e, t};
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
  int* cost_c;      // [64] link costs between the domain's ranks (domains of at most 8 ranks)
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
  s.cost_c = reinterpret_cast<int*>(base);
  base += sizeof(int) * 64;
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
// Returns the number of ranks in domain d (s.dom_ranks / s.local_idx describe it on return).
__device__ int phase0_domain(const SolverParams& p, Smem& s, int d) {
  __shared__ int n_valid;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int R = p.R, E = p.E;
  const int n = collect_domain(p, s, d);
  if (n == 0) return 0;
  // With the cache region available the domain's placement columns live in shared memory while
  // candidates are admitted (one global round trip per candidate otherwise) and are stored once.
  signed char* xc = p.cache_stage2 ? s.x_c : nullptr;
  // link costs inside the domain, for the repair loop of a CTA that keeps this domain (their latency hides here)
  if (n <= 8)
    for (int idx = tid; idx < n * n; idx += nt) s.cost_c[idx] = __ldg(p.cost + (size_t)s.dom_ranks[idx / n] * R + s.dom_ranks[idx % n]);
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
  // gate and benefit (the owner's domain comes from the index collect_domain() left in shared memory, so the
  // loop has no load that depends on another load); valid candidates are also listed compactly in s.order
  // (with one domain, or with cross-domain replicas switched off, nothing can qualify: the loop is skipped)
  for (int e = tid; e < E && p.allow_cross && p.D > 1; e += nt) {
    long long T = 0;
    const int owner = __ldg(p.main_rank + e);
    const long long wb = __ldg(p.weight_bytes + e);
    for (int i = 0; i < n; ++i) T += __ldg(p.omega + (size_t)s.dom_ranks[i] * E + e);
    long long rhs = 2 * T * p.s_tok;
    bool valid = p.allow_cross && s.local_idx[owner] < 0 && T > 0 && wb < rhs;
    s.prio[e] = valid ? rhs - wb : -1;
    if (valid) {
      const int at = atomicAdd(&n_valid, 1);
      if (at < kWarp) s.order[at] = e;  // only used when at most 32 candidates exist
    }
  }
  __syncthreads();
  const int nv = n_valid;
  if (nv > 0 && nv <= kWarp) {
    // Few candidates (the usual case: only experts whose traffic outweighs their weights qualify): one warp
    // ranks them by counting, which gives the same order as sorting the whole row -- descending benefit, ties by
    // ascending expert id; the pairs are distinct, so every rank is taken exactly once.
    if (tid < kWarp) {
      const int lane = tid;
      const int me = lane < nv ? s.order[lane] : -1;
      const long long mp = lane < nv ? s.prio[me] : -1;
      int rank = 0;
      for (int j = 0; j < nv; ++j) {
        const int oe = __shfl_sync(kFull, me, j);
        const long long op = __shfl_sync(kFull, mp, j);
        if (op > mp || (op == mp && oe < me)) ++rank;
      }
      __syncwarp(kFull);
      if (lane < nv) s.order[rank] = me;
      __syncwarp(kFull);
    }
  } else if (nv > 0) {
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
  }
  if (nv > 0) {
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
  return n;
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
// into the shared-memory caches that the repair loop works on, and stores the non-zero ones to global memory
// (the grid cleared q before the barrier that precedes this phase).  The repair loop then needs neither a grid
// barrier after routing nor a cache fill.  Requires R <= 64, u_min == 1 and the quota cache of this domain to fit.
// MaskT: host sets as 32-bit words when R <= 32 (half the instructions of the 64-bit form; this phase runs on one
// SM per domain and is bound by instruction issue, not by memory).
template <typename MaskT>
__device__ __forceinline__ int popc_mask(MaskT m) {
  return sizeof(MaskT) == 8 ? __popcll((unsigned long long)m) : __popc((unsigned)m);
}
template <typename MaskT>
__device__ __forceinline__ int lowest_bit(MaskT m) {
  return sizeof(MaskT) == 8 ? __ffsll((long long)m) - 1 : __ffs((int)m) - 1;
}
// Thread (e, g): expert e, sources g, g + groups, ...  Only the hosts of e inside this domain get a quota, so the
// loop walks the set bits of (active hosts & this domain) -- zero or one bit for most pairs -- instead of testing
// every rank of the domain.  The caches were cleared beforehand; erl[e, rank] is accumulated on the way.
template <typename MaskT>
__device__ void phase1_domain_impl(const SolverParams& p, Smem& s, int n, const unsigned long long* dom_mask, MaskT mine) {
  const int R = p.R, E = p.E;
  const int tid = threadIdx.x, nt = blockDim.x;
  const unsigned long long* host = reinterpret_cast<const unsigned long long*>(s.prio);  // [E]
  const int groups = nt / E > 0 ? (nt / E < R ? nt / E : R) : 1;
  for (int idx = tid; idx < E * groups; idx += nt) {
    const int g = idx / E, e = idx - g * E;
    const MaskT h = (MaskT)host[e];
    for (int src0 = g; src0 < R; src0 += 8 * groups) {
      int need_b[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {  // the loads of up to eight sources are in flight together
        const int src = src0 + j * groups;
        need_b[j] = src < R ? __ldg(p.omega + (size_t)src * E + e) : 0;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int src = src0 + j * groups;
        if (src >= R) break;
        const int need = need_b[j];
        if (need <= 0) continue;
        const MaskT loc = h & (MaskT)dom_mask[src];
        const MaskT act = loc ? loc : h;
        MaskT todo = act & mine;
        if (!todo) continue;
        const int count = popc_mask<MaskT>(act);
        // even split over the active hosts (u_min == 1): need / count each, the first need % count get one more
        const int base = count == 1 ? need : need / count;
        const int extra = need - base * count;
        const size_t pair = (size_t)src * E + e;
        while (todo) {
          const int dst = lowest_bit<MaskT>(todo);
          todo &= todo - (MaskT)1;
          const int pos = popc_mask<MaskT>(act & (((MaskT)1 << dst) - (MaskT)1));
          const int v = base + (pos < extra ? 1 : 0);
          if (v != 0) {
            const int li = s.local_idx[dst];
            p.q[pair * R + dst] = v;
            s.q_c[pair * n + li] = v;
            atomicAdd(&s.erl_c[e * n + li], v);
          }
        }
      }
    }
  }
}

// n_known: the size of domain d when s.dom_ranks / s.local_idx still describe it (left by phase 0), else -1.
__device__ void phase1_domain(const SolverParams& p, Smem& s, int d, int n_known) {
  __shared__ unsigned long long dom_mask[64];
  const int R = p.R, E = p.E;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int n = n_known >= 0 ? n_known : collect_domain(p, s, d);
  if (n == 0) return;
  unsigned long long* host = reinterpret_cast<unsigned long long*>(s.prio);  // [E]
  if ((R & 7) == 0) {
    // a row of x is R bytes, 8-byte aligned: eight hosts per load
    for (int e = tid; e < E; e += nt) {
      unsigned long long m = 0;
      const unsigned long long* row = reinterpret_cast<const unsigned long long*>(p.x + (size_t)e * R);
      for (int w = 0; w < R / 8; ++w) {
        const unsigned long long v = row[w];
#pragma unroll
        for (int b = 0; b < 8; ++b) m |= (unsigned long long)(((v >> (8 * b)) & 0xffull) != 0) << (8 * w + b);
      }
      host[e] = m;
    }
  } else {
    for (int e = tid; e < E; e += nt) {
      unsigned long long m = 0;
      for (int dst = 0; dst < R; ++dst) m |= (unsigned long long)(p.x[(size_t)e * R + dst] != 0) << dst;
      host[e] = m;
    }
  }
  for (int r = tid; r < R; r += nt) {
    unsigned long long m = 0;
    const int dr = p.dom[r];
    for (int o = 0; o < R; ++o) m |= (unsigned long long)(p.dom[o] == dr) << o;
    dom_mask[r] = m;
  }
  // clear the caches while those loads are in flight (q_c and erl_c are contiguous ints; x_c is written below)
  {
    const int q_ints = R * E * n, e_ints = E * n;
    for (int i = tid; i < e_ints; i += nt) s.erl_c[i] = 0;
    if ((reinterpret_cast<uintptr_t>(s.q_c) & 15) == 0 && (q_ints & 3) == 0) {
      uint4* qv = reinterpret_cast<uint4*>(s.q_c);
      for (int i = tid; i < q_ints / 4; i += nt) qv[i] = make_uint4(0, 0, 0, 0);
    } else {
      for (int i = tid; i < q_ints; i += nt) s.q_c[i] = 0;
    }
  }
  __syncthreads();
  const unsigned long long mine = dom_mask[s.dom_ranks[0]];  // the ranks of this domain
  if (R <= 32) phase1_domain_impl<unsigned>(p, s, n, dom_mask, (unsigned)mine);
  else phase1_domain_impl<unsigned long long>(p, s, n, dom_mask, mine);
  __syncthreads();
  for (int cell = tid; cell < E * n; cell += nt) {
    const int e = cell / n, i = cell - e * n;
    p.erl[(size_t)e * R + s.dom_ranks[i]] = s.erl_c[cell];
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
                              bool prefilled = false, int n_known = -1) {
  __shared__ int busy_idx, busy_rank, busy_load, finished;
  __shared__ int best_theta, stagnant;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
  const int R = p.R, E = p.E, u_min = p.u_min;
  const int n = n_known >= 0 ? n_known : collect_domain(p, s, d);
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
  // link costs between the domain's ranks (small domains): the scan below reads one per candidate
  int* cost_c = s.cost_c;
  const bool cost_cached = n <= 8;
  if (cost_cached && n_known < 0)  // (a CTA that kept its domain since phase 0 has them already)
    for (int idx = tid; idx < n * n; idx += nt) cost_c[idx] = p.cost[(size_t)s.dom_ranks[idx / n] * R + s.dom_ranks[idx % n]];
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

  // One iteration = two block barriers.  All threads scan the candidates of the busiest rank; then warp 0 alone
  // picks the best one, applies it (placement, quota move, loads) and selects the busiest rank of the NEXT
  // iteration, while the other warps wait at the second barrier.
  // Busiest rank that is not stuck (first one on ties) and the domain's max load, by all lanes of warp 0.
  auto select_busy = [&](int it) {
    int theta = -1, bl = -1, bi = INT_MAX;
    for (int base = 0; base < n; base += kWarp) {
      const int i = base + lane;
      const int l = i < n ? s.load[i] : -1;
      const int cl = (i < n && s.stuck[i] == 0) ? l : -1;
      theta = max(theta, l);
      if (cl > bl) {  // a lane sees its ranks in ascending order: the first maximum stays
        bl = cl;
        bi = i;
      }
    }
    theta = __reduce_max_sync(kFull, theta);
    const int top = __reduce_max_sync(kFull, bl);
    bi = __reduce_min_sync(kFull, (bl == top && top >= 0) ? bi : INT_MAX);
    if (lane == 0) {
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
      const bool none = bi == INT_MAX;
      busy_idx = none ? -1 : bi;
      busy_rank = none ? -1 : s.dom_ranks[bi];
      busy_load = none ? -1 : top;
      finished = stop || none || top <= 0;
    }
  };
  if (warp == 0) {
    if (lane == 0) finished = 1;
    __syncwarp(kFull);
    if (iters > 0) select_busy(0);
  }
  __syncthreads();
  // Candidates are (expert, target) pairs; tpe threads share an expert's targets so that a domain with few experts
  // still spreads the scan over the whole block.  The mapping does not change between iterations.
  const int tpe = nt / E > 1 ? (nt / E < n ? nt / E : n) : 1;
  const int my_e = tid / tpe, my_sub = tid - my_e * tpe, e_step = nt / tpe;
  int it = 0;
  for (; it < iters; ++it) {
    if (finished) break;
    const int src = busy_rank, top = busy_load, bidx = busy_idx;

    Cand mine = no_cand();
    for (int e = my_e; e < E; e += e_step) {
      const int avail = cached ? s.erl_c[e * n + bidx] : p.erl[(size_t)e * R + src];
      if (avail <= 0) continue;
      for (int ti = my_sub; ti < n; ti += tpe) {
        const int tl = s.load[ti];
        if (ti == bidx || tl >= top) continue;
        const int t = s.dom_ranks[ti];
        const bool host = cached ? s.x_c[e * n + ti] != 0 : p.x[(size_t)e * R + t] != 0;
        if (!host && s.slot[ti] >= p.n_slot) continue;
        const int delta = min(avail, (top - tl) / 2);
        if (delta < u_min) continue;
        Cand c{delta, tl, cost_cached ? cost_c[bidx * n + ti] : p.cost[(size_t)src * R + t], e, t};
        if (better(c, mine)) mine = c;
      }
    }
    mine = warp_best(mine);
    if (lane == 0) s.wcand[warp] = mine;
    __syncthreads();
    if (warp == 0) {
      Cand best = lane < nwarps ? s.wcand[lane] : no_cand();
      best = warp_best(best);  // the same on every lane: they all take the same branches below
      if (u_min == 1) {
        const int sel = best.delta > 0 ? s.local_idx[best.target] : -1;
        const bool apply = best.delta > 0 && sel >= 0;
        if (!apply) {
          if (lane == 0) s.stuck[bidx] = 1;
        } else {
          if (lane == 0) {
            signed char* cell = p.x + (size_t)best.expert * R + best.target;
            const bool hosted = cached ? s.x_c[best.expert * n + sel] != 0 : *cell != 0;
            if (!hosted) {
              *cell = 1;
              if (cached) s.x_c[best.expert * n + sel] = 1;
              s.slot[sel] += 1;
            }
          }
          // prefix over source ranks: source s gives min(q_s, max(delta - sum_{s'<s} q_s', 0))
          int carry = 0;
          for (int base = 0; base < R && carry < best.delta; base += kWarp) {
            const int sr = base + lane;
            int* from = p.q + ((size_t)sr * E + best.expert) * R + src;
            int* to = p.q + ((size_t)sr * E + best.expert) * R + best.target;
            int* cfrom = qcached && sr < R ? s.q_c + ((size_t)sr * E + best.expert) * n + bidx : nullptr;
            int* cto = qcached && sr < R ? s.q_c + ((size_t)sr * E + best.expert) * n + sel : nullptr;
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
          if (lane == 0) {
            if (cached) {
              const int a = (s.erl_c[best.expert * n + bidx] -= best.delta);
              const int b = (s.erl_c[best.expert * n + sel] += best.delta);
              p.erl[(size_t)best.expert * R + src] = a;
              p.erl[(size_t)best.expert * R + best.target] = b;
            } else {
              p.erl[(size_t)best.expert * R + src] -= best.delta;
              p.erl[(size_t)best.expert * R + best.target] += best.delta;
            }
            s.load[bidx] -= best.delta;
            s.load[sel] += best.delta;
            for (int i = 0; i < n; ++i) s.stuck[i] = 0;
          }
        }
      } else if (lane == 0) {
        if (best.delta <= 0) {
          s.stuck[bidx] = 1;
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
            s.stuck[bidx] = 1;
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
              s.erl_c[best.expert * n + bidx] -= actual;
              s.erl_c[best.expert * n + ti] += actual;
            }
            s.load[bidx] -= actual;
            s.load[ti] += actual;
            for (int i = 0; i < n; ++i) s.stuck[i] = 0;
          }
        }
      }
      __syncwarp(kFull);
      if (it + 1 < iters) select_busy(it + 1);
      else if (lane == 0) finished = 1;
    }
    __syncthreads();
  }
  if (p.trace != nullptr && blockIdx.x == 0 && tid == 0) p.trace[7] = it;  // repair iterations of the first domain

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
  // Fast path (every domain has its own CTA, <= 64 ranks, quota cache fits, plain quota floor): each CTA routes
  // exactly its own domain's columns into its caches and goes on repairing them, with no grid barrier between.
  const bool own_columns = p.cache_q && p.u_min == 1 && p.R <= 64 && (int)gridDim.x >= p.D && !p.probe;
  // With several CTAs on the fast path each one folds its domain's max load into theta with an atomic max (no CTA
  // has to wait for the others' loads at the end); the start value is written ahead of the barrier below.
  const bool theta_by_atomics = own_columns && gridDim.x > 1;
  if (theta_by_atomics && blockIdx.x == 0 && threadIdx.x == 0) p.theta[0] = -1;
  if (own_columns) {
    // Most quotas are zero (an expert has a handful of hosts).  The grid clears q here with full-width stores, ahead
    // of the barrier that phase 1 waits on anyway, and phase 1 then stores only the non-zero quotas: a few
    // thousand scattered 4-byte stores per CTA instead of R * E * n of them, which was what phase 1 spent its time on.
    const size_t total = (size_t)p.R * p.E * p.R;
    const size_t vecs = (reinterpret_cast<uintptr_t>(p.q) & 15) == 0 ? total / 4 : 0;  // unaligned caller buffer: scalar stores
    uint4* qv = reinterpret_cast<uint4*>(p.q);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (size_t)gridDim.x * blockDim.x)
      qv[i] = make_uint4(0, 0, 0, 0);
    for (size_t i = vecs * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
      p.q[i] = 0;
  }
  int n_mine = -1;  // fast path: the size of this CTA's own domain, collected once
  for (int d = blockIdx.x; d < p.D; d += gridDim.x) n_mine = phase0_domain(p, s, d);
  if (!own_columns) n_mine = -1;
  trace_mark(p, 2);
  ok = ok && grid_barrier(p, 11);
  trace_mark(p, 3);
  if (ok && !own_columns) {
    if (p.R <= 64) phase1_routing_masks(p, s);
    else phase1_routing(p);
  }
  if (!own_columns) ok = ok && grid_barrier(p, 12);

  if (ok) {
    if (own_columns) {
      if ((int)blockIdx.x < p.D) {
        phase1_domain(p, s, blockIdx.x, n_mine);
        trace_mark(p, 4);
        stage2_domain(p, s, blockIdx.x, p.iters, ProbeState{false, 0}, true, true, n_mine);
        if (theta_by_atomics && threadIdx.x == 0) {
          int top = -1;
          for (int i = 0; i < n_mine; ++i) top = max(top, s.load[i]);
          atomicMax(reinterpret_cast<long long*>(p.theta), (long long)top);
        }
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
    if (!theta_by_atomics && threadIdx.x < kWarp) {
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
  return sizeof(long long) * P + sizeof(int) * P + sizeof(int) * 5 * R + sizeof(Cand) * 32 + sizeof(int) * 64 + 64;
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
