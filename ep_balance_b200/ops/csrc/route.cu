// Token-path and weight-path kernels: count + publish, route assignment, the stand-alone form of the
// item-driven transport (comm.cuh), unit reduce, cross-rank barrier, replica weight pull and owner-side
// gradient return.
//
// Replaces the reference's torch-op chains and NCCL calls on the MoE path:
//   bincount + all_gather (eplb/distributed.py:17-61)            -> count_publish_kernel
//   assign_physical + argsort/index_select (physical.py:30-77,
//       eplb_manager.py:1067-1105)                                -> route_assign + comm (comm.cuh)
//   index_add scatter with gate weight (eplb_manager.py:889-899)  -> unit_reduce_kernel
//   dist.broadcast per expert / GIN get (overlap.py:113-148,
//       gin_weights.py:305-341)                                   -> weight_pull_kernel
//   dist.reduce per expert / GIN put + sum (overlap.py:203-232,
//       gin_weights.py:343-377)                                   -> grad_reduce_kernel
// All remote traffic is plain peer loads/stores through NVSwitch; no cluster-multicast loads.
#include "route.h"

#include <cuda_bf16.h>

#include "comm.cuh"
#include "common.cuh"

namespace epb {
namespace {

constexpr unsigned kFull = 0xffffffffu;

// SM count of the current device (the runtime caches device attributes; this is a cheap host call).
int sm_count() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      sms <= 0)
    return 132;
  return sms;
}

// ------------------------------------------------------------------ count + publish
// One CTA per chunk of kRouteChunk units.  Each CTA keeps its chunk's histogram for the route
// assignment and adds it to the running histogram; the last CTA to finish publishes.
__global__ void __launch_bounds__(kRouteChunk) count_publish_kernel(CountArgs a) {
  extern __shared__ int hist[];  // [E]
  __shared__ int is_last;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int E = a.E, R = a.R;
  for (int e = tid; e < E; e += nt) hist[e] = 0;
  __syncthreads();
  const int u = blockIdx.x * kRouteChunk + tid;
  if (u < a.num_units) {
    const int e = (int)a.unit_expert[u];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = tid; e < E; e += nt) {
    const int c = hist[e];
    a.chunk_hist[(size_t)blockIdx.x * E + e] = c;
    if (c) atomicAdd(&a.hist_acc[e], c);
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = atomicAdd(&a.hist_acc[E], 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // ---- last CTA: take (and clear) the full histogram, publish it, clear the arrival counters
  for (int e = tid; e < E; e += nt) hist[e] = atomicExch(&a.hist_acc[e], 0);
  if (tid == 0) a.hist_acc[E] = 0;
  __syncthreads();
  if (tid < 32) {  // exclusive prefix over experts by one warp
    int run = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + tid;
      const int c = e < E ? hist[e] : 0;
      int incl = c;
      for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(kFull, incl, off);
        if (tid >= off) incl += o;
      }
      if (e < E) a.exp_prefix[e] = run + incl - c;
      run += __shfl_sync(kFull, incl, 31);
    }
    if (tid == 0) a.exp_prefix[E] = run;
  }
  for (int idx = tid; idx < E * R; idx += nt) {
    const int peer = idx / E, e = idx - peer * E;
    a.omega_ptrs[peer][(size_t)a.me * E + e] = hist[e];
  }
  for (int i = tid; i < a.clear_words; i += nt) a.clear[i] = 0u;
  if (tid == 0 && a.epoch_word != nullptr) *a.epoch_word += 1u;
  __threadfence_system();
  __syncthreads();
  if (a.signal_ptrs != nullptr)
    for (int r = tid; r < R; r += nt) red_release_sys_add(a.signal_ptrs[r], 1u);
}

// ------------------------------------------------------------------ route assignment
// One CTA per chunk.  A unit's rank within its expert (original order) = units of that expert in
// earlier chunks + in earlier warps of this chunk + in earlier lanes of its warp; the j-th unit goes
// to the host whose quota prefix covers j.
__global__ void __launch_bounds__(kRouteChunk) route_assign_kernel(RouteArgs a) {
  extern __shared__ int sm[];
  constexpr int kWarps = kRouteChunk / 32;
  const int E = a.E, R = a.R;
  int* before = sm;             // [E] units of each expert in earlier chunks
  int* warp_cnt = sm + E;       // [kWarps, E]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nt = blockDim.x;
  for (int i = tid; i < E * (1 + kWarps); i += nt) sm[i] = 0;
  __syncthreads();
  // earlier chunks: the threads split (expert, chunk residue) pairs
  {
    const int parts = nt / E > 0 ? nt / E : 1;
    for (int idx = tid; idx < E * parts; idx += nt) {
      const int e = idx % E, part = idx / E;
      int acc = 0;
      for (int c = part; c < (int)blockIdx.x; c += parts) acc += a.chunk_hist[(size_t)c * E + e];
      if (acc) atomicAdd(&before[e], acc);
    }
  }
  const int u = blockIdx.x * kRouteChunk + tid;
  int e = u < a.num_units ? (int)a.unit_expert[u] : -1;
  if (e >= E) e = -1;
  const unsigned peers = __match_any_sync(kFull, e);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank_in_warp == 0) warp_cnt[warp * E + e] = __popc(peers);
  __syncthreads();
  if (e < 0) {
    if (u < a.num_units) {
      a.unit_dst[u] = -1;
      a.unit_row[u] = -1;
      if (a.unit_pos != nullptr) a.unit_pos[u] = -1;
    }
    return;
  }
  int j = before[e] + rank_in_warp;
  for (int w = 0; w < warp; ++w) j += warp_cnt[w * E + e];
  const int32_t* qrow = a.q_me + (size_t)e * R;
  int dst = 0, pre = 0, have = qrow[0];
  while (dst + 1 < R && j >= pre + have) {
    pre += have;
    ++dst;
    have = qrow[dst];
  }
  const bool placed = j < pre + have;
  if (!placed) {
    set_status(a.status, kStatusBadArgument, 40, e);
    a.unit_dst[u] = -1;
    a.unit_row[u] = -1;
  } else {
    a.unit_dst[u] = dst;
    a.unit_row[u] = a.row_base[(size_t)e * R + dst] + (j - pre);
  }
  if (a.sorted_units != nullptr) a.sorted_units[a.exp_prefix[e] + j] = u;
  if (a.unit_pos != nullptr) a.unit_pos[u] = placed ? a.exp_prefix[e] + j : -1;
}

// ------------------------------------------------------------------ stand-alone transport
constexpr int kCommKernelWarps = 8;
constexpr int kCommKernelSlots = 4;   // 8 warps x 2 loads of 4 KB in flight per SM
constexpr int kCommKernelSmem = kCommKernelWarps * comm_warp_bytes<kCommKernelSlots>() + 128;

__global__ void __launch_bounds__(kCommKernelWarps * 32) comm_kernel(const __grid_constant__ CommArgs a, int* status) {
  extern __shared__ uint8_t comm_smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(comm_smem_raw) + 127) & ~(uintptr_t)127);
  const int warp = threadIdx.x >> 5;
  comm_run<kCommKernelSlots>(a, (int)blockIdx.x * kCommKernelWarps + warp, (int)gridDim.x * kCommKernelWarps,
                             base + warp * comm_warp_bytes<kCommKernelSlots>(), status);
}

// ------------------------------------------------------------------ unit reduce
__global__ void __launch_bounds__(256) unit_reduce_kernel(const uint4* __restrict__ unit_rows,
                                                         const int32_t* __restrict__ unit_pos,
                                                         const float* __restrict__ unit_scale,
                                                         uint4* __restrict__ out, int num_tokens, int topk,
                                                         int vec_per_row, UnitReduceWait wait,
                                                         const float* __restrict__ copy_src, float* __restrict__ copy_dst) {
  if (wait.signal != nullptr) {
    // rows come from the peers' GEMM epilogues: wait until every rank has signalled completion
    if (threadIdx.x == 0 && !wait_ge<true>(wait.signal, *wait.epoch * (unsigned)wait.R, wait.budget_ns))
      set_status(wait.status, kStatusSignalTimeout, 51);
    __syncthreads();
  }
  if (copy_dst != nullptr) {
    const size_t n = (size_t)num_tokens * topk;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
      const int pos = unit_pos != nullptr ? unit_pos[i] : (int)i;
      copy_dst[i] = pos >= 0 ? copy_src[pos] : 0.f;
    }
  }
  // one warp per (token, 32-vector chunk of the row): small batches still fill the machine
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const int chunks = (vec_per_row + 31) / 32;
  const long long item = (long long)blockIdx.x * wpb + warp;
  const int t = (int)(item / chunks);
  if (t >= num_tokens) return;
  const int v = (int)(item - (long long)t * chunks) * 32 + lane;
  if (v >= vec_per_row) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 8
  for (int k = 0; k < topk; ++k) {
    const size_t u = (size_t)t * topk + k;
    const long long pos = unit_pos != nullptr ? (long long)unit_pos[u] : (long long)u;
    if (pos < 0) continue;
    const uint4 val = unit_rows[(size_t)pos * vec_per_row + v];
    const float s = unit_scale ? unit_scale[u] : 1.f;
    const __nv_bfloat162* pv = reinterpret_cast<const __nv_bfloat162*>(&val);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(pv[i]);
      acc[2 * i] += s * f.x;
      acc[2 * i + 1] += s * f.y;
    }
  }
  uint4 o;
  __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  out[(size_t)t * vec_per_row + v] = o;
}

// ------------------------------------------------------------------ cross-rank barrier
__global__ void symm_barrier_kernel(unsigned* const* signal_ptrs, int slot, int R, int me, unsigned* epoch_word,
                                    int* status) {
  __shared__ unsigned target;
  if (threadIdx.x == 0) {
    unsigned epoch = *epoch_word;
    target = (epoch + 1u) * (unsigned)R;
    *epoch_word = epoch + 1u;
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < R) red_release_sys_add(signal_ptrs[threadIdx.x] + slot, 1u);
  if (threadIdx.x == 0) {
    if (!wait_ge<true>(signal_ptrs[me] + slot, target, kWaitBudgetNs)) set_status(status, kStatusBarrierTimeout, 50, slot);
  }
  __syncthreads();
  __threadfence_system();
}

// ------------------------------------------------------------------ weight pull / grad return
__global__ void __launch_bounds__(512) weight_pull_kernel(WeightPullArgs a) {
  // blockIdx.y = local replica slot ordinal; find the expert that the plan put there
  const int wslot = a.home_cap + blockIdx.y;
  if (wslot >= a.n_slot) return;
  __shared__ int expert;
  if (threadIdx.x == 0) expert = -1;
  __syncthreads();
  for (int e = threadIdx.x; e < a.E; e += blockDim.x)
    if (a.slot_of[(size_t)e * a.R + a.me] == wslot && a.main_rank[e] != a.me) expert = e;
  __syncthreads();
  const int e = expert;
  if (e < 0) return;
  const int owner = a.main_rank[e];
  const size_t n_vec = a.elems_per_slot / 8;
  const uint4* src = reinterpret_cast<const uint4*>(a.w_ptrs[owner]) + (size_t)a.home_index[e] * n_vec;
  uint4* dst = reinterpret_cast<uint4*>(a.w_ptrs[a.me]) + (size_t)wslot * n_vec;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  // four independent 16-byte peer loads in flight per thread
  for (; i + 3 * stride < n_vec; i += 4 * stride) {
    uint4 v0 = src[i], v1 = src[i + stride], v2 = src[i + 2 * stride], v3 = src[i + 3 * stride];
    dst[i] = v0;
    dst[i + stride] = v1;
    dst[i + 2 * stride] = v2;
    dst[i + 3 * stride] = v3;
  }
  for (; i < n_vec; i += stride) dst[i] = src[i];
}

constexpr int kMaxGradHosts = 64;  // replica hosts of one expert a gradient-return CTA can list (ranks R <= 64)

__device__ __forceinline__ void add8(float* acc, const uint4& v) {
  const __nv_bfloat162* pv = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(pv[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

__global__ void __launch_bounds__(512) grad_reduce_kernel(GradReduceArgs a) {
  // blockIdx.y = home slot; find the expert living there and its replica hosts
  const int home = blockIdx.y;
  __shared__ int expert;
  __shared__ int n_hosts;
  __shared__ int host_rank[kMaxGradHosts];
  __shared__ int host_slot[kMaxGradHosts];
  if (threadIdx.x == 0) {
    expert = -1;
    n_hosts = 0;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < a.E; e += blockDim.x)
    if (a.main_rank[e] == a.me && a.home_index[e] == home) expert = e;
  __syncthreads();
  const int e = expert;
  if (e < 0) return;
  if (threadIdx.x == 0) {
    int n = 0;
    for (int h = 0; h < a.R && n < kMaxGradHosts; ++h) {
      int s = a.slot_of[(size_t)e * a.R + h];
      if ((h != a.me || a.include_self) && s >= 0) {
        host_rank[n] = h;
        host_slot[n] = s;
        ++n;
      }
    }
    n_hosts = n;
  }
  __syncthreads();
  const int n = n_hosts;
  const bool accumulate = a.accum != nullptr;
  if (n == 0 && !accumulate) return;  // no replicas: the owner's own slot gradient is already final
  const size_t n_vec = a.elems_per_slot / 8;
  uint4* mine = reinterpret_cast<uint4*>(a.g_ptrs[a.me]) + (size_t)home * n_vec;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  // Four vectors per thread and pass, with the peer loads of all four issued before the first is consumed: an
  // expert with one or two replicas is served by this home slot's CTAs only, and what bounds them is the number of
  // bytes they keep in flight across NVLink, not the link.
  constexpr int kUnroll = 4;
  for (size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < n_vec; i0 += stride * kUnroll) {
    float acc[kUnroll][8];
    uint4 own[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const size_t i = i0 + (size_t)j * stride;
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[j][c] = 0.f;
      own[j] = (!a.include_self && i < n_vec) ? mine[i] : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < kUnroll; ++j)
      if (!a.include_self) add8(acc[j], own[j]);  // the owner's own gradient first, then the hosts in rank order
    for (int k = 0; k < n; ++k) {
      const uint4* peer = reinterpret_cast<const uint4*>(a.g_ptrs[host_rank[k]]) + (size_t)host_slot[k] * n_vec;
      uint4 v[kUnroll];
#pragma unroll
      for (int j = 0; j < kUnroll; ++j) {
        const size_t i = i0 + (size_t)j * stride;
        v[j] = i < n_vec ? peer[i] : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < kUnroll; ++j) add8(acc[j], v[j]);
    }
#pragma unroll
    for (int j = 0; j < kUnroll; ++j) {
      const size_t i = i0 + (size_t)j * stride;
      if (i >= n_vec) break;
      if (accumulate && a.accum_fp32) {
        float4* dst = reinterpret_cast<float4*>(a.accum) + ((size_t)home * n_vec + i) * 2;
        float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
        if (!a.overwrite) {
          lo = dst[0];
          hi = dst[1];
        }
        lo.x += acc[j][0]; lo.y += acc[j][1]; lo.z += acc[j][2]; lo.w += acc[j][3];
        hi.x += acc[j][4]; hi.y += acc[j][5]; hi.z += acc[j][6]; hi.w += acc[j][7];
        dst[0] = lo;
        dst[1] = hi;
        continue;
      }
      uint4* out = accumulate ? reinterpret_cast<uint4*>(a.accum) + (size_t)home * n_vec + i : mine + i;
      if (accumulate && !a.overwrite) add8(acc[j], *out);
      uint4 o;
      __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int c = 0; c < 4; ++c) po[c] = __floats2bfloat162_rn(acc[j][2 * c], acc[j][2 * c + 1]);
      *out = o;
    }
  }
}

// One warp per row: the row's gate-weight gradient is a dot product over the row, reduced by shuffles.
__global__ void __launch_bounds__(256) swiglu_backward_kernel(SwigluBwdArgs a) {
  int rows = a.rows;
  if (a.row_limit != nullptr && *a.row_limit < rows) rows = *a.row_limit;
  const int lane = threadIdx.x & 31;
  const int vec_per_row = a.F / 8;
  const uint4* dact = reinterpret_cast<const uint4*>(a.dact);
  uint4* h = reinterpret_cast<uint4*>(a.h);
  const int warps = (int)((gridDim.x * blockDim.x) >> 5);
  for (int r = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5); r < rows; r += warps) {
    const float p = a.rowp != nullptr ? a.rowp[r] : 1.f;
    uint4* hrow = h + (size_t)r * (2 * vec_per_row);
    const uint4* drow = dact + (size_t)r * vec_per_row;
    float dot = 0.f;
    for (int v = lane; v < vec_per_row; v += 32) {
      const uint4 d4 = drow[v], g4 = hrow[v], u4 = hrow[vec_per_row + v];
      const __nv_bfloat162* dp = reinterpret_cast<const __nv_bfloat162*>(&d4);
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
      const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u4);
      uint4 og, ou;
      __nv_bfloat162* ogp = reinterpret_cast<__nv_bfloat162*>(&og);
      __nv_bfloat162* oup = reinterpret_cast<__nv_bfloat162*>(&ou);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 d = __bfloat1622float2(dp[k]), g = __bfloat1622float2(gp[k]), u = __bfloat1622float2(up[k]);
        const float s0 = __fdividef(1.f, 1.f + __expf(-g.x)), s1 = __fdividef(1.f, 1.f + __expf(-g.y));
        const float a0 = g.x * s0, a1 = g.y * s1;  // silu(g)
        dot += d.x * a0 * u.x + d.y * a1 * u.y;
        const float pd0 = p * d.x, pd1 = p * d.y;
        ogp[k] = __floats2bfloat162_rn(pd0 * u.x * (s0 + a0 * (1.f - s0)), pd1 * u.y * (s1 + a1 * (1.f - s1)));
        oup[k] = __floats2bfloat162_rn(pd0 * a0, pd1 * a1);
      }
      hrow[v] = og;
      hrow[vec_per_row + v] = ou;
    }
    if (a.dprob_ptrs != nullptr) {
      for (int off = 16; off > 0; off >>= 1) dot += __shfl_down_sync(kFull, dot, off);
      if (lane == 0) {
        const int2 m = a.meta[r];
        if (m.x >= 0) a.dprob_ptrs[m.x][m.y] = dot;
      }
    }
  }
}

__global__ void wait_probe_kernel(const unsigned* flag, unsigned target, unsigned long long budget_ns, int* status) {
  if (threadIdx.x == 0 && !wait_ge<true>(flag, target, budget_ns)) set_status(status, kStatusSignalTimeout, 60);
}

}  // namespace

cudaError_t launch_count_publish(const CountArgs& a, cudaStream_t stream) {
  const int chunks = route_chunks(a.num_units);
  if (chunks <= 0 || a.E <= 0) return cudaErrorInvalidValue;
  count_publish_kernel<<<chunks, kRouteChunk, sizeof(int) * a.E, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_route_assign(const RouteArgs& a, cudaStream_t stream) {
  const int chunks = route_chunks(a.num_units);
  if (chunks <= 0) return cudaErrorInvalidValue;
  const size_t smem = sizeof(int) * (size_t)a.E * (1 + kRouteChunk / 32);
  if (smem > 48 * 1024) return cudaErrorInvalidValue;  // E <= 1365
  route_assign_kernel<<<chunks, kRouteChunk, smem, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_comm(const CommArgs& a, int num_sms, int* status, cudaStream_t stream) {
  if (a.H % 8 != 0 || a.block_rows <= 0 || a.tile_rows % a.block_rows != 0 || a.tile_rows % 32 != 0) return cudaErrorInvalidValue;
  if (a.w1_elems % 8 != 0 || a.w2_elems % 8 != 0) return cudaErrorInvalidValue;
  if (num_sms <= 0) num_sms = sm_count();
  static bool configured[kMaxTrackedDevices] = {};
  int dev;
  if (device_needs_setup(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(comm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kCommKernelSmem);
    if (e != cudaSuccess) return e;
    device_setup_done(configured, dev);
  }
  // one CTA per SM
  comm_kernel<<<num_sms, kCommKernelWarps * 32, kCommKernelSmem, stream>>>(a, status);
  return cudaGetLastError();
}

cudaError_t launch_unit_reduce(const void* unit_rows, const int32_t* unit_pos, const float* unit_scale, void* out,
                               int num_tokens, int topk, int H, const UnitReduceWait* wait, const float* copy_src, float* copy_dst,
                               cudaStream_t stream) {
  if (H % 8 != 0) return cudaErrorInvalidValue;
  const int wpb = 8;
  const long long items = (long long)num_tokens * ceil_div(H / 8, 32);
  if (items == 0) return cudaSuccess;
  UnitReduceWait w{};
  if (wait != nullptr) w = *wait;
  unit_reduce_kernel<<<(unsigned)((items + wpb - 1) / wpb), wpb * 32, 0, stream>>>(
      reinterpret_cast<const uint4*>(unit_rows), unit_pos, unit_scale, reinterpret_cast<uint4*>(out), num_tokens, topk, H / 8, w,
      copy_src, copy_src != nullptr ? copy_dst : nullptr);
  return cudaGetLastError();
}

cudaError_t launch_symm_barrier(unsigned* const* signal_ptrs, int slot, int R, int me, unsigned* epoch_word,
                                int* status, cudaStream_t stream) {
  int threads = round_up(R, 32);
  symm_barrier_kernel<<<1, threads, 0, stream>>>(signal_ptrs, slot, R, me, epoch_word, status);
  return cudaGetLastError();
}

cudaError_t launch_weight_pull(const WeightPullArgs& a, cudaStream_t stream) {
  const int replica_slots = a.n_slot - a.home_cap;
  if (replica_slots <= 0) return cudaSuccess;
  if (a.elems_per_slot % 8 != 0) return cudaErrorInvalidValue;
  // about two waves of CTAs over all replica slots: a pull of one or two experts must still keep
  // enough 16-byte peer loads in flight to fill NVLink
  int gx = (2 * sm_count() + replica_slots - 1) / replica_slots;
  if (gx < 32) gx = 32;
  if (gx > 160) gx = 160;
  dim3 grid(gx, replica_slots);
  weight_pull_kernel<<<grid, 512, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_grad_reduce(const GradReduceArgs& a, cudaStream_t stream) {
  if (a.home_cap <= 0) return cudaSuccess;
  if (a.elems_per_slot % 8 != 0 || a.R > kMaxGradHosts) return cudaErrorInvalidValue;
  // Which home slots have replicas is known on the device only.  Every slot gets a full machine's worth of CTAs: the
  // CTAs of slots without replicas leave at once, those of a replicated expert keep every SM loading.
  int gx = sm_count();
  if (gx > 256) gx = 256;
  dim3 grid(gx, a.home_cap);
  grad_reduce_kernel<<<grid, 512, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_swiglu_backward(const SwigluBwdArgs& a, cudaStream_t stream) {
  if (a.F % 8 != 0) return cudaErrorInvalidValue;
  if (a.rows <= 0) return cudaSuccess;
  swiglu_backward_kernel<<<sm_count() * 8, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_wait_probe(const unsigned* flag, unsigned target, unsigned long long budget_ns, int* status,
                              cudaStream_t stream) {
  wait_probe_kernel<<<1, 32, 0, stream>>>(flag, target, budget_ns, status);
  return cudaGetLastError();
}

}  // namespace epb
