// Token-path and weight-path kernels: count + publish, route assignment, dispatch, unit reduce,
// cross-rank barrier, replica weight pull and owner-side gradient return.
//
// Replaces the reference's torch-op chains and NCCL calls on the MoE path:
//   bincount + all_gather (eplb/distributed.py:17-61)            -> count_publish_kernel
//   assign_physical + argsort/index_select (physical.py:30-77,
//       eplb_manager.py:1067-1105)                                -> route_assign + dispatch
//   index_add scatter with gate weight (eplb_manager.py:889-899)  -> unit_reduce_kernel
//   dist.broadcast per expert / GIN get (overlap.py:113-148,
//       gin_weights.py:305-341)                                   -> weight_pull_kernel
//   dist.reduce per expert / GIN put + sum (overlap.py:203-232,
//       gin_weights.py:343-377)                                   -> grad_reduce_kernel
// All remote traffic is plain peer loads/stores through NVSwitch; no cluster-multicast loads.
#include "route.h"

#include <cuda_bf16.h>

#include "common.cuh"

namespace epb {
namespace {

constexpr unsigned kFull = 0xffffffffu;

// ------------------------------------------------------------------ count + publish
__global__ void __launch_bounds__(1024) count_publish_kernel(const int64_t* __restrict__ unit_expert, int U, int E,
                                                            int R, int me, int32_t* const* omega_ptrs,
                                                            unsigned* const* signal_ptrs, unsigned* epoch_word) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  for (int u = threadIdx.x; u < U; u += blockDim.x) {
    int e = (int)unit_expert[u];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < E * R; idx += blockDim.x) {
    int peer = idx / E, e = idx - peer * E;
    omega_ptrs[peer][(size_t)me * E + e] = hist[e];
  }
  if (threadIdx.x == 0 && epoch_word != nullptr) *epoch_word += 1u;
  __threadfence_system();
  __syncthreads();
  if (signal_ptrs != nullptr && threadIdx.x < R) red_release_sys_add(signal_ptrs[threadIdx.x], 1u);
}

// ------------------------------------------------------------------ route assignment
// One CTA per expert.  Units of the expert are ranked in their original order with a block-wide
// ballot scan; the j-th unit goes to the host whose quota prefix covers j.
__global__ void __launch_bounds__(1024) route_assign_kernel(const int64_t* __restrict__ unit_expert, int U, int E,
                                                           int R, const int32_t* __restrict__ q_me,
                                                           const int32_t* __restrict__ row_base,
                                                           int32_t* __restrict__ unit_dst,
                                                           int32_t* __restrict__ unit_row, int* status) {
  extern __shared__ int sm[];
  int* qpre = sm;               // [R + 1] exclusive prefix of q_me[e, :]
  int* base = sm + (R + 1);     // [R]
  int* warp_cnt = base + R;     // [32]
  __shared__ int running;
  const int e = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  if (tid == 0) {
    int acc = 0;
    for (int r = 0; r < R; ++r) {
      qpre[r] = acc;
      acc += q_me[(size_t)e * R + r];
      base[r] = row_base[(size_t)e * R + r];
    }
    qpre[R] = acc;
    running = 0;
  }
  __syncthreads();
  const int total = qpre[R];
  for (int start = 0; start < U; start += blockDim.x) {
    const int u = start + tid;
    const bool hit = u < U && (int)unit_expert[u] == e;
    const unsigned m = __ballot_sync(kFull, hit);
    if (lane == 0) warp_cnt[warp] = __popc(m);
    __syncthreads();
    int before = running;
    for (int w = 0; w < warp; ++w) before += warp_cnt[w];
    if (hit) {
      const int j = before + __popc(m & ((1u << lane) - 1u));
      int dst = 0;
      while (dst + 1 < R && j >= qpre[dst + 1]) ++dst;
      if (j >= total) {
        set_status(status, kStatusBadArgument, 40, e);
        unit_dst[u] = -1;
        unit_row[u] = -1;
      } else {
        unit_dst[u] = dst;
        unit_row[u] = base[dst] + (j - qpre[dst]);
      }
    }
    __syncthreads();
    if (tid == 0) {
      int add = 0;
      for (int w = 0; w < nwarps; ++w) add += warp_cnt[w];
      running += add;
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ dispatch
// One warp per unit: 16-byte loads of the token row, 16-byte stores into the destination rank's
// receive buffer.  Blocks past the unit range zero this rank's padding rows.
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b) {
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
    acc += fa.x * fb.x + fa.y * fb.y;
  }
  return acc;
}
__device__ __forceinline__ uint4 scale8(const uint4& a, float s) {
  uint4 out;
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(pa[i]);
    po[i] = __floats2bfloat162_rn(f.x * s, f.y * s);
  }
  return out;
}

__global__ void __launch_bounds__(256) dispatch_kernel(DispatchArgs a, int unit_blocks) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const int vec_per_row = a.H / 8;  // uint4 = 8 bf16
  if ((int)blockIdx.x < unit_blocks) {
    const int u = blockIdx.x * wpb + warp;
    if (u >= a.num_units) return;
    const int dst = a.unit_dst[u], row = a.unit_row[u];
    const int t = u / a.topk;
    const uint4* src = reinterpret_cast<const uint4*>(a.rows) + (size_t)t * vec_per_row;
    const float s = a.unit_scale ? a.unit_scale[u] : 1.f;
    const uint4* saved = a.saved_out ? reinterpret_cast<const uint4*>(a.saved_out) + (size_t)u * vec_per_row : nullptr;
    uint4* out = (dst >= 0 && row < a.row_capacity) ? reinterpret_cast<uint4*>(a.buf_ptrs[dst]) + (size_t)row * vec_per_row : nullptr;
    float dot = 0.f;
    int v = lane;
    // four independent 16-byte loads in flight per lane before the first store
    for (; v + 96 < vec_per_row; v += 128) {
      uint4 val[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) val[j] = src[v + 32 * j];
      if (saved) {
#pragma unroll
        for (int j = 0; j < 4; ++j) dot += dot8(val[j], saved[v + 32 * j]);
      }
      if (out) {
#pragma unroll
        for (int j = 0; j < 4; ++j) out[v + 32 * j] = a.unit_scale ? scale8(val[j], s) : val[j];
      }
    }
    for (; v < vec_per_row; v += 32) {
      uint4 val = src[v];
      if (saved) dot += dot8(val, saved[v]);
      if (out) out[v] = a.unit_scale ? scale8(val, s) : val;
    }
    if (saved) {
      for (int off = 16; off > 0; off >>= 1) dot += __shfl_down_sync(kFull, dot, off);
      if (lane == 0) a.unit_dot[u] = dot;
    }
    if (lane == 0 && out != nullptr && a.meta_ptrs != nullptr) a.meta_ptrs[dst][row] = make_int2(a.me, u);
  } else {
    // padding rows of slot g: [off + rows, next off)
    const int g = blockIdx.x - unit_blocks;
    if (g >= a.n_slot) return;
    const int lo = min(a.slot_off[g] + a.slot_rows[g], a.row_capacity), hi = min(a.slot_off[g + 1], a.row_capacity);
    uint4* buf = reinterpret_cast<uint4*>(a.local_buf);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const size_t begin = (size_t)lo * vec_per_row, end = (size_t)hi * vec_per_row;
    for (size_t i = begin + threadIdx.x; i < end; i += blockDim.x) buf[i] = zero;
  }
}

// ------------------------------------------------------------------ unit reduce
__global__ void __launch_bounds__(256) unit_reduce_kernel(const uint4* __restrict__ unit_rows,
                                                         const float* __restrict__ unit_scale,
                                                         uint4* __restrict__ out, int num_tokens, int topk,
                                                         int vec_per_row) {
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
    const uint4 val = unit_rows[u * vec_per_row + v];
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
  __shared__ int host_rank[64];
  __shared__ int host_slot[64];
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
    for (int h = 0; h < a.R && n < 64; ++h) {
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
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (!a.include_self) add8(acc, mine[i]);
    for (int k = 0; k < n; ++k) {
      const uint4* peer = reinterpret_cast<const uint4*>(a.g_ptrs[host_rank[k]]) + (size_t)host_slot[k] * n_vec;
      add8(acc, peer[i]);
    }
    if (accumulate && a.accum_fp32) {
      float4* dst = reinterpret_cast<float4*>(a.accum) + ((size_t)home * n_vec + i) * 2;
      float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
      if (!a.overwrite) {
        lo = dst[0];
        hi = dst[1];
      }
      lo.x += acc[0]; lo.y += acc[1]; lo.z += acc[2]; lo.w += acc[3];
      hi.x += acc[4]; hi.y += acc[5]; hi.z += acc[6]; hi.w += acc[7];
      dst[0] = lo;
      dst[1] = hi;
      continue;
    }
    uint4* out = accumulate ? reinterpret_cast<uint4*>(a.accum) + (size_t)home * n_vec + i : mine + i;
    if (accumulate && !a.overwrite) add8(acc, *out);
    uint4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) po[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *out = o;
  }
}

__global__ void __launch_bounds__(256) swiglu_backward_kernel(const uint4* __restrict__ dact, uint4* __restrict__ h,
                                                             int rows, int F, const int32_t* __restrict__ row_limit) {
  if (row_limit != nullptr && *row_limit < rows) rows = *row_limit;
  const int vec_per_row = F / 8;
  const size_t total = (size_t)rows * vec_per_row;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const size_t r = i / vec_per_row;
    const int v = (int)(i - r * vec_per_row);
    uint4* hrow = h + r * (size_t)(2 * vec_per_row);
    const uint4 d4 = dact[i], g4 = hrow[v], u4 = hrow[vec_per_row + v];
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
      ogp[k] = __floats2bfloat162_rn(d.x * u.x * (s0 + g.x * s0 * (1.f - s0)), d.y * u.y * (s1 + g.y * s1 * (1.f - s1)));
      oup[k] = __floats2bfloat162_rn(d.x * g.x * s0, d.y * g.y * s1);
    }
    hrow[v] = og;
    hrow[vec_per_row + v] = ou;
  }
}

__global__ void wait_probe_kernel(const unsigned* flag, unsigned target, unsigned long long budget_ns, int* status) {
  if (threadIdx.x == 0 && !wait_ge<true>(flag, target, budget_ns)) set_status(status, kStatusSignalTimeout, 60);
}

}  // namespace

cudaError_t launch_count_publish(const int64_t* unit_expert, int num_units, int E, int R, int me,
                                 int32_t* const* omega_ptrs, unsigned* const* signal_ptrs, unsigned* epoch_word,
                                 cudaStream_t stream) {
  count_publish_kernel<<<1, 1024, sizeof(int) * E, stream>>>(unit_expert, num_units, E, R, me, omega_ptrs, signal_ptrs,
                                                            epoch_word);
  return cudaGetLastError();
}

cudaError_t launch_route_assign(const int64_t* unit_expert, int num_units, int E, int R, const int32_t* q_me,
                                const int32_t* row_base, int32_t* unit_dst, int32_t* unit_row, int* status,
                                cudaStream_t stream) {
  const size_t smem = sizeof(int) * (2 * R + 1 + 32);
  route_assign_kernel<<<E, 1024, smem, stream>>>(unit_expert, num_units, E, R, q_me, row_base, unit_dst, unit_row, status);
  return cudaGetLastError();
}

cudaError_t launch_dispatch(const DispatchArgs& a, cudaStream_t stream) {
  if (a.H % 8 != 0) return cudaErrorInvalidValue;
  const int wpb = 8;
  const int unit_blocks = ceil_div(a.num_units, wpb);
  dispatch_kernel<<<unit_blocks + a.n_slot, wpb * 32, 0, stream>>>(a, unit_blocks);
  return cudaGetLastError();
}

cudaError_t launch_unit_reduce(const void* unit_rows, const float* unit_scale, void* out, int num_tokens, int topk,
                               int H, cudaStream_t stream) {
  if (H % 8 != 0) return cudaErrorInvalidValue;
  const int wpb = 8;
  const long long items = (long long)num_tokens * ceil_div(H / 8, 32);
  if (items == 0) return cudaSuccess;
  unit_reduce_kernel<<<(unsigned)((items + wpb - 1) / wpb), wpb * 32, 0, stream>>>(
      reinterpret_cast<const uint4*>(unit_rows), unit_scale, reinterpret_cast<uint4*>(out), num_tokens, topk, H / 8);
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
  int gx = (2 * 148 + replica_slots - 1) / replica_slots;
  if (gx < 32) gx = 32;
  if (gx > 160) gx = 160;
  dim3 grid(gx, replica_slots);
  weight_pull_kernel<<<grid, 512, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_grad_reduce(const GradReduceArgs& a, cudaStream_t stream) {
  if (a.home_cap <= 0) return cudaSuccess;
  if (a.elems_per_slot % 8 != 0 || a.R > 64) return cudaErrorInvalidValue;
  int gx = (2 * 148 + a.home_cap - 1) / a.home_cap;  // about two waves of CTAs in total
  if (gx < 64) gx = 64;
  if (gx > 256) gx = 256;
  dim3 grid(gx, a.home_cap);
  grad_reduce_kernel<<<grid, 512, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_swiglu_backward(const void* dact, void* h, int rows, int F, const int32_t* row_limit,
                                   cudaStream_t stream) {
  if (F % 8 != 0) return cudaErrorInvalidValue;
  if (rows <= 0) return cudaSuccess;
  swiglu_backward_kernel<<<148 * 8, 256, 0, stream>>>(reinterpret_cast<const uint4*>(dact), reinterpret_cast<uint4*>(h), rows,
                                                     F, row_limit);
  return cudaGetLastError();
}

cudaError_t launch_wait_probe(const unsigned* flag, unsigned target, unsigned long long budget_ns, int* status,
                              cudaStream_t stream) {
  wait_probe_kernel<<<1, 32, 0, stream>>>(flag, target, budget_ns, status);
  return cudaGetLastError();
}

}  // namespace epb
