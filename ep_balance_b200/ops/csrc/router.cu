// One warp per token.  Element e of the row lives in lane e % 32, register slot e / 32 (up to 32 slots).
// Every selection step is a warp arg-max (value descending, index ascending on ties) followed by
// masking the winner; 2*G + topk_groups + K steps in group-limited mode.
#include "router.h"

#include <math_constants.h>

namespace epb {
namespace {

constexpr int kMaxSlots = 32;
constexpr unsigned kFull = 0xffffffffu;

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }
__device__ __forceinline__ Best warp_argmax(Best x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y{__shfl_xor_sync(kFull, x.v, o), __shfl_xor_sync(kFull, x.i, o)};
    x = better(x, y);
  }
  return x;
}

template <int kSlots>
__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                         int N, int E, int K, int mode, int n_groups, int topk_groups,
                                                         float scale, int64_t* __restrict__ idx,
                                                         float* __restrict__ weights) {
  const int lane = threadIdx.x & 31;
  const int t = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5);
  if (t >= N) return;
  const float kNone = -CUDART_INF_F;
  float s[kSlots];        // selection score of each element held by this lane (-inf: absent or taken)
#pragma unroll
  for (int j = 0; j < kSlots; ++j) {
    const int e = j * 32 + lane;
    float v = kNone;
    if (e < E) {
      v = logits[(size_t)t * E + e] + (bias ? bias[e] : 0.f);
      if (mode == kRouterGroupLimited) v = __fdividef(1.f, 1.f + __expf(-v));
    }
    s[j] = v;
  }
  if (mode == kRouterGroupLimited) {
    const int gsize = E / n_groups;
    // score of group g = sum of its two best members; lane g keeps it
    float my_group_score = kNone;
    for (int g = 0; g < n_groups; ++g) {
      float sum = 0.f;
      int taken = -1;
      for (int pass = 0; pass < 2; ++pass) {
        Best b{kNone, 0x7fffffff};
#pragma unroll
        for (int j = 0; j < kSlots; ++j) {
          const int e = j * 32 + lane;
          if (e < E && e / gsize == g && e != taken) b = better(b, Best{s[j], e});
        }
        b = warp_argmax(b);
        if (b.v > kNone) sum += b.v;
        taken = b.i;
      }
      if (lane == (g & 31)) my_group_score = (g < 32) ? sum : my_group_score;
    }
    // keep the best topk_groups groups (n_groups <= 32)
    unsigned keep = 0u;
    for (int r = 0; r < topk_groups; ++r) {
      Best b = warp_argmax(Best{lane < n_groups ? my_group_score : kNone, lane});
      keep |= 1u << b.i;
      if (lane == b.i) my_group_score = kNone;
    }
#pragma unroll
    for (int j = 0; j < kSlots; ++j) {
      const int e = j * 32 + lane;
      // experts of dropped groups compete with score 0 (they are only chosen when fewer than K remain)
      if (e < E && !((keep >> (e / gsize)) & 1u)) s[j] = 0.f;
    }
  }
  // top-K of s
  float my_val = 0.f;   // lane r keeps the r-th winner
  int my_idx = 0;
  for (int r = 0; r < K; ++r) {
    Best b{kNone, 0x7fffffff};
#pragma unroll
    for (int j = 0; j < kSlots; ++j) {
      const int e = j * 32 + lane;
      if (e < E) b = better(b, Best{s[j], e});
    }
    b = warp_argmax(b);
#pragma unroll
    for (int j = 0; j < kSlots; ++j)
      if (j * 32 + lane == b.i) s[j] = kNone;
    if (lane == r) {
      my_val = b.v;
      my_idx = b.i;
    }
  }
  // gate weights
  float w;
  if (mode == kRouterSoftmaxTopk) {
    const float top = __shfl_sync(kFull, my_val, 0);   // winners are in descending order
    float ex = lane < K ? __expf(my_val - top) : 0.f;
    float sum = ex;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(kFull, sum, o);
    w = ex / sum;
  } else if (mode == kRouterSigmoidTopk) {
    w = __fdividef(1.f, 1.f + __expf(-my_val));
  } else {
    float sum = lane < K ? my_val : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(kFull, sum, o);
    w = my_val / fmaxf(sum, 1e-20f) * scale;
  }
  if (lane < K) {
    idx[(size_t)t * K + lane] = my_idx;
    weights[(size_t)t * K + lane] = w;
  }
}

}  // namespace

cudaError_t launch_router_topk(const float* logits, const float* bias, int N, int E, int K, int mode, int n_groups,
                               int topk_groups, float scale, int64_t* idx, float* weights, cudaStream_t stream) {
  if (N <= 0) return cudaSuccess;
  if (E < K || E > 32 * kMaxSlots || K < 1 || K > 32) return cudaErrorInvalidValue;
  if (mode == kRouterGroupLimited && (n_groups < 1 || n_groups > 32 || E % n_groups != 0 || topk_groups < 1 || topk_groups > n_groups))
    return cudaErrorInvalidValue;
  const int blocks = (N + 7) / 8;
  const int slots = (E + 31) / 32;
#define EPB_ROUTER(S)                                                                                              \
  router_topk_kernel<S><<<blocks, 256, 0, stream>>>(logits, bias, N, E, K, mode, n_groups, topk_groups, scale, idx, \
                                                    weights)
  if (slots <= 2) EPB_ROUTER(2);
  else if (slots <= 4) EPB_ROUTER(4);
  else if (slots <= 8) EPB_ROUTER(8);
  else if (slots <= 16) EPB_ROUTER(16);
  else EPB_ROUTER(32);
#undef EPB_ROUTER
  return cudaGetLastError();
}

}  // namespace epb
