// Fused AdamW: one pass over parameter, gradient and both moments with 16-byte accesses.
// The expert weights of an MoE layer are one flat bf16 tensor per projection, so a single launch
// covers them; this replaces the multi-tensor optimizer launches over per-expert parameters.
#include "optim.h"

#include <cuda_bf16.h>

namespace epb {
namespace {

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const AdamArgs& a) {
  p *= 1.f - a.lr * a.weight_decay;
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  const float denom = sqrtf(v) / a.bias_correction2_sqrt + a.eps;
  p -= (a.lr / a.bias_correction1) * (m / denom);
}

// With a device step counter the two bias corrections are derived here, once per thread.
__device__ __forceinline__ void resolve_step(AdamArgs& a) {
  if (a.step_ptr != nullptr) {
    const float t = (float)(*a.step_ptr);
    a.bias_correction1 = 1.f - powf(a.beta1, t);
    a.bias_correction2_sqrt = sqrtf(1.f - powf(a.beta2, t));
  }
}

// True while any status word of the guard is set (every thread reads the same few words; they are cached).
__device__ __forceinline__ bool guard_tripped(const AdamArgs& a) {
  if (a.guard == nullptr) return false;
  for (int i = 0; i < a.guard_rows; ++i)
    if (a.guard[4 * i] != 0) return true;
  return false;
}

__global__ void __launch_bounds__(256) adamw_bf16_kernel(AdamArgs a) {
  if (guard_tripped(a)) return;
  resolve_step(a);
  const size_t n_vec = a.numel / 8;
  uint4* p4 = reinterpret_cast<uint4*>(a.param);
  const uint4* g4 = reinterpret_cast<const uint4*>(a.grad);
  uint4* m4 = reinterpret_cast<uint4*>(a.exp_avg);
  uint4* v4 = reinterpret_cast<uint4*>(a.exp_avg_sq);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    uint4 pv = p4[i], mv = m4[i], vv = v4[i];
    float gf[8];
    if (a.grad_f32) {
      const float4* gq = reinterpret_cast<const float4*>(a.grad) + i * 2;
      const float4 lo = gq[0], hi = gq[1];
      gf[0] = lo.x; gf[1] = lo.y; gf[2] = lo.z; gf[3] = lo.w;
      gf[4] = hi.x; gf[5] = hi.y; gf[6] = hi.z; gf[7] = hi.w;
    } else {
      const uint4 gv = g4[i];
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 g = __bfloat1622float2(gp[k]);
        gf[2 * k] = g.x;
        gf[2 * k + 1] = g.y;
      }
    }
    __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pv);
    __nv_bfloat162* mp = reinterpret_cast<__nv_bfloat162*>(&mv);
    __nv_bfloat162* vp = reinterpret_cast<__nv_bfloat162*>(&vv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 p = __bfloat1622float2(pp[k]);
      float2 m = __bfloat1622float2(mp[k]), v = __bfloat1622float2(vp[k]);
      adam_one(p.x, gf[2 * k], m.x, v.x, a);
      adam_one(p.y, gf[2 * k + 1], m.y, v.y, a);
      pp[k] = __floats2bfloat162_rn(p.x, p.y);
      mp[k] = __floats2bfloat162_rn(m.x, m.y);
      vp[k] = __floats2bfloat162_rn(v.x, v.y);
    }
    p4[i] = pv;
    m4[i] = mv;
    v4[i] = vv;
  }
  // tail (numel not a multiple of 8)
  const size_t done = n_vec * 8;
  __nv_bfloat16* p1 = reinterpret_cast<__nv_bfloat16*>(a.param);
  const __nv_bfloat16* g1 = reinterpret_cast<const __nv_bfloat16*>(a.grad);
  __nv_bfloat16* m1 = reinterpret_cast<__nv_bfloat16*>(a.exp_avg);
  __nv_bfloat16* v1 = reinterpret_cast<__nv_bfloat16*>(a.exp_avg_sq);
  for (size_t i = done + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.numel; i += stride) {
    float p = __bfloat162float(p1[i]), m = __bfloat162float(m1[i]), v = __bfloat162float(v1[i]);
    const float g = a.grad_f32 ? reinterpret_cast<const float*>(a.grad)[i] : __bfloat162float(g1[i]);
    adam_one(p, g, m, v, a);
    p1[i] = __float2bfloat16_rn(p);
    m1[i] = __float2bfloat16_rn(m);
    v1[i] = __float2bfloat16_rn(v);
  }
}

__global__ void __launch_bounds__(256) adamw_f32_kernel(AdamArgs a) {
  if (guard_tripped(a)) return;
  resolve_step(a);
  float* p = reinterpret_cast<float*>(a.param);
  const float* g = reinterpret_cast<const float*>(a.grad);
  float* m = reinterpret_cast<float*>(a.exp_avg);
  float* v = reinterpret_cast<float*>(a.exp_avg_sq);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.numel; i += stride) {
    float pi = p[i], mi = m[i], vi = v[i];
    adam_one(pi, g[i], mi, vi, a);
    p[i] = pi;
    m[i] = mi;
    v[i] = vi;
  }
}

}  // namespace

cudaError_t launch_adamw(const AdamArgs& a, cudaStream_t stream) {
  if (a.numel == 0) return cudaSuccess;
  const size_t work = a.is_bf16 ? (a.numel + 7) / 8 : a.numel;
  size_t blocks = (work + 255) / 256;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 132;
  if (blocks > (size_t)sms * 16) blocks = (size_t)sms * 16;
  if (a.is_bf16) adamw_bf16_kernel<<<(unsigned)blocks, 256, 0, stream>>>(a);
  else adamw_f32_kernel<<<(unsigned)blocks, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace epb
