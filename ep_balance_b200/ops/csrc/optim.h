// Fused AdamW over one flat tensor (optim.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace epb {

struct AdamArgs {
  void* param;       // bf16 or fp32
  const void* grad;  // same dtype as param, or fp32 for a bf16 param when grad_f32 is set
  void* exp_avg;     // same dtype as param
  void* exp_avg_sq;  // same dtype as param
  size_t numel;
  float lr, beta1, beta2, eps, weight_decay;
  float bias_correction1, bias_correction2_sqrt;  // 1 - beta1^t, sqrt(1 - beta2^t)
  int is_bf16;
  int grad_f32;      // bf16 parameters with an fp32 (accumulated) gradient
  const int* guard;         // optional device status words [guard_rows, 4]: while any row's first int is non-zero the
  int guard_rows;           // kernel returns without touching parameter or moments (a damaged step is not applied)
  const int64_t* step_ptr;  // optional device step counter: when set, the bias corrections are computed from it in the
                            // kernel (the host-side values are ignored), which makes the launch CUDA-graph replayable
};

cudaError_t launch_adamw(const AdamArgs& a, cudaStream_t stream);

}  // namespace epb
