// Fused top-k routing for inference (router.cu): one warp per token turns a row of fp32 logits into
// the selected expert ids and their gate weights.  Replaces the chain of PyTorch kernels (sigmoid / topk /
// scatter / where / topk / normalise: ~15 launches) that dominates a small-batch forward.
// Forward only: training keeps the differentiable PyTorch formulation.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace epb {

enum RouterMode : int {
  kRouterSoftmaxTopk = 0,   // top-k of the logits, softmax over the selected logits
  kRouterSigmoidTopk = 1,   // top-k of the logits, sigmoid of each selected logit
  kRouterGroupLimited = 2,  // DeepSeek-V3: sigmoid scores, groups ranked by the sum of their two best scores,
                            // top-k among the experts of the best `topk_groups` groups, weights normalised
};

// logits fp32 [N, E] (E <= 1024, E % n_groups == 0), optional bias fp32 [E] added first.
// idx int64 [N, K], weights fp32 [N, K]; K <= 32.
cudaError_t launch_router_topk(const float* logits, const float* bias, int N, int E, int K, int mode, int n_groups,
                               int topk_groups, float scale, int64_t* idx, float* weights, cudaStream_t stream);

}  // namespace epb
