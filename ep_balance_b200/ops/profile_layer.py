"""Small single-GPU workload of the fused MoE layer for profiling its kernels (one forward + backward per iteration).

    python -m ep_balance_b200.ops.profile_layer [--tokens 4096] [--experts 16] [--iters 3] [--no-fused-transport]

With the defaults the step launches, per iteration, the fused transport+GEMM kernels
(``grouped_gemm_kernel<0, 2, 1>``: dispatch + GEMM1 + SwiGLU; ``grouped_gemm_kernel<3, 2, 1>``: gradient dispatch +
Dgrad2) besides the plain grouped GEMMs, the count/route kernels, the solver and the reduces.  The receive
buffers (24576 rows x 4 KB = 100 MB) exceed the L2 while the process holds about 1 GB, so a full-metric
capture of a few launches finishes quickly.  Prints the device time of every phase (CUDA events).
"""

from __future__ import annotations

import argparse

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=1408)
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--top-k", type=int, default=6)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--ctas", type=int, default=2, choices=[1, 2])
    ap.add_argument("--no-fused-transport", action="store_true")
    a = ap.parse_args()
    from ..models.emulated import EmulatedCluster
    from ..models.moe_layer import MoEConfig

    torch.manual_seed(0)
    cfg = MoEConfig(hidden=a.hidden, ffn=a.ffn, num_experts=a.experts, top_k=a.top_k, max_tokens=a.tokens,
                    gemm_ctas=a.ctas, fused_comm=not a.no_fused_transport)
    layer = EmulatedCluster(cfg, world=1).layers[0]
    x = torch.randn(a.tokens, a.hidden, device="cuda").bfloat16()
    dout = torch.randn_like(x)
    idx, prob = layer.route_tokens(x)
    prob = prob.detach()
    out, dtok, dprob = torch.empty_like(x), torch.empty_like(x), torch.empty_like(prob)
    rt = layer.rt
    for it in range(a.iters + 1):
        rt.enable_timing(it > 0)
        rt.forward(x.data_ptr(), idx.data_ptr(), prob.data_ptr(), out.data_ptr(), a.tokens)
        rt.backward(dout.data_ptr(), dtok.data_ptr(), dprob.data_ptr(), a.tokens)
        torch.cuda.synchronize()
        if it > 0:
            print(f"iteration {it}: " + "  ".join(f"{name}={ms * 1e3:.0f}us" for name, ms in rt.phase_times()))
    layer.check_status()
    rows = a.tokens * a.top_k
    flops = rows * 3 * (2 * a.hidden * 2 * a.ffn + 2 * a.ffn * a.hidden)
    print(f"rows {rows}, {flops / 1e12:.3f} TFLOP per forward+backward, status ok")


if __name__ == "__main__":
    main()
