"""Multi-GPU correctness check of the fused MoE layer (one process per GPU, NCCL for bootstrap).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29517 -m ep_balance_b200.launch.check_multi [--steps 3] [--headline]

``--headline`` runs the shape of the headline benchmark (hidden 2048, SwiGLU 1408, 64 experts, top-6,
8192 tokens per rank, router skew tuned to expert max/mean 3.5, two logical domains from four ranks on).

Every rank runs forward+backward through the native path, then recomputes its own tokens through
the plain PyTorch oracle with the full set of expert weights (all-gathered).  Outputs, token
gradients, gate gradients and the owners' weight gradients (sum over every rank's contribution,
replicas included) must agree; the plan digest must be identical on all ranks.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def oracle_errors(layer, tokens, idx, prob, dout, out, dtok, dprob, rank: int, world: int) -> dict:
    """Relative L2 errors of one native forward+backward against the plain PyTorch fp32 oracle: this rank's
    outputs, token gradients and gate gradients, and the owners' weight gradients (the oracle's are summed
    over all ranks, replicas included).  Collective: every rank calls it."""
    from ..models.reference_moe import moe_reference

    if world > 1:
        w1s = [torch.empty_like(layer.w1.data) for _ in range(world)]
        w2s = [torch.empty_like(layer.w2.data) for _ in range(world)]
        dist.all_gather(w1s, layer.w1.data.contiguous())
        dist.all_gather(w2s, layer.w2.data.contiguous())
    else:
        w1s, w2s = [layer.w1.data], [layer.w2.data]
    w1 = torch.cat(w1s).float().requires_grad_(True)
    w2 = torch.cat(w2s).float().requires_grad_(True)
    x = tokens.float().requires_grad_(True)
    p = prob.clone().requires_grad_(True)
    o = moe_reference(x, idx, p, w1, w2)
    o.backward(dout.float())
    gw1, gw2 = w1.grad.clone(), w2.grad.clone()
    if world > 1:
        dist.all_reduce(gw1)
        dist.all_reduce(gw2)
    hc = layer.home_cap
    return {
        "out": rel(out, o.detach()), "dtokens": rel(dtok, x.grad), "dprob": rel(dprob, p.grad),
        "dw1": rel(layer.w1.grad, gw1[rank * hc:(rank + 1) * hc]),
        "dw2": rel(layer.w2.grad, gw2[rank * hc:(rank + 1) * hc]),
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--ffn", type=int, default=256)
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--headline", action="store_true", help="the headline benchmark's shape and router skew")
    ap.add_argument("--out", default=None, help="rank 0 also writes its report lines to this file")
    a = ap.parse_args()
    if a.headline:
        a.tokens, a.hidden, a.ffn, a.experts, a.topk = 8192, 2048, 1408, 64, 6
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from ..models.moe_layer import FusedMoE, MoEConfig, heap_layout
    from ..parallel.symm import SymmetricHeap

    domains = 2 if world % 2 == 0 and world >= 4 else 1
    cfg = MoEConfig(hidden=a.hidden, ffn=a.ffn, num_experts=a.experts, top_k=a.topk, max_tokens=a.tokens,
                    extra_slots=2, num_domains=domains, capacity_factor=2.0 if a.headline else float(world))
    heap = SymmetricHeap(heap_layout(cfg, world), dev)
    layer = FusedMoE(cfg, heap, rank, world)
    dist.broadcast(layer.router.data, src=0)
    if a.headline:
        from ..utils.workload import router_bias_for_imbalance

        bias = router_bias_for_imbalance(a.experts, a.topk, 0.02 * a.hidden ** 0.5, 3.5).to(dev)
    else:
        bias = torch.zeros(a.experts, device=dev)
        bias[:3] = 1.0  # three hot experts; the router's own logits (std ~0.3) still reach every expert
    layer.router_bias = bias
    ok = True
    report = []
    for step in range(a.steps):
        g = torch.Generator(device="cpu").manual_seed(100 * step + rank)
        tokens = torch.randn(a.tokens, a.hidden, generator=g).to(dev, torch.bfloat16)
        dout = torch.randn(a.tokens, a.hidden, generator=g).to(dev, torch.bfloat16)
        idx, prob = layer.route_tokens(tokens)
        prob = prob.detach()
        out = torch.empty_like(tokens)
        dtok = torch.empty_like(tokens)
        dprob = torch.empty_like(prob)
        layer.rt.trace_launches(step == a.steps - 1)
        layer.rt.forward(tokens.data_ptr(), idx.data_ptr(), prob.data_ptr(), out.data_ptr(), a.tokens)
        layer.rt.backward(dout.data_ptr(), dtok.data_ptr(), dprob.data_ptr(), a.tokens)
        torch.cuda.synchronize()
        layer.check_status()
        if step == a.steps - 1 and world > 1:
            # launch order of the multi-rank step: the gradient return (barrier + owner-side reduce, on the side
            # stream) is issued after the last weight-gradient GEMM and before Dgrad1, so that it runs beside it
            log = layer.rt.launch_log()
            side = [i for i, n in enumerate(log) if n.startswith("side:")]
            gemms = [i for i, n in enumerate(log) if n.startswith("grouped_gemm")]
            order_ok = (log[:3] == ["count_publish", "solver", "route_assign"] and len(side) == 3
                        and log[side[0]] == "side:symm_barrier" and side == list(range(side[0], side[0] + 3))
                        and gemms[-2] < side[0] < gemms[-1] and log[-1] == "unit_reduce(bwd)")
            if not order_ok:
                ok = False
                print(f"[rank {rank}] unexpected launch order: {log}", flush=True)
        dist.barrier()

        errs = oracle_errors(layer, tokens, idx, prob, dout, out, dtok, dprob, rank, world)
        digests = [None] * world
        dist.all_gather_object(digests, layer.last_plan().digest())
        same_plan = len(set(digests)) == 1
        replicas = int(layer.last_plan().x.sum()) - a.experts
        good = all(v < 3e-2 for v in errs.values()) and same_plan
        ok = ok and good
        loads = layer.rank_loads().float()
        line = (f"[rank {rank}/{world}] step {step} {'PASS' if good else 'FAIL'} plan_identical={same_plan} replicas={replicas} "
                f"rank_load_max_over_mean={float(loads.max() / loads.mean()):.3f} "
                + " ".join(f"{k}={v:.2e}" for k, v in errs.items()))
        print(line, flush=True)
        lines = [None] * world
        dist.all_gather_object(lines, line)
        report += lines
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        verdict = "CHECK_MULTI " + ("PASS" if int(flag) else "FAIL")
        print(verdict, flush=True)
        if a.out:
            shape = f"tokens/rank {a.tokens} hidden {a.hidden} ffn {a.ffn} experts {a.experts} top-{a.topk} ranks {world} domains {domains}"
            with open(a.out, "w") as fh:
                fh.write("\n".join([shape] + report + [verdict]) + "\n")
    return 0 if int(flag) else 1


if __name__ == "__main__":
    sys.exit(main())
