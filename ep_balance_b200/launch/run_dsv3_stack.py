"""DeepSeek-V3-shaped MoE stack: one training step timing plus an inference-only forward sweep.

    python -m ep_balance_b200.launch.run_dsv3_stack --layers 1 --experts 32 --tokens 1024          # one GPU, reduced
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29523 -m ep_balance_b200.launch.run_dsv3_stack

Synthetic N(0,1) tokens, random-init weights, skewed router (bias tuned to expert max/mean ~= 4).
Device-timed with CUDA events, max over ranks.  Training runs bf16 expert GEMMs; ``--fp8`` adds the
inference forward with block-scaled fp8 expert GEMMs (1 x 128 activation, 128 x 128 weight scales).
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--layers", type=int, default=4)
    p.add_argument("--hidden", type=int, default=7168)
    p.add_argument("--ffn", type=int, default=2048)
    p.add_argument("--experts", type=int, default=256)
    p.add_argument("--tokens", type=int, default=4096)
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=2)
    p.add_argument("--infer-batches", type=int, nargs="*", default=[64, 256, 1024, 4096])
    p.add_argument("--graphs", action="store_true",
                   help="also time the inference forward replayed from a CUDA graph (one graph per batch size)")
    p.add_argument("--fp8", action="store_true", help="also time the inference forward with block-scaled fp8 expert GEMMs")
    a = p.parse_args(argv)
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from ..models.dsv3 import DSv3Config, DSv3Stack
    from ..utils.optim import FusedAdamW
    from ..utils.workload import router_bias_for_imbalance

    cfg = DSv3Config(layers=a.layers, hidden=a.hidden, ffn=a.ffn, experts=a.experts, shared_ffn=a.ffn,
                     max_tokens=a.tokens, num_domains=2 if world >= 4 else 1, fp8_inference=a.fp8)
    model = DSv3Stack(cfg, dev, rank=rank, world=world)
    if world > 1:
        for prm in model.dense_parameters():
            dist.broadcast(prm.data, src=0)
    bias = router_bias_for_imbalance(a.experts, cfg.top_k, 0.02 * a.hidden ** 0.5, 4.0).to(dev)
    model.set_router_bias(bias[None].expand(a.layers, -1))
    dense_opt = torch.optim.AdamW(model.dense_parameters(), lr=1e-5, fused=True)
    expert_opt = FusedAdamW(list(model.expert_parameters()), lr=1e-5)
    g = torch.Generator().manual_seed(5 + rank)
    x = torch.randn(a.tokens, a.hidden, generator=g).to(dev, torch.bfloat16)

    def timed(fn, n):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n):
            fn()
        t1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([t0.elapsed_time(t1) / n], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    def train_step():
        y = model(x.detach().requires_grad_(True))
        y.float().square().mean().backward()
        dense_opt.step()
        expert_opt.step()
        dense_opt.zero_grad(set_to_none=True)

    for _ in range(a.warmup):
        train_step()
    out = {"world": world, "layers": a.layers, "hidden": a.hidden, "experts": a.experts, "tokens_per_rank": a.tokens,
           "dtype": "bf16", "train_ms_per_step": timed(train_step, a.steps)}
    out["train_tokens_per_s"] = a.tokens * world / (out["train_ms_per_step"] * 1e-3)
    loads = model.blocks[0].moe.rank_loads().float()
    out["rank_load_max_over_mean_layer0"] = float(loads.max() / loads.mean().clamp_min(1))
    def graphed(xb):
        """Capture one forward of the whole stack and return a replay function (static input and output)."""
        static_in = xb.clone()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                model(static_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_out = model(static_in)
        return graph.replay, static_out

    infer = {}
    with torch.no_grad():
        for nb in a.infer_batches:
            if nb > a.tokens:
                continue
            xb = x[:nb].contiguous()
            model(xb)
            infer[str(nb)] = timed(lambda: model(xb), a.steps)
            if a.graphs:
                replay, _ = graphed(xb)
                infer[f"{nb}_graph"] = timed(replay, a.steps)
    out["inference_forward_ms"] = infer
    if a.fp8:
        model.quantize_weights()
        infer8, err = {}, {}
        with torch.no_grad():
            for nb in a.infer_batches:
                if nb > a.tokens:
                    continue
                xb = x[:nb].contiguous()
                # numerical error of the fp8 expert GEMMs: first layer's routed output for the same input and the
                # same routing.  (Whole-stack outputs differ by more: a few per cent of noise flips near-tied
                # top-k choices in later layers, which is a property of discrete routing, not of the kernels.)
                moe0, h0 = model.blocks[0].moe, model.blocks[0].norm(xb)
                y8 = moe0(h0)
                moe0._fp8_ready = False
                y16 = moe0(h0)
                moe0._fp8_ready = True
                err[str(nb)] = float((y8.float() - y16.float()).norm() / y16.float().norm().clamp_min(1e-12))
                model(xb)  # first use of a kernel variant at this batch size loads it: keep that out of the timing
                infer8[str(nb)] = timed(lambda: model(xb), a.steps)
                if a.graphs:
                    replay, _ = graphed(xb)
                    infer8[f"{nb}_graph"] = timed(replay, a.steps)
        out["inference_forward_fp8_ms"] = infer8
        out["fp8_vs_bf16_layer_relative_error"] = err
    model.check_status()
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out


if __name__ == "__main__":
    main()
