"""Training entry point: GPT-MoE on synthetic tokens with per-layer drifting router skew.

    python -m ep_balance_b200.launch.train_gpt_moe --layers 2 --steps 5                    # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29521 -m ep_balance_b200.launch.train_gpt_moe --steps 20

Environment knobs kept from the reference launcher (scripts/run_real_moe.sh, pretrain_eplb_moe.py):
``EPLB_MODE=off|apply`` (``off`` gives every rank zero replica slots, i.e. plain expert parallelism),
``EPLB_N_SLOT`` (TOTAL slots per rank), ``GPUS_PER_NODE`` (ranks per logical domain),
``ROUTER_SKEW`` (scale of the drifting logit bias).  Iteration lines use Megatron's format so
``ep_balance_b200.eval.extract_train_metrics`` parses them.
"""

from __future__ import annotations

import argparse
import os
import time

import torch
import torch.distributed as dist


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--layers", type=int, default=16)
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--ffn", type=int, default=1024)
    p.add_argument("--experts", type=int, default=64)
    p.add_argument("--top-k", type=int, default=8)
    p.add_argument("--vocab", type=int, default=32000)
    p.add_argument("--seq-len", type=int, default=2048)
    p.add_argument("--micro-batch", type=int, default=4)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--lr", type=float, default=1e-4)
    p.add_argument("--log-every", type=int, default=1)
    p.add_argument("--seed", type=int, default=0)
    a = p.parse_args(argv)

    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from ..models.gpt_moe import GPTMoE, GPTMoEConfig
    from ..utils.optim import FusedAdamW
    from ..utils.workload import DriftingRouterSkew

    mode = os.environ.get("EPLB_MODE", "apply").strip().lower()
    if mode not in ("off", "apply"):
        raise SystemExit("EPLB_MODE must be off or apply for this entry point")
    home = a.experts // world
    n_slot_total = int(os.environ.get("EPLB_N_SLOT", "0") or 0) or (home + 2)
    extra = 0 if (mode == "off" or world == 1) else max(0, n_slot_total - home)
    gpn = int(os.environ.get("GPUS_PER_NODE", str(world)) or world)
    domains = world // gpn if gpn > 0 and world % gpn == 0 else 1
    cfg = GPTMoEConfig(vocab=a.vocab, layers=a.layers, hidden=a.hidden, heads=a.heads, ffn=a.ffn, experts=a.experts,
                       top_k=a.top_k, seq_len=a.seq_len, micro_batch=a.micro_batch, extra_slots=extra,
                       num_domains=max(domains, 1))
    torch.manual_seed(a.seed)
    model = GPTMoE(cfg, dev, rank=rank, world=world)
    model.sync_dense_parameters()
    dense_opt = torch.optim.AdamW(model.dense_parameters(), lr=a.lr, fused=True)
    expert_opt = FusedAdamW(list(model.expert_parameters()), lr=a.lr)
    skew = DriftingRouterSkew(a.layers, a.experts, rho=0.9, scale=float(os.environ.get("ROUTER_SKEW", "1.0")),
                              seed=a.seed, device=dev)
    n_params = sum(p.numel() for p in model.dense_parameters()) + sum(p.numel() for p in model.expert_parameters()) * world
    if rank == 0:
        print(f"Total number of parameters in billions: {n_params / 1e9:.2f}", flush=True)
        print(f"[ep_balance_b200] mode={mode} world={world} domains={cfg.num_domains} extra_slots={extra}", flush=True)

    gen = torch.Generator(device="cpu").manual_seed(1000 + rank)
    gbs = a.micro_batch * world
    for step in range(1, a.steps + 1):
        ids = torch.randint(0, a.vocab, (a.micro_batch, a.seq_len + 1), generator=gen).to(dev, non_blocking=True)
        model.set_router_bias(skew.step())
        t0 = time.perf_counter()
        loss = model(ids[:, :-1], ids[:, 1:])
        loss.backward()
        model.allreduce_dense_grads()
        gn = torch.nn.utils.clip_grad_norm_(model.dense_parameters(), 1.0)
        dense_opt.step()
        expert_opt.step()
        dense_opt.zero_grad(set_to_none=True)
        if step % a.log_every == 0:
            torch.cuda.synchronize()
            ms = (time.perf_counter() - t0) * 1e3
            lv = loss.detach().clone()
            if world > 1:
                dist.all_reduce(lv)
                lv /= world
            if rank == 0:
                loads = torch.stack([b.moe.rank_loads().float() for b in model.blocks])
                imb = float((loads.max(1).values / loads.mean(1).clamp_min(1)).mean())
                print(f" iteration {step:8d}/{a.steps:8d} | consumed samples: {step * gbs:12d} | "
                      f"elapsed time per iteration (ms): {ms:.1f} | learning rate: {a.lr:.6E} | "
                      f"global batch size: {gbs:5d} | lm loss: {float(lv):.6E} | grad norm: {float(gn):.3f} | "
                      f"rank load max/mean: {imb:.3f} |", flush=True)
    model.check_status()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
