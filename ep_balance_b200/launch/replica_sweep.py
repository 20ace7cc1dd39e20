"""Replica transport and plan quality of the fused layer over logical-domain layouts and replica-slot budgets.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29531 -m ep_balance_b200.launch.replica_sweep --json sweep.json

For every layout (1 x R, 2 x R/2, 4 x R/4 logical domains) and every number of replica slots per rank, a
fused layer with large experts (default 3 x 7168 x 2048 bf16 = 88 MB each) is built, a Zipf-skewed routing
is drawn, the plan is solved on the device, and the product's own kernels are timed with CUDA events
(max over ranks):

* ``solve_us``   the on-device solver launch (every rank solves the same plan),
* ``pull``       replica weight pull: every host copies its replicas' weights from the owners' slots
                 (bulk async copies, peer loads) -- ``MoeRuntime.pull_weights``,
* ``return``     gradient return: every owner adds its replicas' gradient slots with peer loads
                 -- ``MoeRuntime.reduce_weight_grads``.

GB/s = bytes that cross the busiest NVLink port / time: for the pull that is the larger of what one host receives
and what one owner sends (a hot expert's owner serves all its replicas at once), for the return what one owner
receives; the figure to compare with is the peer-copy bandwidth of one GPU and direction.  Plan quality (rank load max/mean) is printed beside DeepSeek-EPLB's
on the same load matrix; the reference's CUDA solver returns bit-identical plans
(``tests/test_gpu_solver_vs_reference.py``), so its max/mean equals ours.
Reference sweep definition: scripts/run_slot_sweep.sh, scripts/run_solver_scaling.sh.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _timed(fn, iters: int, dev) -> float:
    fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([t0.elapsed_time(t1) / iters], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=2048, help="tokens per rank (only sizes the routing problem)")
    ap.add_argument("--zipf", type=float, default=1.2)
    ap.add_argument("--slots", type=int, nargs="*", default=[0, 1, 2, 4])
    ap.add_argument("--domains", type=int, nargs="*", default=[1, 2, 4])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world < 2:
        print("replica_sweep needs at least two ranks")
        return 0
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from .. import Loads
    from ..baselines.adapters import run_deepseek_eplb
    from ..models.moe_layer import FusedMoE, MoEConfig, heap_layout
    from ..parallel.symm import SymmetricHeap

    E, K, N = a.experts, a.top_k, a.tokens
    per_expert = 3 * a.hidden * a.ffn * 2
    # Zipf popularity over a fixed random permutation of the experts; every rank draws its own tokens
    g = torch.Generator().manual_seed(1234)
    popularity = (1.0 / (torch.arange(E, dtype=torch.float64) + 1) ** a.zipf)[torch.randperm(E, generator=g)]
    gr = torch.Generator().manual_seed(99 + rank)
    idx = torch.multinomial((popularity / popularity.sum()).expand(N, E), K, replacement=False, generator=gr).to(dev)
    rows = []
    for domains in a.domains:
        if world % domains or domains > world:
            continue
        for slots in a.slots:
            cfg = MoEConfig(hidden=a.hidden, ffn=a.ffn, num_experts=E, top_k=K, max_tokens=N, extra_slots=slots,
                            num_domains=domains, capacity_factor=float(world))
            heap = SymmetricHeap(heap_layout(cfg, world), dev)
            layer = FusedMoE(cfg, heap, rank, world)
            rt = layer.rt
            rt.publish(idx.data_ptr(), N * K)
            rt.solve()
            rt.route(idx.data_ptr(), N * K)
            torch.cuda.synchronize()
            dist.barrier()
            layer.check_status()
            plan = layer.last_plan()
            loads = layer.rank_loads().float()
            hosted_here = int(plan.x[:, rank].sum()) - layer.home_cap           # replicas this rank pulls
            served_here = int(plan.x[rank * layer.home_cap:(rank + 1) * layer.home_cap].sum()) - layer.home_cap  # replicas of my experts
            counts = torch.tensor([hosted_here, served_here], device=dev)
            worst = counts.clone()
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            row = {"ranks": world, "domains": f"{domains}x{world // domains}", "slots": slots, "experts": E,
                   "expert_mb": per_expert / 2 ** 20, "replicas": int(plan.x.sum()) - E,
                   "rank_load_max_over_mean": float(loads.max() / loads.mean()),
                   "max_replicas_pulled_by_a_rank": int(worst[0]), "max_replicas_returned_to_an_owner": int(worst[1])}
            row["solve_us"] = _timed(rt.solve, 20, dev) * 1e3
            if slots > 0:
                row["pull_ms"] = _timed(rt.pull_weights, a.iters, dev)
                row["return_ms"] = _timed(rt.reduce_weight_grads, a.iters, dev)
                busiest = max(int(worst[0]), int(worst[1]))
                row["pull_gbs"] = busiest * per_expert / row["pull_ms"] / 1e6 if busiest else 0.0
                row["return_gbs"] = int(worst[1]) * per_expert / row["return_ms"] / 1e6 if worst[1] else 0.0
            torch.cuda.synchronize()
            layer.check_status()
            if rank == 0:
                omega = layer.omega().to(torch.int64).cpu()
                try:
                    ds = run_deepseek_eplb(Loads(omega), num_nodes=domains, num_gpus=world, n_slot=slots,
                                           num_groups=domains if E % domains == 0 else 1)
                    row["deepseek_eplb_max_over_mean"] = float(ds.rank_load.max() / ds.rank_load.mean())
                except Exception as exc:  # the vendored baseline rejects some shapes (e.g. groups that do not divide)
                    row["deepseek_eplb_max_over_mean"] = None
                    row["deepseek_eplb_error"] = str(exc)[:120]
                unbalanced = torch.zeros(world, dtype=torch.float64).index_add_(
                    0, layer.spec.main_rank.cpu(), omega.sum(0).double())
                row["unbalanced_max_over_mean"] = float(unbalanced.max() / unbalanced.mean())
                print(json.dumps(row), flush=True)
                rows.append(row)
            dist.barrier()
            del layer, rt
            heap.close()
            torch.cuda.empty_cache()
    if rank == 0 and a.json:
        with open(a.json, "w") as fh:
            json.dump(rows, fh, indent=1)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
