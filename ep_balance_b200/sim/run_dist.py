"""Multi-rank determinism check: every rank gathers omega, solves, and the plan digests must agree.

    python -m ep_balance_b200.sim.run_dist --world 4                 # spawns gloo ranks on the CPU
    torchrun --nproc-per-node 8 -m ep_balance_b200.sim.run_dist      # NCCL ranks, device solver

Reference: sim/run_dist.py:18-121.
"""

from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ..core.config import EPLBConfig
from ..core.problem import ProblemSpec
from ..core.topology import Topology
from ..parallel.omega import all_gather_omega
from ..solver import solve
from ..utils.workload import make_loads


def worker(rank: int, world: int, args, port: int, results=None) -> bool:
    launched = "RANK" in os.environ and results is None
    if not launched:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
    use_cuda = args.backend == "nccl"
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group(args.backend, rank=rank, world_size=world)
    device = torch.device("cuda") if use_cuda else torch.device("cpu")
    loads = make_loads(world, args.experts, args.tokens_per_rank, args.top_k, args.skew, 0.25, args.seed)
    gpn = args.gpus_per_node if world % args.gpus_per_node == 0 else world
    topo = Topology.from_nvlink_rdma(world // gpn, gpn, device=device)
    spec = ProblemSpec.uniform_main_placement(args.experts, world, args.weight_bytes, args.s_tok, args.n_slot, device)
    gathered = all_gather_omega(loads.omega[rank].to(device))
    plan = solve(gathered, topo, spec, EPLBConfig(), validate=False)
    digests = [None] * world
    dist.all_gather_object(digests, plan.digest())
    same = len(set(digests)) == 1
    if rank == 0:
        print(f"world={world} backend={args.backend} plan digests identical: {same} ({digests[0][:16]}...)")
    dist.barrier()
    dist.destroy_process_group()
    if results is not None:
        results[rank] = same
    return same


def main(argv=None) -> bool:
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--world", type=int, default=4)
    p.add_argument("--backend", default="gloo", choices=["gloo", "nccl"])
    p.add_argument("--experts", type=int, default=64)
    p.add_argument("--n-slot", type=int, default=0, help="TOTAL slots per rank; 0 = experts/world + 2")
    p.add_argument("--gpus-per-node", type=int, default=4)
    p.add_argument("--tokens-per-rank", type=int, default=1024)
    p.add_argument("--top-k", type=int, default=4)
    p.add_argument("--skew", type=float, default=1.5)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--weight-bytes", type=int, default=3 * 512 * 256 * 2)
    p.add_argument("--s-tok", type=int, default=1024)
    p.add_argument("--port", type=int, default=6231)
    args = p.parse_args(argv)
    if "RANK" in os.environ:  # launched by torchrun
        world = int(os.environ["WORLD_SIZE"])
        args.n_slot = args.n_slot or -(-args.experts // world) + 2
        return worker(int(os.environ["RANK"]), world, args, args.port)
    args.n_slot = args.n_slot or -(-args.experts // args.world) + 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(worker, args=(args.world, args, args.port, results), nprocs=args.world, join=True)
        return all(results.values())


if __name__ == "__main__":
    raise SystemExit(0 if main() else 1)
