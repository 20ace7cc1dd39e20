"""One-shot host simulation: synthetic loads -> plan -> metrics report.

    python -m ep_balance_b200.sim.run_sim --nodes 4 --gpus-per-node 8 --experts 64 --n-slot 4

Reference: sim/run_sim.py:1-105 (``--n-slot`` here is the TOTAL slot count per rank, as there).
"""

from __future__ import annotations

import argparse
import time

from ..core.config import EPLBConfig
from ..core.metrics import check_constraints, compute_metrics
from ..core.plan import Plan
from ..core.problem import ProblemSpec
from ..core.topology import Topology
from ..solver import solve, solve_bisect, solve_device_semantics
from ..utils.workload import make_loads


def run(args) -> dict:
    R = args.nodes * args.gpus_per_node
    loads = make_loads(R, args.experts, args.tokens_per_rank, args.top_k, args.skew, args.hotspot_ranks, args.seed)
    topo = Topology.from_nvlink_rdma(args.nodes, args.gpus_per_node, args.intra_cost, args.inter_cost)
    spec = ProblemSpec.uniform_main_placement(args.experts, R, args.weight_bytes, args.s_tok, args.n_slot)
    cfg = EPLBConfig(u_min=args.u_min)
    fn = {"exact": solve, "device": solve_device_semantics, "bisect": solve_bisect}[args.solver]
    t0 = time.perf_counter()
    plan: Plan = fn(loads, topo, spec, cfg)
    ms = (time.perf_counter() - t0) * 1e3
    import torch

    x0 = torch.zeros_like(plan.x)
    x0[torch.arange(args.experts), spec.main_rank] = 1
    q0 = torch.zeros_like(plan.q)
    q0[:, torch.arange(args.experts), spec.main_rank] = loads.omega
    before = compute_metrics(Plan(x0, q0, int(q0.sum((0, 1)).max())), loads, topo, spec, cfg)
    after = compute_metrics(plan, loads, topo, spec, cfg)
    rep = check_constraints(plan, loads, topo, spec, cfg)
    return {"solve_ms": ms, "before": before, "after": after, "constraints_ok": rep.ok, "violations": rep.violations}


def main(argv=None) -> dict:
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--nodes", type=int, default=4)
    p.add_argument("--gpus-per-node", type=int, default=8)
    p.add_argument("--experts", type=int, default=64)
    p.add_argument("--n-slot", type=int, default=4, help="TOTAL slots per rank, owners included")
    p.add_argument("--tokens-per-rank", type=int, default=4096)
    p.add_argument("--top-k", type=int, default=8)
    p.add_argument("--skew", type=float, default=1.5)
    p.add_argument("--hotspot-ranks", type=float, default=0.25)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--intra-cost", type=int, default=1)
    p.add_argument("--inter-cost", type=int, default=8)
    p.add_argument("--weight-bytes", type=int, default=3 * 2048 * 1408 * 2)
    p.add_argument("--s-tok", type=int, default=4096)
    p.add_argument("--u-min", type=int, default=1)
    p.add_argument("--solver", default="exact", choices=["exact", "device", "bisect"])
    out = run(p.parse_args(argv))
    b, a = out["before"], out["after"]
    print(f"solve: {out['solve_ms']:.1f} ms   constraints: {'OK' if out['constraints_ok'] else out['violations']}")
    print(f"imbalance {b.imbalance:.3f} -> {a.imbalance:.3f}   theta {b.theta} -> {a.theta}   "
          f"replicas {a.total_replicas - b.total_replicas}   phi_token {b.phi_token} -> {a.phi_token}   "
          f"phi_weight {a.phi_weight}")
    return out


if __name__ == "__main__":
    main()
