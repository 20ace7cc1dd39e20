"""Solver latency driver: device time of one plan solve over a grid of shapes.

    python -m ep_balance_b200.launch.solver_scaling --json out.json            # full sweeps
    python -m ep_balance_b200.launch.solver_scaling --ranks 8 --experts 64 --domains 2 --extra-slots 2

All logical ranks are simulated on one GPU (the solver is replicated, not distributed).  Timing is
kernel-only: CUDA events around ``iters`` back-to-back solves after ``warmup`` solves; ``min_us`` is
the smallest single-solve time over ``repeats`` such batches.  ``--impl reference`` times the
upstream CUDA solver from ``baseline/_ref`` the same way.  Reference driver:
tests/test_gpu_solver.py:287-679, scripts/run_solver_scaling.sh:10-22.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Any, Dict, List

import torch


def _time(fn, warmup: int, iters: int, repeats: int) -> Dict[str, float]:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    per = []
    for _ in range(repeats):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        per.append(a.elapsed_time(b) * 1e3 / iters)
    per.sort()
    return {"min_us": per[0], "median_us": per[len(per) // 2]}


def measure(ranks: int, experts: int, domains: int, extra: int, skew: float, impl: str, warmup: int, iters: int,
            repeats: int) -> Dict[str, Any]:
    from ..utils.workload import make_loads

    dev = torch.device("cuda")
    omega = make_loads(ranks, experts, 4096, 8, skew, 0.25, 0).omega.to(dev)
    n_slot = -(-experts // ranks) + extra
    wb, s_tok = 3 * 7168 * 2048 * 2, 7168 * 2
    if impl == "reference":
        root = "/root/repo/baseline/_ref" if os.path.isdir("/root/repo/baseline/_ref/eplb") else os.path.join(
            os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "baseline", "_ref")
        os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(root, "_torch_ext"))
        os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0+PTX")
        if root not in sys.path:
            sys.path.insert(0, root)
        import eplb

        topo = eplb.Topology.from_nvlink_rdma(domains, ranks // domains, device=dev)
        spec = eplb.ProblemSpec.uniform_main_placement(experts, ranks, wb, s_tok, n_slot, device=dev)
        loads, cfg = eplb.Loads(omega), eplb.EPLBConfig()
        fn = lambda: eplb.solve(loads, topo, spec, cfg, validate=False)
        plan = fn()
    else:
        from .. import EPLBConfig, Loads, ProblemSpec, Topology, solve

        topo = Topology.from_nvlink_rdma(domains, ranks // domains)
        spec = ProblemSpec.uniform_main_placement(experts, ranks, wb, s_tok, n_slot)
        loads, cfg = Loads(omega), EPLBConfig()
        fn = lambda: solve(loads, topo, spec, cfg, validate=False)
        plan = fn()
    t = _time(fn, warmup, iters, repeats)
    load = plan.q.sum((0, 1)).double()
    return {"impl": impl, "ranks": ranks, "experts": experts, "domains": domains, "extra_slots": extra, "skew": skew,
            "imbalance": float(load.max() / load.mean()), "replicas": int(plan.x.sum()) - experts, **t}


def main(argv=None) -> List[Dict[str, Any]]:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--ranks", type=int, default=0)
    p.add_argument("--experts", type=int, default=0)
    p.add_argument("--domains", type=int, default=0)
    p.add_argument("--extra-slots", type=int, default=2)
    p.add_argument("--skew", type=float, default=1.2)
    p.add_argument("--warmup", type=int, default=20)
    p.add_argument("--iters", type=int, default=50)
    p.add_argument("--repeats", type=int, default=4)
    p.add_argument("--grid", default="headline", choices=["headline", "scaling"],
                   help="headline: 8 ranks x E {64..512} x domains {1,2,4} x slots {0,1,2,4}; scaling: R and E sweeps")
    p.add_argument("--json", default=None)
    a = p.parse_args(argv)
    rows: List[Dict[str, Any]] = []
    kw = dict(impl=a.impl, warmup=a.warmup, iters=a.iters, repeats=a.repeats)
    if a.ranks and a.experts:
        rows.append(measure(a.ranks, a.experts, a.domains or 1, a.extra_slots, a.skew, **kw))
    elif a.grid == "headline":
        for E in (64, 128, 256, 512):
            for d in (1, 2, 4):
                for slots in (0, 1, 2, 4):
                    rows.append(measure(8, E, d, slots, a.skew, **kw))
    else:
        for R in (8, 16, 32, 64, 128):
            rows.append({"sweep": "ranks", "x": R, **measure(R, 640, max(1, R // 8), 2, 1.5, **kw)})
        for E in (64, 128, 256, 512, 1024):
            rows.append({"sweep": "experts", "x": E, **measure(32, E, 4, 2, 1.5, **kw)})
    for r in rows:
        print(json.dumps(r), flush=True)
    if a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f)
    return rows


if __name__ == "__main__":
    main()
