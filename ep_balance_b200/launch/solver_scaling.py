"""Solver latency driver: device time of one plan solve over a grid of shapes.

    python -m ep_balance_b200.launch.solver_scaling --json out.json            # full sweeps
    python -m ep_balance_b200.launch.solver_scaling --ranks 8 --experts 64 --domains 2 --extra-slots 2

All logical ranks are simulated on one GPU (the solver is replicated, not distributed).  Timing is
reported twice: ``min_us`` / ``median_us`` are API-level (CUDA events around ``iters`` back-to-back
``solve()`` calls, so tensor allocation, dtype casts and Python dispatch count), ``kernel_min_us`` /
``kernel_median_us`` are the solver kernels alone, one event pair per call.  ``--impl reference`` times the
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


def _time_each(fn, before, warmup: int, iters: int) -> Dict[str, float]:
    """Per-launch device time: an event pair around every call, state reset outside the pair."""
    for _ in range(warmup):
        before()
        fn()
    torch.cuda.synchronize()
    pairs = []
    for _ in range(iters):
        before()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        pairs.append((a, b))
    torch.cuda.synchronize()
    us = sorted(a.elapsed_time(b) * 1e3 for a, b in pairs)
    return {"kernel_min_us": us[0], "kernel_median_us": us[len(us) // 2]}


def kernel_only(ranks: int, experts: int, domains: int, extra: int, skew: float, impl: str, warmup: int,
                iters: int) -> Dict[str, float]:
    """Solver kernels alone (no tensor allocation, casts or Python-side preparation in the timed span).

    Ours: the single cooperative launch behind ``ext.solve_plan``.  Reference: its three-kernel
    ``backend.fast_solve`` call on candidate arrays prepared beforehand, with its accumulators and
    placement reset before every call outside the timed span (the method of its own perf driver,
    tests/test_gpu_solver.py:407-435)."""
    from ..utils.workload import make_loads

    dev = torch.device("cuda")
    omega = make_loads(ranks, experts, 4096, 8, skew, 0.25, 0).omega.to(dev)
    n_slot = -(-experts // ranks) + extra
    wb, s_tok = 3 * 7168 * 2048 * 2, 7168 * 2
    if impl == "reference":
        import eplb
        from eplb import cuda_solve as cs

        topo = eplb.Topology.from_nvlink_rdma(domains, ranks // domains, device=dev)
        spec = eplb.ProblemSpec.uniform_main_placement(experts, ranks, wb, s_tok, n_slot, device=dev)
        loads, cfg = eplb.Loads(omega), eplb.EPLBConfig()
        backend = cs._get_backend()
        om = loads.omega.to(torch.int64).contiguous()
        dom = topo.domain_of_rank.to(torch.int64).contiguous()
        cost = topo.cost.to(torch.int64).contiguous()
        x0 = torch.zeros((experts, ranks), dtype=torch.int8, device=dev)
        x0.scatter_(1, spec.main_rank.view(experts, 1), 1)
        su0 = x0.sum(0).to(torch.int64)
        ce, cd, cv = cs._stage1_candidates(loads, topo, spec)
        x, su = x0.clone(), su0.clone()
        q = torch.zeros((ranks, experts, ranks), dtype=torch.int64, device=dev)
        erl = torch.zeros((experts, ranks), dtype=torch.int64, device=dev)
        rl = torch.zeros(ranks, dtype=torch.int64, device=dev)
        stuck = torch.zeros(ranks, dtype=torch.uint8, device=dev)
        ctl = torch.zeros(3, dtype=torch.int64, device=dev)

        def before():
            x.copy_(x0)
            su.copy_(su0)
            erl.zero_()
            rl.zero_()
            stuck.zero_()

        fn = lambda: backend.fast_solve(om, x, cost, dom, q, erl, ce, cd, cv, su, rl, stuck, ctl, int(domains),
                                        int(n_slot), 64, 8, False, 1, True)
        return _time_each(fn, before, warmup, iters)
    from .. import EPLBConfig, ProblemSpec, Topology
    from ..ops.extension import load
    from ..ops.solver_op import _static_inputs, workspace

    ext = load()
    topo = Topology.from_nvlink_rdma(domains, ranks // domains)
    spec = ProblemSpec.uniform_main_placement(experts, ranks, wb, s_tok, n_slot)
    d, c, m, w = _static_inputs(topo, spec, dev)
    ws = workspace(ranks, experts, dev)
    om = omega.to(torch.int32).contiguous()
    x = torch.empty((experts, ranks), dtype=torch.int8, device=dev)
    q = torch.empty((ranks, experts, ranks), dtype=torch.int32, device=dev)
    theta = torch.empty(1, dtype=torch.int64, device=dev)
    fn = lambda: ext.solve_plan(om, d, c, m, w, s_tok, domains, n_slot, 1, 64, 8, True, False, x, q, ws.erl,
                                ws.rank_load, ws.slot_used, ws.stuck, theta, ws.control, ws.sync, ws.status)
    return _time_each(fn, lambda: None, warmup, iters)


def measure(ranks: int, experts: int, domains: int, extra: int, skew: float, impl: str, warmup: int, iters: int,
            repeats: int) -> Dict[str, Any]:
    from ..utils.workload import make_loads

    dev = torch.device("cuda")
    omega = make_loads(ranks, experts, 4096, 8, skew, 0.25, 0).omega.to(dev)
    n_slot = -(-experts // ranks) + extra
    wb, s_tok = 3 * 7168 * 2048 * 2, 7168 * 2
    if impl == "reference":
        from ..baselines.reference_install import use_reference

        repo_root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        if use_reference(repo_root) is None:
            raise SystemExit("the reference is not installed under baseline/_ref")
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
    t.update(kernel_only(ranks, experts, domains, extra, skew, impl, warmup, iters))
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
