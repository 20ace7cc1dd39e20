"""Common harness: every strategy on the same load matrix (synthetic or replayed from a trace).

    python -m ep_balance_b200.baselines.benchmark --strategies scale,eplb,fastermoe,flexmoe [--json]
    python -m ep_balance_b200.baselines.benchmark --trace trace.pt --strategies scale,eplb

Defaults follow the reference harness (baseline/benchmark.py:800-875): 4x8 ranks, 640 experts,
4 additional replica slots per rank, 4096 tokens per rank, top-8, Zipf 1.5, 25 % hotspot ranks.
``--n-slot`` counts ADDITIONAL replica slots; the solver's ``ProblemSpec.n_slot`` is the total.
"""

from __future__ import annotations

import argparse
import json
import statistics
import time
from typing import Any, Callable, Dict, List, Optional

import torch

from ..core.config import EPLBConfig
from ..core.loads import Loads
from ..core.problem import ProblemSpec
from ..core.topology import Topology
from ..core.trace import load_routing_trace, spec_and_topology_from_meta
from ..solver.api import solve
from ..utils.workload import make_loads
from .adapters import (BaselineResult, LPLBBaseline, LPLBUnavailableError, run_deepseek_eplb, run_fastermoe,
                       run_flexmoe, run_scale_eplb, slot_budget)

KNOWN = ("scale", "eplb", "fastermoe", "flexmoe", "lplb")


def time_cpu(fn: Callable[[], Any], warmup: int, iterations: int) -> float:
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(iterations):
        fn()
    return (time.perf_counter() - t0) * 1e3 / max(iterations, 1)


def time_cuda(fn: Callable[[], Any], warmup: int, iterations: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iterations):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / max(iterations, 1)


def _row(name: str, res: BaselineResult, **timings: Optional[float]) -> Dict[str, Any]:
    return {"strategy": name, "quality_theta": res.theta, "quality_mean_load": res.mean_load,
            "quality_imbalance": res.imbalance, "rank_load_by_rank": [float(v) for v in res.rank_load.tolist()],
            **{k: v for k, v in res.metadata.items() if k != "placement_details"}, **timings}


def no_balance_result(loads: Loads, spec: ProblemSpec, num_ranks: int) -> BaselineResult:
    load = torch.zeros(num_ranks, dtype=torch.float64)
    load.index_add_(0, spec.main_rank.cpu(), loads.expert_load().cpu().double())
    x = torch.zeros((spec.num_experts, num_ranks), dtype=torch.int64)
    x[torch.arange(spec.num_experts), spec.main_rank.cpu()] = 1
    return BaselineResult("no-balance", load, x, {"load_kind": "owner-only load", "replicas": 0})


def placement_details(res: BaselineResult, loads: Loads, spec: ProblemSpec) -> Dict[str, Any]:
    """Per-expert instance counts and the hottest experts' hosts, for ``--details``."""
    if res.placement is None:
        return {}
    x = res.placement.cpu()
    per_e = loads.expert_load().cpu()
    hot = torch.argsort(per_e, descending=True)[:8].tolist()
    return {"instances_per_expert": x.sum(1).tolist(), "slots_per_rank": (x > 0).sum(0).tolist(),
            "hot_experts": [{"expert": e, "load": int(per_e[e]), "main": int(spec.main_rank[e]),
                             "hosts": (x[e] > 0).nonzero().flatten().tolist()} for e in hot]}


def run_strategies(strategies, loads: Loads, history: Loads, topo: Topology, spec: ProblemSpec, *, nodes: int,
                   n_slot: int, num_groups: int, warmup: int, iterations: int, details: bool = False,
                   include_no_balance: bool = False, lplb_topology: str = "auto") -> List[Dict[str, Any]]:
    ranks = topo.num_ranks
    cfg = EPLBConfig()
    rows: List[Dict[str, Any]] = []

    def emit(name, res, **t):
        row = _row(name, res, **t)
        if details:
            row["placement_details"] = placement_details(res, loads, spec)
        rows.append(row)

    if include_no_balance:
        emit("no-balance", no_balance_result(loads, spec, ranks), solve_ms=0.0)
    if "scale" in strategies:
        timer = time_cuda if loads.omega.is_cuda else time_cpu
        ms = timer(lambda: solve(loads, topo, spec, cfg, validate=False), warmup, iterations)
        emit("scale-eplb", run_scale_eplb(loads, topo, spec, cfg), solve_ms=ms, total_ms=ms)
    cpu_loads, cpu_hist, cpu_spec = Loads(loads.omega.cpu()), Loads(history.omega.cpu()), spec.to("cpu")
    if "eplb" in strategies:
        fn = lambda: run_deepseek_eplb(cpu_loads, num_nodes=nodes, num_gpus=ranks, n_slot=n_slot,
                                       num_groups=num_groups, placement_loads=cpu_hist)
        emit("deepseek-eplb", fn(), solve_ms=time_cpu(fn, warmup, iterations))
    if "fastermoe" in strategies:
        fn = lambda: run_fastermoe(cpu_loads, cpu_spec, num_ranks=ranks, n_slot=n_slot)
        emit("fastermoe", fn(), solve_ms=time_cpu(fn, warmup, iterations))
    if "flexmoe" in strategies:
        fn = lambda: run_flexmoe(cpu_loads, cpu_spec, num_ranks=ranks, n_slot=n_slot)
        emit("flexmoe", fn(), solve_ms=time_cpu(fn, warmup, iterations))
    if "lplb" in strategies:
        try:
            base = LPLBBaseline(num_experts=spec.num_experts, num_ranks=ranks, n_slot=n_slot, topology=lplb_topology)
            emit("lplb", base.solve(cpu_loads.omega.float()), solve_ms=None)
        except LPLBUnavailableError as exc:
            rows.append({"strategy": "lplb", "unavailable": str(exc)})
    return rows


def safe_num_groups(num_experts: int, num_nodes: int, requested: int) -> int:
    g = max(1, int(requested))
    while g > 1 and (num_experts % g or g % max(num_nodes, 1)):
        g -= 1
    return g


def benchmark(args) -> List[Dict[str, Any]]:
    strategies = {s.strip().lower() for s in args.strategies.split(",") if s.strip()}
    if strategies - set(KNOWN):
        raise ValueError(f"unknown strategies: {sorted(strategies - set(KNOWN))}")
    ranks = args.nodes * args.gpus_per_node
    _, _, phys = slot_budget(args.experts, ranks, args.n_slot)
    device = torch.device(args.device if args.device != "auto" else ("cuda" if torch.cuda.is_available() else "cpu"))
    loads = make_loads(ranks, args.experts, args.tokens_per_rank, args.top_k, args.skew, args.hotspot_ranks, args.seed, device)
    history = make_loads(ranks, args.experts, args.tokens_per_rank, args.top_k, args.history_skew, args.hotspot_ranks,
                         args.history_seed, device)
    topo = Topology.from_nvlink_rdma(args.nodes, args.gpus_per_node, args.intra_cost, args.inter_cost, device)
    spec = ProblemSpec.uniform_main_placement(args.experts, ranks, args.weight_bytes, args.s_tok, phys, device)
    return run_strategies(strategies, loads, history, topo, spec, nodes=args.nodes, n_slot=args.n_slot,
                          num_groups=safe_num_groups(args.experts, args.nodes, args.num_groups), warmup=args.warmup,
                          iterations=args.iterations, details=args.details,
                          include_no_balance=args.include_no_balance, lplb_topology=args.lplb_topology)


def _agg(values: List[float]) -> Dict[str, float]:
    s = sorted(values)
    q = lambda p: s[min(len(s) - 1, int(p * (len(s) - 1) + 0.5))]
    return {"mean": statistics.fmean(s), "p50": q(0.5), "p90": q(0.9), "max": s[-1], "min": s[0]}


def benchmark_trace(args) -> List[Dict[str, Any]]:
    """Replay every captured omega of a routing trace through every strategy; aggregate per strategy."""
    trace = load_routing_trace(args.trace)
    meta = trace["meta"]
    topo, spec = spec_and_topology_from_meta(meta)
    ranks, E = topo.num_ranks, spec.num_experts
    main = E // ranks
    extra = int(args.replica_slots_per_rank) if args.replica_slots_per_rank is not None else int(spec.n_slot) - main
    spec = ProblemSpec(E, spec.main_rank, spec.weight_bytes, spec.s_tok, main + extra)
    strategies = {s.strip().lower() for s in args.strategies.split(",") if s.strip()}
    samples = trace["samples"][: args.max_samples] if args.max_samples else trace["samples"]
    acc: Dict[str, Dict[str, List[float]]] = {}
    prev = None
    for s in samples:
        loads = Loads(torch.as_tensor(s["omega"], dtype=torch.int64))
        rows = run_strategies(strategies, loads, prev or loads, topo, spec, nodes=topo.num_domains, n_slot=extra,
                              num_groups=safe_num_groups(E, topo.num_domains, args.num_groups), warmup=0, iterations=1,
                              include_no_balance=True)
        prev = loads
        for r in rows:
            if "quality_imbalance" in r:
                a = acc.setdefault(r["strategy"], {"imbalance": [], "theta": [], "solve_ms": []})
                a["imbalance"].append(r["quality_imbalance"])
                a["theta"].append(r["quality_theta"])
                a["solve_ms"].append(float(r.get("solve_ms") or 0.0))
    return [{"strategy": k, "samples": len(v["imbalance"]), "imbalance": _agg(v["imbalance"]), "theta": _agg(v["theta"]),
             "solve_ms": _agg(v["solve_ms"]), "replica_slots_per_rank": extra} for k, v in acc.items()]


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--strategies", default="scale,eplb,fastermoe,flexmoe")
    p.add_argument("--nodes", type=int, default=4)
    p.add_argument("--gpus-per-node", type=int, default=8)
    p.add_argument("--experts", type=int, default=640)
    p.add_argument("--n-slot", type=int, default=4, help="ADDITIONAL replica slots per rank")
    p.add_argument("--tokens-per-rank", type=int, default=4096)
    p.add_argument("--top-k", type=int, default=8)
    p.add_argument("--skew", type=float, default=1.5)
    p.add_argument("--history-skew", type=float, default=1.5)
    p.add_argument("--hotspot-ranks", type=float, default=0.25)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--history-seed", type=int, default=1)
    p.add_argument("--intra-cost", type=int, default=1)
    p.add_argument("--inter-cost", type=int, default=8)
    p.add_argument("--weight-bytes", type=int, default=3 * 2048 * 1408 * 2)
    p.add_argument("--s-tok", type=int, default=2048 * 2)
    p.add_argument("--num-groups", type=int, default=8)
    p.add_argument("--warmup", type=int, default=2)
    p.add_argument("--iterations", type=int, default=10)
    p.add_argument("--device", default="auto")
    p.add_argument("--lplb-topology", default="auto", choices=["auto", "cube", "ring"])
    p.add_argument("--include-no-balance", action="store_true")
    p.add_argument("--details", action="store_true")
    p.add_argument("--json", action="store_true")
    p.add_argument("--trace", default=None, help="replay a routing trace instead of synthetic loads")
    p.add_argument("--max-samples", type=int, default=0)
    p.add_argument("--replica-slots-per-rank", type=int, default=None)
    return p.parse_args(argv)


def main(argv=None) -> List[Dict[str, Any]]:
    args = parse_args(argv)
    rows = benchmark_trace(args) if args.trace else benchmark(args)
    if args.json:
        print(json.dumps(rows))
    elif args.trace:
        for r in rows:
            print(f"{r['strategy']:<14} samples={r['samples']:<4} imbalance mean={r['imbalance']['mean']:.3f} "
                  f"p90={r['imbalance']['p90']:.3f} max={r['imbalance']['max']:.3f} solve_ms p50={r['solve_ms']['p50']:.3f}")
    else:
        for r in rows:
            if "unavailable" in r:
                print(f"{r['strategy']:<14} unavailable: {r['unavailable']}")
                continue
            ms = r.get("solve_ms")
            print(f"{r['strategy']:<14} theta={r['quality_theta']:<10.1f} imbalance={r['quality_imbalance']:.3f} "
                  f"replicas={r.get('replicas', 0):<4} solve_ms={'n/a' if ms is None else f'{ms:.3f}'}")
    return rows


if __name__ == "__main__":
    main()
