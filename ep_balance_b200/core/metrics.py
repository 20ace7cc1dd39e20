"""Plan quality numbers and the C1-C7 feasibility check.

Reference: eplb/metrics.py:17-158.  The constraint check here is vectorised
(one pass of tensor ops) instead of per-expert Python loops, and reports the
same violation classes:

C1 conservation   sum_dst q[r,e,dst] == omega[r,e]
C2 reachability   q[r,e,dst] > 0 only where x[e,dst] == 1
C3 theta          plan.theta == max_dst sum_{r,e} q[r,e,dst]
C4 slot budget    sum_e x[e,r] <= n_slot
C5 granularity    q == 0 or q >= u_min
C6 gate           a cross-domain instance needs |W_e| < 2 * T[dom(r), e] * s_tok
C7 owner fixed    x[e, main(e)] == 1
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

from .config import EPLBConfig
from .loads import Loads
from .plan import Plan
from .problem import ProblemSpec
from .topology import Topology


@dataclass
class Metrics:
    theta: int
    mean_load: float
    imbalance: float
    phi_token: int
    phi_weight: int
    objective: int
    total_replicas: int
    max_slots_used: int


def compute_metrics(plan: Plan, loads: Loads, topo: Topology, spec: ProblemSpec,
                    cfg: Optional[EPLBConfig] = None) -> Metrics:
    cfg = cfg or EPLBConfig()
    R = topo.num_ranks
    q = plan.q.to(torch.int64)
    load = q.sum((0, 1))
    theta = int(load.max()) if R else 0
    total = int(loads.omega.sum())
    mean = total / R if R else 0.0
    # token movement: every unit from src to dst pays cost[src, dst]
    phi_token = int((q.sum(1) * topo.cost).sum())
    # weight movement: each non-owner instance pays the round trip owner -> host -> owner
    x = plan.x.to(torch.int64).clone()
    ar = torch.arange(spec.num_experts, device=x.device)
    x[ar, spec.main_rank] = 0
    phi_weight = int((2 * topo.cost[spec.main_rank] * spec.weight_bytes[:, None] * x).sum())
    return Metrics(
        theta=theta,
        mean_load=mean,
        imbalance=(theta / mean) if mean > 0 else 1.0,
        phi_token=phi_token,
        phi_weight=phi_weight,
        objective=cfg.alpha * theta + cfg.beta * phi_token + cfg.gamma * phi_weight,
        total_replicas=int(plan.x.sum()),
        max_slots_used=int(plan.x.sum(0).max()) if R else 0,
    )


@dataclass
class ConstraintReport:
    ok: bool
    violations: List[str] = field(default_factory=list)

    def __bool__(self) -> bool:
        return self.ok


def check_constraints(plan: Plan, loads: Loads, topo: Topology, spec: ProblemSpec,
                      cfg: Optional[EPLBConfig] = None) -> ConstraintReport:
    cfg = cfg or EPLBConfig()
    bad: List[str] = []
    omega = loads.omega
    x = plan.x
    q = plan.q.to(torch.int64)
    E = spec.num_experts
    dom = topo.domain_of_rank
    n_slot = int(spec.n_slot)

    served = q.sum(2)
    if not torch.equal(served, omega):
        bad.append(f"C1 conservation violated for {int((served != omega).sum())} (r,e) pairs")

    if bool(((q != 0) & (x == 0)[None]).any()):
        bad.append("C2 reachability violated: quota routed to a rank without an instance")

    load_max = int(q.sum((0, 1)).max()) if q.numel() else 0
    if load_max != int(plan.theta):
        bad.append(f"C3/theta mismatch: plan.theta={int(plan.theta)} but max rank load={load_max}")

    slots = x.sum(0)
    if bool((slots > n_slot).any()):
        bad.append(f"C4 slot budget violated: a rank uses {int(slots.max())} > N_slot={n_slot}")

    if cfg.u_min > 1:
        pos = q[q > 0]
        if pos.numel() and int(pos.min()) < cfg.u_min:
            bad.append(f"C5 granularity violated: a nonzero quota < u_min={cfg.u_min}")

    demand = loads.domain_demand(dom, topo.num_domains)  # [M, E]
    main_dom = dom[spec.main_rank]  # [E]
    foreign = (x == 1) & (dom[None, :] != main_dom[:, None])  # [E, R]
    gate_rhs = 2 * demand.t()[:, dom] * int(spec.s_tok)  # [E, R]: 2*T[dom(r), e]*s_tok
    broken = foreign & ~(spec.weight_bytes[:, None] < gate_rhs)
    for e, r in broken.nonzero(as_tuple=False).tolist():
        bad.append(
            f"C6 violated: cross-domain replica e={e} on rank {r} "
            f"(|W_e|={int(spec.weight_bytes[e])} !< 2*T[d,e]*s_tok={int(gate_rhs[e, r])})")

    if E and not bool((x[torch.arange(E, device=x.device), spec.main_rank] == 1).all()):
        bad.append("C7 violated: some main instance is not present")

    return ConstraintReport(ok=not bad, violations=bad)
