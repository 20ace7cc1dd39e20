"""theta-bisection heuristic (host only).

A different search than :func:`solve_exact`: after Stage 0/1 it repeatedly routes,
picks a target half-way between the current max load and the even-split lower
bound, and proposes intra-domain replicas of the hottest expert on every rank
above the target (reference: eplb/algorithm.py:390-576).  Returns the best routed
placement seen.  Not bit-comparable with the other solvers.
"""

from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..core.config import EPLBConfig
from ..core.loads import Loads
from ..core.plan import Plan
from ..core.problem import ProblemSpec
from ..core.topology import Topology
from .exact import _as_np, stage1_placement, update_routing, waterfill


def _propose(load, contrib, x, slot_used, dom, cost, n_slot, u_min, target):
    R = len(load)
    load = list(load)
    cell = [{int(e): int(contrib[e, r]) for e in np.nonzero(contrib[:, r] > 0)[0]} for r in range(R)]
    hosts = {}
    for e, r in zip(*np.nonzero(x)):
        hosts.setdefault(int(e), set()).add(int(r))
    used = list(slot_used)
    stuck, added = set(), []
    while True:
        over = [r for r in range(R) if load[r] > target and r not in stuck]
        if not over:
            return added
        src = min(over, key=lambda r: (-load[r], r))
        mine = cell[src]
        top = max(mine.values()) if mine else 0
        if top == 0:
            stuck.add(src)
            continue
        e = min(k for k, v in mine.items() if v == top)
        he = hosts.get(e, set())
        d = dom[src]
        elig = [t for t in range(R) if dom[t] == d and used[t] < n_slot and t not in he]
        if not elig:
            stuck.add(src)
            continue
        t = min(elig, key=lambda t_: (load[t_], int(cost[src, t_]), t_))
        group = sorted(h for h in he if dom[h] == d) + [t]
        base = [load[h] - cell[h].get(e, 0) for h in group]
        pool = sum(cell[h].get(e, 0) for h in group)
        for h, a, b in zip(group, waterfill(pool, base, [0] * len(group), u_min), base):
            load[h] = b + a
            cell[h][e] = a
        hosts.setdefault(e, set()).add(t)
        used[t] += 1
        added.append((e, t))
        stuck = set()


def solve_bisect(loads: Loads, topo: Topology, spec: ProblemSpec, cfg: Optional[EPLBConfig] = None) -> Plan:
    cfg = cfg or EPLBConfig()
    device = loads.device
    R, E = topo.num_ranks, spec.num_experts
    if R == 0 or E == 0:
        return Plan(torch.zeros((E, R), dtype=torch.int8, device=device),
                    torch.zeros((R, E, R), dtype=torch.int64, device=device), 0)
    omega, dom, cost = _as_np(loads.omega), _as_np(topo.domain_of_rank), _as_np(topo.cost)
    n_slot, u_min = int(spec.n_slot), int(cfg.u_min)
    x, used = stage1_placement(omega, dom, _as_np(spec.main_rank), _as_np(spec.weight_bytes),
                               int(spec.s_tok), n_slot, topo.num_domains, bool(cfg.allow_cross_domain))
    lower = -(-int(omega.sum()) // R)
    best_x = x.copy()
    best_q, best_load = update_routing(omega, best_x, cost, dom, u_min)
    best_theta = int(best_load.max())
    for _ in range(int(cfg.theta_bisect_iters)):
        q, load = update_routing(omega, x, cost, dom, u_min)
        theta = int(load.max())
        if theta < best_theta:
            best_theta, best_x, best_q = theta, x.copy(), q
        if theta <= lower:
            break
        added = _propose(load.tolist(), q.sum(0), x, used.tolist(), dom.tolist(), cost, n_slot, u_min,
                         (lower + theta) // 2)
        if not added:
            break
        for e, t in added:
            x[e, t] = 1
            used[t] += 1
    return Plan(torch.from_numpy(best_x).to(device), torch.from_numpy(best_q).to(device), best_theta)
