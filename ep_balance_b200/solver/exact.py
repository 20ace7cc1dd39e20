"""Serial host solver: load-aware LPT routing + global greedy repair.

This is the semantics the reference uses for CPU tensors (eplb/algorithm.py:191-387):

* Stage 1 admits one instance of expert ``e`` into a foreign domain ``d`` when
  ``W[e] < 2*T[d,e]*s_tok``, walking candidates by (benefit desc, e asc, d asc) and
  picking the domain rank with the fewest used slots.
* Update Routing visits ``(r, e)`` pairs by (omega desc, e asc, r asc) and
  water-fills each pair's units over the in-domain hosts (all hosts when the
  domain has none) on top of the running rank load.
* Stage 2 repeatedly takes the busiest non-stuck rank and moves part of one
  expert's quota to a less loaded rank of the same domain, adding an instance
  there when a slot is free.

The implementation below works on NumPy int64 arrays with vectorised candidate
search; it makes the same decision at every step, so plans compare bit-equal to
the reference's on identical inputs.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np
import torch

from ..core.config import EPLBConfig
from ..core.loads import Loads
from ..core.plan import Plan
from ..core.problem import ProblemSpec
from ..core.topology import Topology


# ------------------------------------------------------------------ helpers

def waterfill(need: int, base: List[int], tie: List[int], u_min: int = 1) -> List[int]:
    """Split ``need`` units over destinations so that max(base+add) is minimal.

    Destinations are ranked by (base, tie, index).  With ``u_min > 1`` only as many
    destinations as can each receive ``u_min`` are activated.
    """
    n = len(base)
    add = [0] * n
    if need <= 0 or n == 0:
        return add
    if n == 1:
        add[0] = int(need)
        return add
    order = sorted(range(n), key=lambda i: (base[i], tie[i], i))
    if u_min > 1 and need >= u_min:
        count = min(n, need // u_min)
        chosen = order[:count]
        for i in chosen:
            add[i] = u_min
        rest = need - count * u_min
        if rest > 0:
            more = waterfill(rest, [base[i] + u_min for i in chosen], [tie[i] for i in chosen], 1)
            for i, m in zip(chosen, more):
                add[i] += m
        return add
    b = [base[i] for i in order]
    prefix = b[0]
    k = 1
    while k < n:
        if b[k] * k - prefix > need:
            break
        prefix += b[k]
        k += 1
    floor = b[k - 1]
    left = need - (floor * k - prefix)
    share, extra = divmod(left, k)
    for pos in range(k):
        add[order[pos]] = floor - b[pos] + share + (1 if pos < extra else 0)
    return add


def plan_quota_transfer(q_from: np.ndarray, q_to: np.ndarray, limit: int, u_min: int) -> Tuple[np.ndarray, int]:
    """Move up to ``limit`` units source by source without leaving a fragment below ``u_min``."""
    moves = np.zeros_like(q_from)
    left = int(limit)
    if left <= 0:
        return moves, 0
    for s in range(q_from.shape[0]):
        if left <= 0:
            break
        have, there = int(q_from[s]), int(q_to[s])
        upper = min(have, left)
        if upper <= 0:
            continue
        mv = 0
        if upper == have and there + upper >= u_min:
            mv = upper
        else:
            cap = min(upper, have - u_min)
            if cap >= (1 if there > 0 else u_min):
                mv = cap
        if mv > 0:
            moves[s] = mv
            left -= mv
    return moves, int(moves.sum())


def stage1_placement(omega: np.ndarray, dom: np.ndarray, main_rank: np.ndarray, W: np.ndarray,
                     s_tok: int, n_slot: int, M: int, allow: bool) -> Tuple[np.ndarray, np.ndarray]:
    """Owners plus gate-admitted cross-domain instances.  Returns ``(x[E,R], slot_used[R])``."""
    R, E = omega.shape
    x = np.zeros((E, R), dtype=np.int8)
    x[np.arange(E), main_rank] = 1
    slot_used = x.sum(0).astype(np.int64)
    if not allow or M <= 1:
        return x, slot_used
    T = np.zeros((M, E), dtype=np.int64)
    np.add.at(T, dom, omega)
    main_dom = dom[main_rank]
    rhs = 2 * T * int(s_tok)  # [M, E]
    ok = (np.arange(M)[:, None] != main_dom[None, :]) & (T > 0) & (W[None, :] < rhs)
    dd, ee = np.nonzero(ok)
    if dd.size == 0:
        return x, slot_used
    benefit = rhs[dd, ee] - W[ee]
    for i in np.lexsort((dd, ee, -benefit)):
        e, d = int(ee[i]), int(dd[i])
        ranks = np.nonzero(dom == d)[0]
        if x[e, ranks].any():
            continue
        free = ranks[slot_used[ranks] < n_slot]
        if free.size == 0:
            continue
        pick = int(free[np.lexsort((free, slot_used[free]))[0]])
        x[e, pick] = 1
        slot_used[pick] += 1
    return x, slot_used


def update_routing(omega: np.ndarray, x: np.ndarray, cost: np.ndarray, dom: np.ndarray,
                   u_min: int = 1) -> Tuple[np.ndarray, np.ndarray]:
    """Full quota construction; returns ``(q[R,E,R], load[R])``."""
    R, E = omega.shape
    q = np.zeros((R, E, R), dtype=np.int64)
    load = [0] * R
    flat = omega.reshape(-1)
    rr, ee = np.divmod(np.arange(R * E), E)
    hosts = [np.nonzero(x[e])[0] for e in range(E)]
    hosts_in = {}
    for i in np.lexsort((rr, ee, -flat)):
        need = int(flat[i])
        if need == 0:
            break  # sorted descending: the rest are zero too
        r, e = int(rr[i]), int(ee[i])
        key = (e, int(dom[r]))
        dests = hosts_in.get(key)
        if dests is None:
            inside = hosts[e][dom[hosts[e]] == dom[r]]
            dests = (inside if inside.size else hosts[e]).tolist()
            hosts_in[key] = dests
        add = waterfill(need, [load[t] for t in dests], [int(cost[r, t]) for t in dests], u_min)
        for t, a in zip(dests, add):
            if a:
                q[r, e, t] += a
                load[t] += a
    return q, np.asarray(load, dtype=np.int64)


# ------------------------------------------------------------------ solve

def _as_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().to("cpu", torch.int64).contiguous().numpy()


def solve_exact(loads: Loads, topo: Topology, spec: ProblemSpec, cfg: Optional[EPLBConfig] = None) -> Plan:
    cfg = cfg or EPLBConfig()
    device = loads.device
    omega, dom, cost = _as_np(loads.omega), _as_np(topo.domain_of_rank), _as_np(topo.cost)
    main_rank, W = _as_np(spec.main_rank), _as_np(spec.weight_bytes)
    R, E = omega.shape
    n_slot, u_min = int(spec.n_slot), int(cfg.u_min)
    M = topo.num_domains

    x, slot_used = stage1_placement(omega, dom, main_rank, W, int(spec.s_tok), n_slot, M,
                                    bool(cfg.allow_cross_domain))
    q, load = update_routing(omega, x, cost, dom, u_min)
    contrib = q.sum(0)  # [E, R]
    stuck = np.zeros(R, dtype=bool)
    e_ids = np.arange(E)

    it = 0
    while it < cfg.max_stage2_iters and R > 0:
        it += 1
        masked = np.where(stuck, -1, load)
        top = int(masked.max())
        if top <= 0:
            break
        src = int(np.nonzero(masked == top)[0][0])
        tg = np.nonzero((dom == dom[src]) & (load < top))[0]
        choice = None
        if tg.size:
            avail = contrib[:, src]  # [E]
            half = (top - load[tg]) // 2  # [T]
            desired = np.minimum(avail[:, None], half[None, :])  # [E, T]
            legal = (avail[:, None] > 0) & ((x[:, tg] != 0) | (slot_used[tg] < n_slot)[None, :]) & (desired >= u_min)
            if legal.any():
                best = desired[legal].max()
                m = legal & (desired == best)
                # prefer emptier target, then cheaper link, then lower expert id, then lower rank id
                tl = np.where(m, load[tg][None, :], np.iinfo(np.int64).max)
                m &= tl == tl.min()
                tc = np.where(m, cost[src, tg][None, :], np.iinfo(np.int64).max)
                m &= tc == tc.min()
                e_star = int(e_ids[m.any(1)][0])
                t_star = int(tg[np.nonzero(m[e_star])[0][0]])
                choice = (e_star, t_star, int(best))
        if choice is None:
            stuck[src] = True
            if stuck.all():
                break
            continue
        e_star, t_star, want = choice
        moves, moved = plan_quota_transfer(q[:, e_star, src], q[:, e_star, t_star], want, u_min)
        if moved < u_min:
            moves, moved = plan_quota_transfer(q[:, e_star, src], q[:, e_star, t_star],
                                               top - int(load[t_star]) - 1, u_min)
        if moved < u_min:
            stuck[src] = True
            if stuck.all():
                break
            continue
        if x[e_star, t_star] == 0:
            x[e_star, t_star] = 1
            slot_used[t_star] += 1
        q[:, e_star, src] -= moves
        q[:, e_star, t_star] += moves
        contrib[e_star, src] -= moved
        contrib[e_star, t_star] += moved
        load[src] -= moved
        load[t_star] += moved
        stuck[dom == dom[src]] = False

    theta = int(load.max()) if R else 0
    return Plan(x=torch.from_numpy(x).to(device), q=torch.from_numpy(q).to(device), theta=theta)
