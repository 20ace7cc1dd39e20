"""Host restatement of the on-device solver, used as its bit-identity oracle.

The device algorithm differs from the serial host solver in two places
(reference: eplb/cuda_solve.py:36-68, eplb/csrc/fast_solver.cu:108-197, 277-643):

* Update Routing is an even, load-blind split: the units of ``(src, e)`` are divided
  over the active hosts in ascending rank id (in-domain hosts when the source's
  domain has any, otherwise all hosts), remainder to the lowest ids.
* Stage 2 runs independently inside each domain for a bounded number of
  iterations, and its quota transfer is a prefix over source ranks.

Everything is integer arithmetic, so this NumPy version and the CUDA kernel in
``ops/csrc/solver.cu`` must agree on every element of ``x``, ``q`` and ``theta``.
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

I64_MAX = np.iinfo(np.int64).max


def _safe_move(have: int, there: int, left: int, u_min: int) -> int:
    upper = min(have, left)
    if upper <= 0:
        return 0
    if upper == have and there + upper >= u_min:
        return upper
    cap = min(upper, max(have - u_min, 0))
    return cap if cap >= (1 if there > 0 else u_min) else 0


def stage1_device(omega, dom, main_rank, W, s_tok, n_slot, D, allow):
    """Per-domain candidate rows (stable descending by benefit) consumed in order."""
    R, E = omega.shape
    x = np.zeros((E, R), dtype=np.int8)
    x[np.arange(E), main_rank] = 1
    slot_used = x.sum(0).astype(np.int64)
    if not allow or D == 0:
        return x, slot_used
    T = np.zeros((D, E), dtype=np.int64)
    np.add.at(T, dom, omega)
    rhs = 2 * T * int(s_tok)
    valid = (np.arange(D)[:, None] != dom[main_rank][None, :]) & (T > 0) & (W[None, :] < rhs)
    prio = np.where(valid, rhs - W[None, :], -1)
    for d in range(D):
        ranks = np.nonzero(dom == d)[0]
        for e in np.argsort(-prio[d], kind="stable"):
            if not valid[d, e]:
                break
            if ranks.size == 0 or x[e, ranks].any():
                continue
            free = ranks[slot_used[ranks] < n_slot]
            if free.size == 0:
                continue
            pick = int(free[np.lexsort((free, slot_used[free]))[0]])
            x[e, pick] = 1
            slot_used[pick] += 1
    return x, slot_used


def even_split_routing(omega, x, dom, u_min):
    R, E = omega.shape
    q = np.zeros((R, E, R), dtype=np.int64)
    for e in range(E):
        hosts = np.nonzero(x[e])[0]
        for src in range(R):
            need = int(omega[src, e])
            if need <= 0 or hosts.size == 0:
                continue
            inside = hosts[dom[hosts] == dom[src]]
            act = inside if inside.size else hosts
            n = act.size
            if u_min > 1 and need >= u_min:
                n = min(n, need // u_min)
            elif need < u_min:
                n = 1
            base, rem = divmod(need, n)
            q[src, e, act[:n]] = base + (np.arange(n) < rem)
    return q


def stage2_domain(d, x, q, erl, load, slot_used, stuck, dom, cost, n_slot, u_min, iters):
    """Greedy repair of one domain, in place.  ``load/slot_used/stuck`` are global arrays."""
    ranks = np.nonzero(dom == d)[0]
    if ranks.size == 0:
        return
    stuck[ranks] = False
    for _ in range(iters):
        cand = ranks[~stuck[ranks]]
        if cand.size == 0:
            break
        top = int(load[cand].max())
        if top <= 0:
            break
        src = int(cand[load[cand] == top][0])
        tg = ranks[(ranks != src) & (load[ranks] < top)]
        best = None
        if tg.size:
            avail = erl[:, src]
            half = (top - load[tg]) // 2
            delta = np.minimum(avail[:, None], half[None, :])
            legal = (avail[:, None] > 0) & ((x[:, tg] != 0) | (slot_used[tg] < n_slot)[None, :]) & (delta >= u_min)
            if legal.any():
                bd = delta[legal].max()
                m = legal & (delta == bd)
                tl = np.where(m, load[tg][None, :], I64_MAX)
                m &= tl == tl.min()
                tc = np.where(m, cost[src, tg][None, :], I64_MAX)
                m &= tc == tc.min()
                e = int(np.nonzero(m.any(1))[0][0])
                t = int(tg[np.nonzero(m[e])[0][0]])
                best = (e, t, int(bd))
        if best is None or best[2] <= 0:
            stuck[src] = True
            continue
        e, t, delta = best
        if u_min == 1:
            if x[e, t] == 0:
                x[e, t] = 1
                slot_used[t] += 1
            col = q[:, e, src].copy()
            before = np.cumsum(col) - col
            mv = np.minimum(col, np.maximum(delta - before, 0))
            q[:, e, src] -= mv
            q[:, e, t] += mv
            moved = delta
        else:
            def dry(limit):
                left, tot = limit, 0
                for s in range(q.shape[0]):
                    m_ = _safe_move(int(q[s, e, src]), int(q[s, e, t]), left, u_min)
                    left -= m_
                    tot += m_
                return tot
            limit = delta
            moved = dry(limit)
            if moved < u_min:
                limit = top - int(load[t]) - 1
                moved = dry(limit)
            if moved < u_min:
                stuck[src] = True
                continue
            if x[e, t] == 0:
                x[e, t] = 1
                slot_used[t] += 1
            left = limit
            for s in range(q.shape[0]):
                m_ = _safe_move(int(q[s, e, src]), int(q[s, e, t]), left, u_min)
                q[s, e, src] -= m_
                q[s, e, t] += m_
                left -= m_
        erl[e, src] -= moved
        erl[e, t] += moved
        load[src] -= moved
        load[t] += moved
        stuck[ranks] = False


def _np(t):
    return t.detach().to("cpu", torch.int64).contiguous().numpy()


def solve_device_semantics(loads: Loads, topo: Topology, spec: ProblemSpec,
                           cfg: Optional[EPLBConfig] = None) -> Plan:
    """Plan the CUDA solver must reproduce bit for bit (probe mode excluded)."""
    cfg = cfg or EPLBConfig()
    device = loads.device
    omega, dom, cost = _np(loads.omega), _np(topo.domain_of_rank), _np(topo.cost)
    main_rank, W = _np(spec.main_rank), _np(spec.weight_bytes)
    R, E = omega.shape
    D = topo.sync_free_num_domains
    n_slot, u_min = int(spec.n_slot), int(cfg.u_min)

    x, slot_used = stage1_device(omega, dom, main_rank, W, int(spec.s_tok), n_slot, D,
                                 bool(cfg.allow_cross_domain))
    q = even_split_routing(omega, x, dom, u_min)
    erl = q.sum(0)
    load = erl.sum(0)
    stuck = np.zeros(R, dtype=bool)
    for d in range(D):
        stage2_domain(d, x, q, erl, load, slot_used, stuck, dom, cost, n_slot, u_min,
                      cfg.device_stage2_iters)
    theta = int(load.max()) if R else 0
    return Plan(x=torch.from_numpy(x).to(device), q=torch.from_numpy(q).to(device), theta=theta)
