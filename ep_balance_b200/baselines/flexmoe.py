"""FlexMoE dynamic device placement (SIGMOD'23, Algorithms 1-2) as a placement baseline.

Experts are managed as vExperts: expert ``e`` holds ``n_e`` of them, each carrying
``I_e / n_e`` tokens.  While the balance ratio ``max/mean`` is above the trigger and replica slots
remain, the expert with the largest per-vExpert load is expanded if the cost model predicts a win;
vExperts are then packed onto ranks heaviest first.  Reference port: baseline/flexmoe.py:37-160.
"""

from __future__ import annotations

import heapq
from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np
import torch


@dataclass
class FlexMoECostModel:
    tps: float = 1.0e6
    sync_bps: float = 50e9 / 8
    sync_weight: float = 0.0
    threshold: float = 1.2


def _balanced_pack(cap: np.ndarray, counts: List[int], num_ranks: int, slots: int) -> Tuple[torch.Tensor, torch.Tensor]:
    items = sorted(((float(cap[e]), e) for e in range(len(counts)) for _ in range(counts[e])),
                   key=lambda t: t[0], reverse=True)
    load = np.zeros(num_ranks)
    place = np.zeros((len(counts), num_ranks), dtype=np.int64)
    heap = [(0.0, g) for g in range(num_ranks)]
    heapq.heapify(heap)
    free = [slots] * num_ranks
    for w, e in items:
        cur, g = heapq.heappop(heap)
        load[g] = cur + w
        place[e, g] = 1
        free[g] -= 1
        if free[g] > 0:
            heapq.heappush(heap, (cur + w, g))
    return torch.from_numpy(load), torch.from_numpy(place)


def flexmoe_schedule(omega: torch.Tensor, weight_bytes: torch.Tensor, num_ranks: int, n_slot: int,
                     cost: Optional[FlexMoECostModel] = None):
    """``(vExpert counts per expert, rank_load float64 [R], presence [E, R])``; ``n_slot`` = extra slots."""
    cost = cost or FlexMoECostModel()
    load_e = omega.detach().to("cpu", torch.float64).sum(0).numpy()
    wb = weight_bytes.detach().to("cpu", torch.float64).numpy()
    E = load_e.size
    if num_ranks <= 0 or E % num_ranks:
        raise ValueError("num_experts must be divisible by num_ranks")
    if n_slot < 0:
        raise ValueError("n_slot must be non-negative")
    mean = float(load_e.sum()) / num_ranks
    n = [1] * E
    cap = load_e.copy()
    left = num_ranks * int(n_slot)
    sync = 0.0

    def objective(max_cap: float, sync_total: float) -> float:
        return max(max_cap, mean) / cost.tps + cost.sync_weight * sync_total / cost.sync_bps

    while left > 0 and mean > 0:
        top = float(cap.max())
        if top / mean <= cost.threshold:
            break
        e = int(cap.argmax())
        before = objective(top, sync)
        old = cap[e]
        cap[e] = load_e[e] / (n[e] + 1)
        if objective(float(cap.max()), sync + wb[e]) < before:
            n[e] += 1
            sync += wb[e]
            left -= 1
        else:
            cap[e] = old
            break
    rank_load, placement = _balanced_pack(cap, n, num_ranks, E // num_ranks + int(n_slot))
    return n, rank_load, placement


__all__ = ["FlexMoECostModel", "flexmoe_schedule"]
