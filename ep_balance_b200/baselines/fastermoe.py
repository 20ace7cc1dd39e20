"""FasterMoE dynamic shadowing (PPoPP'22, Algorithm 1) as a placement baseline.

Hot experts are "shadowed": replicated on every rank so that each source rank computes its own
tokens of that expert locally.  Experts are tried in descending load; one is kept while the
performance model (compute on the busiest rank + weight broadcast, counted twice for the gradient
reduce) predicts a faster step and while every rank still has a free replica slot.
Reference port: baseline/fastermoe.py:24-140.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch


@dataclass
class ShadowCostModel:
    bw_net: float = 50e9 / 8  # bytes/s between workers
    bw_mm: float = 11.5e12  # GEMM rate used as compute speed
    grad_factor: float = 2.0  # broadcast forward + reduce backward
    fwd_bwd_gemms: int = 3
    comm_rounds: int = 4  # token all-to-alls per iteration


def select_shadow_experts(omega: torch.Tensor, main_rank: torch.Tensor, weight_bytes: torch.Tensor, s_tok: int,
                          num_ranks: int, cost: Optional[ShadowCostModel] = None, n_slot: Optional[int] = None
                          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(shadow_mask bool [E], rank_load float64 [R])`` after redistribution."""
    cost = cost or ShadowCostModel()
    if n_slot is not None and int(n_slot) < 0:
        raise ValueError("n_slot must be non-negative")
    om = omega.detach().to("cpu", torch.float64).numpy()
    home = main_rank.detach().to("cpu", torch.int64).numpy()
    wb = weight_bytes.detach().to("cpu", torch.float64).numpy()
    E = om.shape[1]
    per_expert = om.sum(0)
    load = np.zeros(num_ranks)
    np.add.at(load, home, per_expert)
    comp = cost.fwd_bwd_gemms * 4.0 * float((wb / 2.0).mean()) / cost.bw_mm  # seconds per token
    best = comp * load.max() + cost.comm_rounds * load.max() * s_tok / cost.bw_net
    mask = np.zeros(E, dtype=bool)
    extra = np.zeros(num_ranks, dtype=np.int64)
    moved_bytes = 0.0
    for e in np.argsort(-per_expert, kind="stable"):
        need = np.ones(num_ranks, dtype=np.int64)
        need[home[e]] = 0
        if n_slot is not None and np.any(extra + need > int(n_slot)):
            break
        trial = load.copy()
        trial[home[e]] -= per_expert[e]
        trial += om[:, e]
        t = comp * trial.max() + cost.grad_factor * (moved_bytes + wb[e]) / cost.bw_net
        if t >= best:
            break
        best, load, moved_bytes = t, trial, moved_bytes + wb[e]
        mask[e] = True
        extra += need
    return torch.from_numpy(mask), torch.from_numpy(load)


__all__ = ["ShadowCostModel", "select_shadow_experts"]
