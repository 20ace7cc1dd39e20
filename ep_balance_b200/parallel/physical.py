"""Routing unit -> physical expert instance, from the plan's quota tensor.

Rule (reference: eplb/integration/physical.py:30-77): the units a source rank routes to
expert ``e``, taken in their original order, go to the hosts of ``e`` in ascending rank id,
``q[src, e, host]`` units each.  Local slots on a rank are ordered by ascending expert id, so
``phys_id = dst * n_slot + (number of hosted experts on dst with id <= e) - 1``.

This module is the host-tensor version (any device, no data-dependent shapes).  The fused layer
computes the same assignment plus the destination row with ``ops/csrc/route.cu``.
"""

from __future__ import annotations

from typing import Tuple

import torch

from ..core.plan import Plan
from ..core.problem import ProblemSpec


def build_phys_slot_table(x: torch.Tensor, n_slot: int) -> torch.Tensor:
    """int64 ``[E, R]``: physical id of ``(e, r)``; meaningful only where ``x[e, r] == 1``."""
    xi = x.to(torch.int64)
    R = xi.shape[1]
    return torch.arange(R, device=x.device, dtype=torch.int64)[None, :] * int(n_slot) + (xi.cumsum(0) - 1)


def rank_within_group(keys: torch.Tensor, num_keys: int) -> torch.Tensor:
    """For each element, how many earlier elements carry the same key (stable counting rank)."""
    order = torch.argsort(keys, stable=True)
    sorted_keys = keys[order]
    counts = torch.zeros(num_keys, dtype=torch.int64, device=keys.device).scatter_add_(
        0, keys, torch.ones_like(keys))
    starts = counts.cumsum(0) - counts
    pos = torch.arange(keys.numel(), device=keys.device, dtype=torch.int64) - starts[sorted_keys]
    out = torch.empty_like(pos)
    out[order] = pos
    return out


def assign_physical(unit_expert: torch.Tensor, plan: Plan, spec: ProblemSpec, src_rank: int
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(phys_id[U], dst_rank[U])`` for the units of ``src_rank``."""
    ue = unit_expert.to(torch.int64)
    q_me = plan.q[int(src_rank)].to(torch.int64)  # [E, R]
    j = rank_within_group(ue, int(spec.num_experts))  # index of the unit among its expert's units
    upper = q_me.cumsum(1)  # [E, R] inclusive prefix over hosts
    dst = (upper[ue] <= j[:, None]).sum(1)  # first host whose prefix exceeds j
    dst = dst.clamp_(max=q_me.shape[1] - 1)
    phys = build_phys_slot_table(plan.x, int(spec.n_slot))[ue, dst]
    return phys, dst
