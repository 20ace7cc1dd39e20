"""Solver output: placement ``x``, routing quota ``q`` and the max rank load ``theta``.

Reference: eplb/plan.py:10-64.  ``theta`` may be a 0-dim device tensor when the
plan came from the on-device solver; converting it to ``int`` is the only host
sync a plan can cause.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Dict, Tuple, Union

import torch


@dataclass
class Plan:
    x: torch.Tensor  # int8 [E, R]
    q: torch.Tensor  # int64 [R, E, R]  q[src, expert, dst]
    theta: Union[int, torch.Tensor]

    @property
    def num_experts(self) -> int:
        return int(self.x.shape[0])

    @property
    def num_ranks(self) -> int:
        return int(self.x.shape[1])

    def num_replicas(self) -> torch.Tensor:
        return self.x.sum(1).to(torch.int64)

    def replicas_of(self, e: int) -> torch.Tensor:
        return (self.x[int(e)] == 1).nonzero(as_tuple=False).flatten()

    def rank_load(self) -> torch.Tensor:
        return self.q.sum((0, 1)).to(torch.int64)

    def slots_used(self) -> torch.Tensor:
        return self.x.sum(0).to(torch.int64)

    def dispatch_indices(self, src_rank: int) -> Dict[int, Tuple[torch.Tensor, torch.Tensor]]:
        """``{expert: (dst ranks, unit counts)}`` for every expert ``src_rank`` sends to."""
        rows = self.q[int(src_rank)]
        out: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        for e in (rows.sum(1) > 0).nonzero(as_tuple=False).flatten().tolist():
            dst = (rows[e] > 0).nonzero(as_tuple=False).flatten()
            out[e] = (dst, rows[e][dst].clone())
        return out

    def equals(self, other: "Plan") -> bool:
        return (int(self.theta) == int(other.theta) and torch.equal(self.x, other.x)
                and torch.equal(self.q.to(torch.int64), other.q.to(torch.int64)))

    def digest(self) -> str:
        """sha256 over ``x || q || theta``; equal digests on every rank prove a replicated plan."""
        h = hashlib.sha256()
        h.update(self.x.detach().to("cpu", torch.int8).contiguous().numpy().tobytes())
        h.update(self.q.detach().to("cpu", torch.int64).contiguous().numpy().tobytes())
        h.update(int(self.theta).to_bytes(8, "little", signed=True))
        return h.hexdigest()

    def to(self, device) -> "Plan":
        th = self.theta.to(device) if isinstance(self.theta, torch.Tensor) else self.theta
        return Plan(self.x.to(device), self.q.to(device), th)
