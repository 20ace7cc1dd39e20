"""The per-micro-batch load matrix ``omega[r, e]`` (reference: eplb/loads.py:10-48)."""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class Loads:
    omega: torch.Tensor  # int64 [R, E]: routed (token, top-k) units from source rank r to expert e

    def __post_init__(self) -> None:
        self.omega = self.omega.to(torch.int64)

    @property
    def num_ranks(self) -> int:
        return int(self.omega.shape[0])

    @property
    def num_experts(self) -> int:
        return int(self.omega.shape[1])

    @property
    def device(self) -> torch.device:
        return self.omega.device

    def expert_load(self) -> torch.Tensor:
        return self.omega.sum(0)

    def domain_demand(self, domain_of_rank: torch.Tensor, num_domains: int) -> torch.Tensor:
        """``T[d, e]``: units that sources of domain ``d`` route to expert ``e``."""
        out = self.omega.new_zeros((int(num_domains), self.num_experts))
        out.index_add_(0, domain_of_rank.to(torch.int64), self.omega)
        return out

    def validate(self, num_ranks: int, num_experts: int) -> None:
        if tuple(self.omega.shape) != (num_ranks, num_experts):
            raise ValueError(
                f"omega must be [R, E]=[{num_ranks},{num_experts}], got {tuple(self.omega.shape)}")
        if bool((self.omega < 0).any()):
            raise ValueError("token counts must be non-negative")
