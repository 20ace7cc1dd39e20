"""Rank -> domain map and the integer per-token cost matrix.

On one NVSwitch box the wire is uniform; domains are *logical* partitions that
only exist in the solver's cost model (reference: eplb/topology.py:10-100).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Union

import torch


@dataclass
class Topology:
    domain_of_rank: torch.Tensor  # int64 [R]
    cost: torch.Tensor  # int64 [R, R], zero diagonal
    num_domains_hint: Optional[int] = None  # host-known domain count (avoids a device read)

    def __post_init__(self) -> None:
        self.domain_of_rank = self.domain_of_rank.to(torch.int64)
        self.cost = self.cost.to(torch.int64)
        if self.num_domains_hint is not None and int(self.num_domains_hint) < 0:
            raise ValueError("num_domains_hint must be non-negative")

    # ---- sizes -----------------------------------------------------------
    @property
    def num_ranks(self) -> int:
        return int(self.domain_of_rank.numel())

    @property
    def num_domains(self) -> int:
        if self.num_domains_hint is not None:
            return int(self.num_domains_hint)
        if self.num_ranks == 0:
            return 0
        return int(self.domain_of_rank.max().item()) + 1

    @property
    def sync_free_num_domains(self) -> int:
        """Domain count without touching device memory (upper bound R when no hint)."""
        if self.num_domains_hint is not None:
            return int(self.num_domains_hint)
        return self.num_ranks

    @property
    def device(self) -> torch.device:
        return self.domain_of_rank.device

    def ranks_in_domain(self, d: int) -> torch.Tensor:
        return (self.domain_of_rank == int(d)).nonzero(as_tuple=False).flatten()

    def to(self, device) -> "Topology":
        return Topology(self.domain_of_rank.to(device), self.cost.to(device), self.num_domains_hint)

    # ---- checks ----------------------------------------------------------
    def validate(self) -> None:
        R = self.num_ranks
        if tuple(self.cost.shape) != (R, R):
            raise ValueError(f"cost must be [R, R]=[{R},{R}], got {tuple(self.cost.shape)}")
        if bool((self.cost.diagonal() != 0).any()):
            raise ValueError("cost matrix diagonal must be zero (c[r,r]=0)")
        if bool((self.cost < 0).any()):
            raise ValueError("cost matrix must be non-negative")
        ids = torch.unique(self.domain_of_rank)
        if not torch.equal(ids, torch.arange(ids.numel(), dtype=torch.int64, device=ids.device)):
            raise ValueError("domain ids must be contiguous starting at 0")
        if self.num_domains_hint is not None and int(self.num_domains_hint) != int(ids.numel()):
            raise ValueError("num_domains_hint must equal the number of domains in domain_of_rank")

    # ---- builders --------------------------------------------------------
    @staticmethod
    def from_nvlink_rdma(
        num_nodes: int,
        gpus_per_node: int,
        intra_cost: int = 1,
        inter_cost: int = 8,
        device: Union[torch.device, str] = "cpu",
    ) -> "Topology":
        """``num_nodes`` domains of ``gpus_per_node`` consecutive ranks each."""
        if intra_cost <= 0 or inter_cost <= 0:
            raise ValueError("costs must be positive integers")
        R = int(num_nodes) * int(gpus_per_node)
        dom = torch.arange(R, dtype=torch.int64, device=device) // int(gpus_per_node)
        same = dom[:, None] == dom[None, :]
        cost = torch.where(same, int(intra_cost), int(inter_cost)).to(torch.int64)
        cost.fill_diagonal_(0)
        topo = Topology(dom, cost, num_domains_hint=int(num_nodes))
        topo.validate()
        return topo

    @staticmethod
    def logical(num_ranks: int, num_domains: int, intra_cost: int = 1, inter_cost: int = 8,
                device: Union[torch.device, str] = "cpu") -> "Topology":
        """Split ``num_ranks`` GPUs of one NVSwitch box into equal logical domains."""
        if num_ranks % num_domains:
            raise ValueError("num_ranks must be divisible by num_domains")
        return Topology.from_nvlink_rdma(num_domains, num_ranks // num_domains, intra_cost, inter_cost, device)
