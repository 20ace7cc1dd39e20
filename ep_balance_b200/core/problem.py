"""Per-layer constants: owner of each expert, weight bytes, token bytes, slot budget.

``n_slot`` is the TOTAL number of physical expert slots per rank, owners included
(reference: eplb/problem.py:10-65).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Union

import torch


@dataclass
class ProblemSpec:
    num_experts: int
    main_rank: torch.Tensor  # int64 [E]; never changes (C7)
    weight_bytes: torch.Tensor  # int64 [E]
    s_tok: int  # bytes of one token activation
    n_slot: int  # physical slots per rank, mains included (C4)

    def __post_init__(self) -> None:
        self.main_rank = self.main_rank.to(torch.int64)
        self.weight_bytes = self.weight_bytes.to(torch.int64)

    @property
    def device(self) -> torch.device:
        return self.main_rank.device

    def to(self, device) -> "ProblemSpec":
        return ProblemSpec(self.num_experts, self.main_rank.to(device), self.weight_bytes.to(device),
                           self.s_tok, self.n_slot)

    def validate(self, num_ranks: int) -> None:
        E = int(self.num_experts)
        if tuple(self.main_rank.shape) != (E,):
            raise ValueError(f"main_rank must be [E]=[{E}], got {tuple(self.main_rank.shape)}")
        if tuple(self.weight_bytes.shape) != (E,):
            raise ValueError(f"weight_bytes must be [E]=[{E}], got {tuple(self.weight_bytes.shape)}")
        if E and (bool((self.main_rank < 0).any()) or bool((self.main_rank >= num_ranks).any())):
            raise ValueError("main_rank entries must be in [0, num_ranks)")
        if int(self.s_tok) <= 0:
            raise ValueError("s_tok must be a positive integer")
        if int(self.n_slot) <= 0:
            raise ValueError("n_slot must be a positive integer")
        if E and int(torch.bincount(self.main_rank, minlength=num_ranks).max()) > int(self.n_slot):
            raise ValueError("n_slot too small: some rank's primary instances already exceed N_slot")

    @staticmethod
    def uniform_main_placement(num_experts: int, num_ranks: int, weight_bytes_each: int, s_tok: int,
                               n_slot: int, device: Union[torch.device, str] = "cpu") -> "ProblemSpec":
        """Round-robin owners ``main(e) = e mod R`` with equal weight sizes."""
        e = torch.arange(num_experts, dtype=torch.int64, device=device)
        spec = ProblemSpec(num_experts, e % num_ranks, torch.full_like(e, int(weight_bytes_each)), s_tok, n_slot)
        spec.validate(num_ranks)
        return spec

    @staticmethod
    def contiguous_main_placement(num_experts: int, num_ranks: int, weight_bytes_each: int, s_tok: int,
                                  n_slot: int, device: Union[torch.device, str] = "cpu") -> "ProblemSpec":
        """Block owners ``main(e) = e // (E/R)`` -- the layout expert-parallel training frameworks use."""
        if num_experts % num_ranks:
            raise ValueError("num_experts must be divisible by num_ranks")
        e = torch.arange(num_experts, dtype=torch.int64, device=device)
        spec = ProblemSpec(num_experts, e // (num_experts // num_ranks),
                           torch.full_like(e, int(weight_bytes_each)), s_tok, n_slot)
        spec.validate(num_ranks)
        return spec
