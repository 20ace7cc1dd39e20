"""Seams between the balancer and a training framework (reference: eplb/integration/hooks.py:13-65)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol, runtime_checkable

import torch

from ..core.plan import Plan


@dataclass
class RebalanceResult:
    plan: Plan
    weight_handle: object = None


@runtime_checkable
class WeightMaterializer(Protocol):
    """Brings replica weights onto their hosts and returns their gradients to the owner."""

    def materialize(self, plan: Plan, layer_id: int, micro_batch_id: int) -> object: ...

    def release(self, handle: object) -> None: ...

    def aggregate_gradients(self, plan: Plan, layer_id: int, micro_batch_id: int) -> None: ...


class NullWeightMaterializer:
    """Moves nothing; for observe mode, simulation and tests."""

    def materialize(self, plan: Plan, layer_id: int, micro_batch_id: int) -> object:
        return {"layer_id": layer_id, "micro_batch_id": micro_batch_id}

    def release(self, handle: object) -> None:
        return None

    def aggregate_gradients(self, plan: Plan, layer_id: int, micro_batch_id: int) -> None:
        return None


@runtime_checkable
class Dispatcher(Protocol):
    """Token transport driven by a plan's quota tensor."""

    def dispatch(self, hidden_states: torch.Tensor, plan: Plan, src_rank: int): ...

    def combine(self, expert_outputs: torch.Tensor, plan: Plan, src_rank: int): ...
