"""Collect omega -> solve -> hand the plan to a weight materializer, per (layer, micro-batch).

Backward needs the forward's plan again.  Because every solver here is
deterministic, the default is to remember only ``omega`` and re-solve; caching the
plan itself is opt-in (reference: eplb/integration/rebalancer.py:20-137).
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Optional, Tuple

import torch

from ..core.config import EPLBConfig
from ..core.loads import Loads
from ..core.plan import Plan
from ..core.problem import ProblemSpec
from ..core.topology import Topology
from ..solver.api import solve
from ..utils import profiling
from .hooks import NullWeightMaterializer, RebalanceResult, WeightMaterializer
from .omega import all_gather_omega


class EPLBRebalancer:
    def __init__(self, topo: Topology, spec: ProblemSpec, cfg: Optional[EPLBConfig] = None,
                 materializer: Optional[WeightMaterializer] = None, *, cache_plans: bool = False,
                 ring_size: int = 64) -> None:
        topo.validate()
        spec.validate(topo.num_ranks)
        self.topo, self.spec = topo, spec
        self.cfg = cfg or EPLBConfig()
        self.materializer = materializer or NullWeightMaterializer()
        self.cache_plans = bool(cache_plans)
        self.ring_size = int(ring_size)
        # insertion-ordered: the oldest (layer, mb) is evicted first
        self._omega_ring: "OrderedDict[Tuple[int, int], torch.Tensor]" = OrderedDict()
        self._plan_ring: dict = {}

    # ---- forward ----------------------------------------------------------
    def plan_from_omega(self, loads: Loads) -> Plan:
        with profiling.record("solve", time_it=True, device=loads.device):
            return solve(loads, self.topo, self.spec, self.cfg, validate=False)

    def rebalance_from_omega(self, loads: Loads, layer_id: int, micro_batch_id: int) -> RebalanceResult:
        plan = self.plan_from_omega(loads)
        self._remember(layer_id, micro_batch_id, loads.omega, plan)
        return RebalanceResult(plan, self.materializer.materialize(plan, layer_id, micro_batch_id))

    def rebalance(self, local_row: torch.Tensor, layer_id: int, micro_batch_id: int, *, group=None) -> RebalanceResult:
        with profiling.record("all_gather_omega", time_it=True, device=local_row.device):
            loads = all_gather_omega(local_row, group=group)
        return self.rebalance_from_omega(loads, layer_id, micro_batch_id)

    # ---- backward ---------------------------------------------------------
    def backward(self, layer_id: int, micro_batch_id: int) -> Plan:
        key = (int(layer_id), int(micro_batch_id))
        plan = self._plan_ring.get(key) if self.cache_plans else None
        if plan is None:
            if key not in self._omega_ring:
                raise KeyError(f"no cached Ω for (layer={layer_id}, mb={micro_batch_id}); "
                               f"increase ring_size (current={self.ring_size})")
            plan = self.plan_from_omega(Loads(self._omega_ring[key]))
        self.materializer.aggregate_gradients(plan, layer_id, micro_batch_id)
        return plan

    # ---- ring -------------------------------------------------------------
    def _remember(self, layer_id: int, micro_batch_id: int, omega: torch.Tensor, plan: Plan) -> None:
        if self.ring_size <= 0:
            return
        key = (int(layer_id), int(micro_batch_id))
        self._omega_ring[key] = omega
        if self.cache_plans:
            self._plan_ring[key] = plan
        while len(self._omega_ring) > self.ring_size:
            old, _ = self._omega_ring.popitem(last=False)
            self._plan_ring.pop(old, None)

    def clear(self) -> None:
        self._omega_ring.clear()
        self._plan_ring.clear()
