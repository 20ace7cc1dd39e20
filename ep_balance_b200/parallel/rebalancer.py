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


class _StepRing:
    """What backward needs from the last ``size`` (layer, micro-batch) steps: the load matrix, and the plan too when
    plans are kept.  One ordered map of records; the oldest step leaves first."""

    def __init__(self, size: int, keep_plans: bool) -> None:
        self.size, self.keep_plans = int(size), bool(keep_plans)
        self._steps: "OrderedDict[Tuple[int, int], Tuple[torch.Tensor, Optional[Plan]]]" = OrderedDict()

    def put(self, key: Tuple[int, int], omega: torch.Tensor, plan: Plan) -> None:
        if self.size <= 0:
            return
        self._steps[key] = (omega, plan if self.keep_plans else None)
        self._steps.move_to_end(key)
        while len(self._steps) > self.size:
            self._steps.popitem(last=False)

    def get(self, key: Tuple[int, int]) -> Optional[Tuple[torch.Tensor, Optional[Plan]]]:
        return self._steps.get(key)

    def clear(self) -> None:
        self._steps.clear()

    def __len__(self) -> int:
        return len(self._steps)


class EPLBRebalancer:
    def __init__(self, topo: Topology, spec: ProblemSpec, cfg: Optional[EPLBConfig] = None,
                 materializer: Optional[WeightMaterializer] = None, *, cache_plans: bool = False,
                 ring_size: int = 64) -> None:
        topo.validate()
        spec.validate(topo.num_ranks)
        self.topo, self.spec = topo, spec
        self.cfg = cfg or EPLBConfig()
        self.materializer = materializer or NullWeightMaterializer()
        self.cache_plans, self.ring_size = bool(cache_plans), int(ring_size)
        self._ring = _StepRing(self.ring_size, self.cache_plans)

    # ---- forward ----------------------------------------------------------
    def plan_from_omega(self, loads: Loads) -> Plan:
        with profiling.record("solve", time_it=True, device=loads.device):
            return solve(loads, self.topo, self.spec, self.cfg, validate=False)

    def rebalance_from_omega(self, loads: Loads, layer_id: int, micro_batch_id: int) -> RebalanceResult:
        plan = self.plan_from_omega(loads)
        self._ring.put((int(layer_id), int(micro_batch_id)), loads.omega, plan)
        handle = self.materializer.materialize(plan, layer_id, micro_batch_id)
        return RebalanceResult(plan, handle)

    def rebalance(self, local_row: torch.Tensor, layer_id: int, micro_batch_id: int, *, group=None) -> RebalanceResult:
        with profiling.record("all_gather_omega", time_it=True, device=local_row.device):
            loads = all_gather_omega(local_row, group=group)
        return self.rebalance_from_omega(loads, layer_id, micro_batch_id)

    # ---- backward ---------------------------------------------------------
    def backward(self, layer_id: int, micro_batch_id: int) -> Plan:
        """The forward's plan of that step (kept, or solved again from the kept load matrix: the solvers are
        deterministic), after telling the materializer to fold the replicas' gradients."""
        step = self._ring.get((int(layer_id), int(micro_batch_id)))
        if step is None:
            raise KeyError(f"no cached Ω for (layer={layer_id}, mb={micro_batch_id}); "
                           f"increase ring_size (current={self.ring_size})")
        omega, plan = step
        if plan is None:
            plan = self.plan_from_omega(Loads(omega))
        self.materializer.aggregate_gradients(plan, layer_id, micro_batch_id)
        return plan

    def omega_of(self, layer_id: int, micro_batch_id: int) -> Optional[torch.Tensor]:
        """The load matrix the plan of that step was solved from, while the step is still remembered."""
        step = self._ring.get((int(layer_id), int(micro_batch_id)))
        return None if step is None else step[0]

    def clear(self) -> None:
        self._ring.clear()
