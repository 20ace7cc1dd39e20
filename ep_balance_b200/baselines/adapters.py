"""Every balancing strategy reduced to the same comparable result (per-rank load + placement).

Throughout the baseline harness ``n_slot`` means ADDITIONAL replica slots per rank (mains excluded);
``ProblemSpec.n_slot`` is the total.  Reference: baseline/adapters.py:22-429.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

import torch

from ..core.config import EPLBConfig
from ..core.loads import Loads
from ..core.problem import ProblemSpec
from ..core.topology import Topology
from ..solver.api import solve
from .deepseek_eplb import rebalance_experts
from .fastermoe import ShadowCostModel, select_shadow_experts
from .flexmoe import FlexMoECostModel, flexmoe_schedule


@dataclass
class BaselineResult:
    name: str
    rank_load: torch.Tensor
    placement: Optional[torch.Tensor] = None
    metadata: Dict[str, Any] = field(default_factory=dict)

    @property
    def theta(self) -> float:
        return float(self.rank_load.max()) if self.rank_load.numel() else 0.0

    @property
    def mean_load(self) -> float:
        return float(self.rank_load.double().mean()) if self.rank_load.numel() else 0.0

    @property
    def imbalance(self) -> float:
        m = self.mean_load
        return self.theta / m if m > 0 else 1.0


class LPLBUnavailableError(RuntimeError):
    """The optional compiled LPLB package cannot be imported."""


def slot_budget(num_experts: int, num_ranks: int, n_slot: int) -> Tuple[int, int, int]:
    """``(main, replica, physical)`` slots per rank for ``n_slot`` additional replica slots."""
    if num_ranks <= 0 or num_experts % num_ranks:
        raise ValueError("num_experts must be divisible by num_ranks")
    if int(n_slot) < 0:
        raise ValueError("n_slot must be non-negative")
    main = num_experts // num_ranks
    return main, int(n_slot), main + int(n_slot)


def _budget(num_experts: int, num_ranks: int, n_slot: int, instances: int) -> Dict[str, int]:
    main, rep, phys = slot_budget(num_experts, num_ranks, n_slot)
    return {"main_slots_per_rank": main, "replica_slots_per_rank": rep, "physical_slots_per_rank": phys,
            "replica_budget": num_ranks * rep, "physical_instances": int(instances),
            "replicas": max(0, int(instances) - num_experts)}


def run_scale_eplb(loads: Loads, topology: Topology, spec: ProblemSpec, cfg: Optional[EPLBConfig] = None,
                   solver=None) -> BaselineResult:
    """This framework's solver (``solver`` overrides the default dispatch, e.g. ``solve_device_semantics``)."""
    plan = (solver or (lambda l, t, s, c: solve(l, t, s, c, validate=False)))(loads, topology, spec, cfg or EPLBConfig())
    main, _, _ = slot_budget(spec.num_experts, topology.num_ranks, 0)
    return BaselineResult("scale-eplb", plan.rank_load(), plan.x, {
        "load_kind": "realized quota load", "placement_kind": "binary expert presence",
        **_budget(spec.num_experts, topology.num_ranks, int(spec.n_slot) - main, int(plan.x.sum()))})


def run_deepseek_eplb(loads: Loads, *, num_nodes: int, num_gpus: int, n_slot: int, num_groups: int,
                      placement_loads: Optional[Loads] = None) -> BaselineResult:
    """DeepSeek-EPLB with its own quality notion: an expert's load divides equally over its replicas."""
    E = loads.num_experts
    _, _, phys = slot_budget(E, num_gpus, n_slot)
    P = E + num_gpus * int(n_slot)
    now = loads.expert_load().cpu()
    basis = placement_loads.expert_load().cpu() if placement_loads is not None else now
    phy2log, _, logcnt = rebalance_experts(basis[None], P, num_groups, num_nodes, num_gpus)
    phy2log, logcnt = phy2log[0], logcnt[0]
    per_phys = now.double() / logcnt.double()
    rank_load = per_phys[phy2log].view(num_gpus, phys).sum(1)
    placement = torch.zeros((E, num_gpus), dtype=torch.int64)
    placement.index_put_((phy2log, torch.arange(num_gpus).repeat_interleave(phys)), torch.ones_like(phy2log),
                         accumulate=True)
    return BaselineResult("deepseek-eplb", rank_load, placement, {
        "load_kind": "ideal equal-split predicted load", "placement_kind": "physical replica count",
        "num_groups": num_groups, **_budget(E, num_gpus, n_slot, P)})


def run_fastermoe(loads: Loads, spec: ProblemSpec, *, num_ranks: int, n_slot: int,
                  cost: Optional[ShadowCostModel] = None) -> BaselineResult:
    mask, rank_load = select_shadow_experts(loads.omega, spec.main_rank, spec.weight_bytes, spec.s_tok, num_ranks,
                                            cost, n_slot)
    placement = torch.zeros((spec.num_experts, num_ranks), dtype=torch.int64)
    placement[torch.arange(spec.num_experts), spec.main_rank.cpu()] = 1
    placement[mask] = 1
    return BaselineResult("fastermoe", rank_load, placement, {
        "load_kind": "shadow-redistributed token load", "placement_kind": "binary expert presence (shadow=all ranks)",
        "shadowed_experts": int(mask.sum()), **_budget(spec.num_experts, num_ranks, n_slot, int(placement.sum()))})


def run_flexmoe(loads: Loads, spec: ProblemSpec, *, num_ranks: int, n_slot: int,
                cost: Optional[FlexMoECostModel] = None) -> BaselineResult:
    counts, rank_load, placement = flexmoe_schedule(loads.omega, spec.weight_bytes, num_ranks, n_slot, cost)
    mean = float(rank_load.mean()) if rank_load.numel() else 0.0
    return BaselineResult("flexmoe", rank_load, placement, {
        "load_kind": "even-split vExpert load (balance ratio)",
        "placement_kind": "binary expert presence (vExpert replicas)",
        "balance_ratio": float(rank_load.max()) / mean if mean > 0 else 1.0,
        **_budget(spec.num_experts, num_ranks, n_slot, int(sum(counts)))})


def cube8_topology() -> torch.Tensor:
    """Edges of the 3-cube on 8 ranks (two outgoing edges per rank), LPLB's even-budget topology."""
    edges = []
    for r in range(8):
        edges += [[r, r ^ 1], [r, r ^ 2]]
    return torch.tensor(edges, dtype=torch.int64)


def ring8_topology() -> torch.Tensor:
    return torch.tensor([[r, (r + 1) % 8] for r in range(8)], dtype=torch.int64)


def select_lplb_topology(name: str, n_slot: int) -> Tuple[str, torch.Tensor]:
    if name == "auto":
        name = "ring" if int(n_slot) % 2 else "cube"
    if name == "cube":
        return name, cube8_topology()
    if name == "ring":
        return name, ring8_topology()
    raise ValueError("lplb topology must be auto, cube or ring")


def load_lplb(lplb_root=None):
    """Import the external LPLB planner; it needs its own compiled CUDA extension."""
    import sys

    if lplb_root is not None and str(lplb_root) not in sys.path:
        sys.path.insert(0, str(lplb_root))
    try:
        import lplb  # type: ignore

        return lplb
    except Exception as exc:  # pragma: no cover - depends on an external package
        raise LPLBUnavailableError(f"LPLB is not importable: {exc}") from exc


class LPLBBaseline:
    """Thin adapter around LPLB's ``Planner`` (constructed lazily; raises :class:`LPLBUnavailableError`)."""

    def __init__(self, *, num_experts: int, num_ranks: int, n_slot: int, topology: str = "auto", lplb_root=None) -> None:
        self.lplb = load_lplb(lplb_root)
        self.num_experts, self.num_ranks, self.n_slot = num_experts, num_ranks, n_slot
        self.topology_name, self.edges = select_lplb_topology(topology, n_slot)
        self.planner = self.lplb.Planner(self.edges, num_experts + num_ranks * n_slot, num_experts)  # pragma: no cover

    def solve(self, workload: torch.Tensor) -> BaselineResult:  # pragma: no cover - external package
        probs = self.planner.run(workload)
        load = (probs * workload.sum(0, keepdim=True)).sum(0).view(self.num_ranks, -1).sum(1)
        return BaselineResult("lplb", load, None, {"topology": self.topology_name})
