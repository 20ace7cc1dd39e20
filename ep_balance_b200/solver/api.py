"""``solve()``: one entry point, backend chosen by where ``omega`` lives.

Host tensors go to the serial solver (:mod:`.exact`); CUDA tensors go to the
single-launch device solver (:mod:`ep_balance_b200.ops.solver_op`) and never fall
back to the host -- the same contract as the reference (eplb/algorithm.py:228-236).
"""

from __future__ import annotations

from typing import Optional

import torch

from ..core.config import EPLBConfig
from ..core.loads import Loads
from ..core.plan import Plan
from ..core.problem import ProblemSpec
from ..core.topology import Topology
from .exact import solve_exact


def validate_inputs(loads: Loads, topo: Topology, spec: ProblemSpec, cfg: EPLBConfig) -> None:
    topo.validate()
    spec.validate(topo.num_ranks)
    loads.validate(topo.num_ranks, spec.num_experts)
    if cfg.u_min > 1 and bool(((loads.omega > 0) & (loads.omega < cfg.u_min)).any()):
        raise ValueError("u_min is infeasible: every positive Ω[r,e] must be >= u_min")


def solve(loads: Loads, topo: Topology, spec: ProblemSpec, cfg: Optional[EPLBConfig] = None, *,
          validate: bool = True) -> Plan:
    cfg = cfg or EPLBConfig()
    if validate:
        validate_inputs(loads, topo, spec, cfg)
    if loads.omega.is_cuda and topo.num_ranks > 0 and spec.num_experts > 0:
        from ..ops.solver_op import solve_cuda

        return solve_cuda(loads, topo, spec, cfg)
    return solve_exact(loads, topo, spec, cfg)
