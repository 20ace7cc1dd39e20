"""Tensor-level wrapper of the device solver (``csrc/solver.cu``).

``solve_cuda`` is what :func:`ep_balance_b200.solve` calls for CUDA inputs.  Static inputs
(domain map, cost, owners, weight bytes) are converted to the kernel's dtypes once per
``(Topology, ProblemSpec)`` pair; per-call work is one int32 cast of ``omega``, one kernel
launch and one widening cast of ``q``.  Nothing here reads device memory on the host.
Reference counterpart: eplb/cuda_solve.py:71-119.
"""

from __future__ import annotations

import weakref
from typing import Dict, Tuple

import torch

from ..core.config import EPLBConfig
from ..core.loads import Loads
from ..core.plan import Plan
from ..core.problem import ProblemSpec
from ..core.topology import Topology
from .extension import load

_STATIC: "Dict[Tuple[int, int, str], tuple]" = {}


def _static_inputs(topo: Topology, spec: ProblemSpec, device: torch.device):
    key = (id(topo), id(spec), str(device))
    hit = _STATIC.get(key)
    if hit is not None and hit[0]() is topo and hit[1]() is spec:
        return hit[2]
    vals = (
        topo.domain_of_rank.to(device=device, dtype=torch.int32).contiguous(),
        topo.cost.to(device=device, dtype=torch.int32).contiguous(),
        spec.main_rank.to(device=device, dtype=torch.int32).contiguous(),
        spec.weight_bytes.to(device=device, dtype=torch.int64).contiguous(),
    )
    _STATIC[key] = (weakref.ref(topo), weakref.ref(spec), vals)
    return vals


class SolverWorkspace:
    """Scratch reused across solves of one (R, E) shape on one device."""

    def __init__(self, R: int, E: int, device: torch.device) -> None:
        i32 = dict(dtype=torch.int32, device=device)
        self.erl = torch.empty((E, R), **i32)
        self.rank_load = torch.empty(R, **i32)
        self.slot_used = torch.empty(R, **i32)
        self.stuck = torch.empty(R, dtype=torch.uint8, device=device)
        self.control = torch.zeros(3, dtype=torch.int64, device=device)
        self.sync = torch.zeros(2, **i32)
        self.status = torch.zeros(4, **i32)


_WS: Dict[Tuple[int, int, str], SolverWorkspace] = {}


def workspace(R: int, E: int, device: torch.device) -> SolverWorkspace:
    key = (R, E, str(device))
    ws = _WS.get(key)
    if ws is None:
        ws = _WS[key] = SolverWorkspace(R, E, device)
    return ws


def solve_cuda(loads: Loads, topo: Topology, spec: ProblemSpec, cfg: EPLBConfig, *, q_dtype=torch.int64,
               return_aux: bool = False):
    ext = load()
    device = loads.omega.device
    R, E = topo.num_ranks, spec.num_experts
    dom, cost, main_rank, wbytes = _static_inputs(topo, spec, device)
    ws = workspace(R, E, device)
    omega = loads.omega.to(torch.int32).contiguous()
    x = torch.empty((E, R), dtype=torch.int8, device=device)
    q = torch.empty((R, E, R), dtype=torch.int32, device=device)
    theta = torch.empty(1, dtype=torch.int64, device=device)
    iters = cfg.device_stage2_iters
    probe = bool(cfg.stage2_patience_all_scales) and iters > cfg.stage2_stagnation_patience + 1
    ext.solve_plan(omega, dom, cost, main_rank, wbytes, int(spec.s_tok), int(topo.sync_free_num_domains),
                   int(spec.n_slot), int(cfg.u_min), int(iters), int(cfg.stage2_stagnation_patience),
                   bool(cfg.allow_cross_domain), probe, x, q, ws.erl, ws.rank_load, ws.slot_used, ws.stuck,
                   theta, ws.control, ws.sync, ws.status)
    plan = Plan(x=x, q=q if q_dtype == torch.int32 else q.to(q_dtype), theta=theta[0])
    if return_aux:
        return plan, ws
    return plan
