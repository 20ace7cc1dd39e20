"""Device solver vs its host restatement: every element of x, q and theta must agree.

Mirrors the reference's GPU solver tests (tests/test_gpu_solver.py:31-284): quality relative to
the serial solver, repeat-solve bit equality, quota floors, and no host sync on a warmed solve.
"""

import pytest
import torch

from ep_balance_b200 import EPLBConfig, Loads, ProblemSpec, Topology, check_constraints, solve
from ep_balance_b200.solver import solve_device_semantics, solve_exact
from ep_balance_b200.utils.workload import make_loads

pytestmark = pytest.mark.gpu

GRID = [
    # nodes, gpus, E, extra, skew, seed, u_min
    (1, 8, 64, 2, 1.2, 0, 1),
    (2, 4, 64, 2, 1.4, 1, 1),
    (4, 2, 128, 1, 1.0, 2, 1),
    (2, 4, 256, 4, 1.3, 3, 1),
    (1, 8, 512, 0, 1.2, 4, 1),
    (4, 8, 640, 4, 1.5, 5, 1),
    (2, 4, 64, 2, 1.4, 6, 4),
    (8, 8, 128, 2, 1.5, 7, 1),
    (1, 1, 16, 0, 1.0, 8, 1),
    (3, 3, 45, 3, 1.1, 9, 2),
]


def _problem(nodes, gpus, E, extra, skew, seed, u_min, device):
    R = nodes * gpus
    loads = make_loads(R, E, 1024, 4, skew, 0.25, seed)
    if u_min > 1:
        om = loads.omega
        loads = Loads(torch.where((om > 0) & (om < u_min), torch.full_like(om, u_min), om))
    topo = Topology.from_nvlink_rdma(nodes, gpus)
    n_slot = -(-E // R) + extra
    spec = ProblemSpec.uniform_main_placement(E, R, 3 * 512 * 256 * 2, 512 * 2, n_slot)
    cfg = EPLBConfig(u_min=u_min)
    return loads, topo, spec, cfg


@pytest.mark.parametrize("case", GRID)
def test_device_solver_matches_host_restatement(case):
    loads, topo, spec, cfg = _problem(*case, device="cuda")
    want = solve_device_semantics(loads, topo, spec, cfg)
    got = solve(Loads(loads.omega.cuda()), topo, spec, cfg)
    assert got.x.is_cuda and got.q.dtype == torch.int64
    assert torch.equal(got.x.cpu(), want.x)
    assert torch.equal(got.q.cpu(), want.q)
    assert int(got.theta) == int(want.theta)
    rep = check_constraints(got.to("cpu"), loads, topo, spec, cfg)
    assert rep.ok, rep.violations


@pytest.mark.parametrize("case", GRID[:6])
def test_quality_close_to_serial_solver(case):
    loads, topo, spec, cfg = _problem(*case, device="cuda")
    serial = solve_exact(loads, topo, spec, cfg)
    dev = solve(Loads(loads.omega.cuda()), topo, spec, cfg)
    assert int(dev.theta) <= 1.25 * int(serial.theta) + 1


def test_repeat_solves_are_bit_identical():
    loads, topo, spec, cfg = _problem(2, 4, 128, 2, 1.5, 11, 1, "cuda")
    om = Loads(loads.omega.cuda())
    first = solve(om, topo, spec, cfg)
    for _ in range(5):
        again = solve(om, topo, spec, cfg)
        assert first.equals(again)


def test_probe_mode_matches_host_and_full_run_theta():
    loads, topo, spec, _ = _problem(2, 4, 64, 2, 1.5, 12, 1, "cuda")
    om = Loads(loads.omega.cuda())
    full = solve(om, topo, spec, EPLBConfig())
    probe = solve(om, topo, spec, EPLBConfig(stage2_patience_all_scales=True))
    assert int(probe.theta) == int(full.theta)
    rep = check_constraints(probe.to("cpu"), loads, topo, spec)
    assert rep.ok, rep.violations


def test_warm_solve_has_no_host_sync():
    loads, topo, spec, cfg = _problem(2, 4, 64, 2, 1.4, 13, 1, "cuda")
    om = Loads(loads.omega.cuda())
    solve(om, topo, spec, cfg)
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        plan = solve(om, topo, spec, cfg, validate=False)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    assert isinstance(plan.theta, torch.Tensor) and plan.theta.is_cuda
