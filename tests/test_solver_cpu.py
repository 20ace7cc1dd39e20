"""Host solvers: constraint validity on a grid, determinism, exact small cases, and decision-for-
decision equality with the upstream serial solver when it is importable (reference strategy:
tests/test_constraints.py, test_determinism.py, test_incremental_solver.py, test_bisect.py)."""

import pytest
import torch

from ep_balance_b200 import EPLBConfig, Loads, Plan, ProblemSpec, Topology, check_constraints, compute_metrics, solve
from ep_balance_b200.solver import solve_bisect, solve_device_semantics, solve_exact
from ep_balance_b200.solver.exact import plan_quota_transfer, waterfill
from ep_balance_b200.utils.workload import make_loads, softmax_router_loads

GRID = [(1, 4, 8, 3, 1.0), (2, 4, 64, 10, 1.5), (4, 8, 64, 4, 1.5), (2, 2, 16, 6, 2.0), (4, 2, 40, 7, 1.2), (1, 8, 32, 5, 0.8)]


def _case(nodes, gpus, E, n_slot, skew, seed=0, tokens=512, top_k=4):
    R = nodes * gpus
    return (make_loads(R, E, tokens, top_k, skew, 0.25, seed), Topology.from_nvlink_rdma(nodes, gpus),
            ProblemSpec.uniform_main_placement(E, R, 3 * 256 * 512 * 2, 512, n_slot))


@pytest.mark.parametrize("case", GRID)
@pytest.mark.parametrize("solver", [solve_exact, solve_device_semantics, solve_bisect])
def test_plans_satisfy_all_constraints(case, solver):
    loads, topo, spec = _case(*case)
    plan = solver(loads, topo, spec, EPLBConfig())
    rep = check_constraints(plan, loads, topo, spec)
    assert rep.ok, rep.violations
    m = compute_metrics(plan, loads, topo, spec)
    assert m.theta == int(plan.theta) and m.max_slots_used <= spec.n_slot
    assert m.objective == m.theta + m.phi_token + m.phi_weight


@pytest.mark.parametrize("case", GRID)
def test_exact_solver_equals_upstream_decisions(case, ref_eplb):
    loads, topo, spec = _case(*case, seed=3)
    mine = solve_exact(loads, topo, spec, EPLBConfig())
    nodes, gpus = case[0], case[1]
    rtopo = ref_eplb.Topology.from_nvlink_rdma(nodes, gpus)
    rspec = ref_eplb.ProblemSpec.uniform_main_placement(spec.num_experts, nodes * gpus, 3 * 256 * 512 * 2, 512, spec.n_slot)
    theirs = ref_eplb.solve(ref_eplb.Loads(loads.omega), rtopo, rspec, ref_eplb.EPLBConfig())
    assert torch.equal(mine.x, theirs.x) and torch.equal(mine.q, theirs.q) and int(mine.theta) == int(theirs.theta)


def test_bisect_equals_upstream(ref_eplb):
    import eplb.algorithm as ra

    loads, topo, spec = _case(2, 4, 32, 6, 1.5, seed=5)
    mine = solve_bisect(loads, topo, spec)
    theirs = ra.solve_bisect(ref_eplb.Loads(loads.omega), ref_eplb.Topology.from_nvlink_rdma(2, 4),
                             ref_eplb.ProblemSpec.uniform_main_placement(32, 8, 3 * 256 * 512 * 2, 512, 6))
    assert torch.equal(mine.x, theirs.x) and torch.equal(mine.q, theirs.q)


def test_u_min_floor_is_respected():
    loads, topo, spec = _case(2, 4, 64, 10, 1.5, seed=4)
    om = loads.omega
    loads = Loads(torch.where((om > 0) & (om < 4), torch.full_like(om, 4), om))
    for solver in (solve_exact, solve_device_semantics):
        plan = solver(loads, topo, spec, EPLBConfig(u_min=4))
        rep = check_constraints(plan, loads, topo, spec, EPLBConfig(u_min=4))
        assert rep.ok, rep.violations
    with pytest.raises(ValueError):
        solve(Loads(torch.tensor([[1, 0], [0, 9]])), Topology.from_nvlink_rdma(1, 2),
              ProblemSpec.uniform_main_placement(2, 2, 10, 1, 2), EPLBConfig(u_min=4))


def test_repeat_and_noncontiguous_inputs_give_identical_plans():
    loads, topo, spec = _case(2, 4, 32, 6, 1.3, seed=7)
    a = solve(loads, topo, spec)
    b = solve(loads, topo, spec)
    wide = torch.zeros(8, 64, dtype=torch.int64)
    wide[:, ::2] = loads.omega
    c = solve(Loads(wide[:, ::2]), topo, spec)
    assert a.equals(b) and a.equals(c) and a.digest() == c.digest()


def test_tiny_exact_cases():
    topo = Topology.from_nvlink_rdma(1, 2)
    spec = ProblemSpec.uniform_main_placement(1, 2, 10, 1, 2)
    plan = solve(Loads(torch.tensor([[11], [0]])), topo, spec)
    assert sorted(plan.rank_load().tolist()) == [5, 6] and int(plan.theta) == 6
    assert plan.x.tolist() == [[1, 1]]
    # no slot to spare: nothing can move
    spec1 = ProblemSpec.uniform_main_placement(2, 2, 10, 1, 1)
    plan1 = solve(Loads(torch.tensor([[9, 1], [9, 1]])), topo, spec1)
    assert plan1.rank_load().tolist() == [18, 2] and int(plan1.x.sum()) == 2


def test_cross_domain_gate():
    topo = Topology.from_nvlink_rdma(2, 1)
    # expert 0 lives on rank 0; rank 1 (other domain) sends it 10 units of 4 bytes: 2*10*4=80
    omega = torch.tensor([[0, 0], [10, 0]])
    heavy = ProblemSpec(2, torch.tensor([0, 1]), torch.tensor([80, 80]), 4, 2)
    light = ProblemSpec(2, torch.tensor([0, 1]), torch.tensor([79, 79]), 4, 2)
    for solver in (solve_exact, solve_device_semantics):
        assert int(solver(Loads(omega), topo, heavy).x[0, 1]) == 0  # 80 < 80 is false: not admitted
        p = solver(Loads(omega), topo, light)
        assert int(p.x[0, 1]) == 1 and int(p.q[1, 0, 1]) == 10
        off = solver(Loads(omega), topo, light, EPLBConfig(allow_cross_domain=False))
        assert int(off.x[0, 1]) == 0


def test_waterfill_and_quota_transfer_units():
    assert waterfill(10, [0, 0, 0], [0, 0, 0]) == [4, 3, 3]
    assert waterfill(5, [10, 0], [0, 0]) == [0, 5]
    assert waterfill(12, [10, 0], [0, 0]) == [1, 11]
    assert sum(waterfill(7, [3, 1, 2], [1, 1, 0], 2)) == 7
    import numpy as np

    mv, tot = plan_quota_transfer(np.array([5, 5]), np.array([0, 0]), 6, 1)
    assert mv.tolist() == [5, 1] and tot == 6
    mv, tot = plan_quota_transfer(np.array([5, 5]), np.array([0, 0]), 6, 4)
    assert mv.tolist() == [5, 0] and tot == 5  # second source cannot leave or give a fragment < 4


def test_device_semantics_quality_vs_serial():
    for case in GRID:
        loads, topo, spec = _case(*case, seed=11)
        assert int(solve_device_semantics(loads, topo, spec).theta) <= 1.25 * int(solve_exact(loads, topo, spec).theta) + 1


def test_headline_cpu_plan_config():
    """E=64, R=8 as 2x4, +2 slots, top-6 of softmax(g/0.5) with Dirichlet(5) per-rank perturbation."""
    loads = softmax_router_loads(8, 64, 4096, 6, tau=0.5, dirichlet_alpha=5.0, seed=0)
    assert int(loads.omega.sum()) == 8 * 4096 * 6
    topo = Topology.from_nvlink_rdma(2, 4)
    spec = ProblemSpec.uniform_main_placement(64, 8, 3 * 2048 * 1408 * 2, 2048 * 2, 10)
    plan = solve(loads, topo, spec)
    assert check_constraints(plan, loads, topo, spec).ok
    before = compute_metrics(Plan(*_no_balance(loads, spec)), loads, topo, spec).imbalance
    after = compute_metrics(plan, loads, topo, spec).imbalance
    assert after < before and after < 1.35
    assert plan.digest() == solve(loads, topo, spec).digest()


def _no_balance(loads, spec):
    R, E = loads.omega.shape
    x = torch.zeros(E, R, dtype=torch.int8)
    x[torch.arange(E), spec.main_rank] = 1
    q = torch.zeros(R, E, R, dtype=torch.int64)
    q[:, torch.arange(E), spec.main_rank] = loads.omega
    return x, q, int(q.sum((0, 1)).max())
