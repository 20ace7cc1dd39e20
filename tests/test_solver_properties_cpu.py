"""Property tests: for ANY load matrix and topology the host solvers return plans that satisfy the
constraints C1-C7 (conservation, reachability, theta consistency, slot budget, quota floor, cross-domain
gate, fixed owners) and are deterministic."""

import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from ep_balance_b200 import EPLBConfig, Loads, ProblemSpec, Topology, check_constraints
from ep_balance_b200.solver import solve_device_semantics, solve_exact


@st.composite
def problems(draw):
    nodes = draw(st.integers(1, 3))
    gpus = draw(st.integers(1, 4))
    R = nodes * gpus
    per_rank = draw(st.integers(1, 4))
    E = R * per_rank
    extra = draw(st.integers(0, 3))
    u_min = draw(st.sampled_from([1, 1, 1, 2, 4]))
    hot = draw(st.integers(0, E - 1))
    scale = draw(st.sampled_from([1, 8, 200, 5000]))
    cells = draw(st.lists(st.integers(0, scale), min_size=R * E, max_size=R * E))
    omega = torch.tensor(cells, dtype=torch.int64).view(R, E)
    omega[:, hot] *= draw(st.integers(1, 20))                 # one expert much hotter than the rest
    if u_min > 1:                                             # the quota floor is only feasible for cells that are 0 or >= u_min
        omega = torch.where((omega > 0) & (omega < u_min), torch.full_like(omega, u_min), omega)
    weight_bytes = draw(st.sampled_from([64, 4096, 1 << 20]))
    s_tok = draw(st.sampled_from([16, 512, 4096]))
    contiguous = draw(st.booleans())
    spec = (ProblemSpec.contiguous_main_placement if contiguous else ProblemSpec.uniform_main_placement)(
        E, R, weight_bytes, s_tok, per_rank + extra)
    cfg = EPLBConfig(u_min=u_min, allow_cross_domain=draw(st.booleans()))
    return Loads(omega), Topology.from_nvlink_rdma(nodes, gpus), spec, cfg


@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(problems())
def test_exact_solver_properties(problem):
    loads, topo, spec, cfg = problem
    plan = solve_exact(loads, topo, spec, cfg)
    rep = check_constraints(plan, loads, topo, spec, cfg)
    assert rep.ok, rep.violations
    again = solve_exact(loads, topo, spec, cfg)
    assert plan.equals(again)


@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(problems())
def test_device_semantics_solver_properties(problem):
    loads, topo, spec, cfg = problem
    plan = solve_device_semantics(loads, topo, spec, cfg)
    rep = check_constraints(plan, loads, topo, spec, cfg)
    assert rep.ok, rep.violations
    assert plan.equals(solve_device_semantics(loads, topo, spec, cfg))
    # owners are never moved, and every unit is routed somewhere: total load is conserved
    assert int(plan.q.sum()) == int(loads.omega.sum())
    assert bool((plan.x[torch.arange(spec.num_experts), spec.main_rank] == 1).all())
