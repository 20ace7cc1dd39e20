"""Our device solver against the reference's own CUDA solver on the same inputs: placement ``x`` and
quotas ``q`` must be bit-identical (the reference's device semantics are the contract).  Runs only
where the reference was installed under ``baseline/_ref`` (with its solver extension pre-built)."""

import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference():
    from ep_balance_b200.baselines.reference_install import use_reference

    if use_reference(ROOT) is None:
        pytest.skip("reference is not installed under baseline/_ref")
    import eplb

    return eplb


@pytest.mark.parametrize("ranks,experts,domains,extra,skew", [
    (8, 64, 2, 2, 1.2), (8, 64, 1, 1, 1.4), (8, 128, 4, 4, 1.0), (16, 128, 2, 2, 1.3), (32, 256, 4, 2, 1.2),
    (8, 64, 2, 0, 1.2), (4, 16, 2, 3, 1.5),
])
def test_plan_is_bit_identical_to_the_reference_cuda_solver(ranks, experts, domains, extra, skew):
    eplb = _reference()
    from ep_balance_b200 import EPLBConfig, Loads, ProblemSpec, Topology, solve
    from ep_balance_b200.utils.workload import make_loads

    dev = torch.device("cuda")
    omega = make_loads(ranks, experts, 4096, 8, skew, 0.25, 7).omega.to(dev)
    n_slot = -(-experts // ranks) + extra
    wb, s_tok = 3 * 2048 * 1408 * 2, 2048 * 2
    r_topo = eplb.Topology.from_nvlink_rdma(domains, ranks // domains, device=dev)
    r_spec = eplb.ProblemSpec.uniform_main_placement(experts, ranks, wb, s_tok, n_slot, device=dev)
    theirs = eplb.solve(eplb.Loads(omega), r_topo, r_spec, eplb.EPLBConfig(), validate=False)

    topo = Topology.from_nvlink_rdma(domains, ranks // domains)
    spec = ProblemSpec.uniform_main_placement(experts, ranks, wb, s_tok, n_slot)
    ours = solve(Loads(omega), topo, spec, EPLBConfig(), validate=False)
    torch.cuda.synchronize()
    assert torch.equal(ours.x.to(torch.int8).cpu(), theirs.x.to(torch.int8).cpu())
    assert torch.equal(ours.q.to(torch.int64).cpu(), theirs.q.to(torch.int64).cpu())
    assert int(ours.theta) == int(theirs.theta)
