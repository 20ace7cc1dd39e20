"""Data model, metrics, physical routing, trace files, profiling line formats, rebalancer ring."""

from collections import OrderedDict

import pytest
import torch

from ep_balance_b200 import (EPLBConfig, EPLBRebalancer, Loads, Plan, ProblemSpec, Topology, check_constraints,
                             compute_metrics, solve)
from ep_balance_b200.core import trace as tr
from ep_balance_b200.parallel.physical import assign_physical, build_phys_slot_table
from ep_balance_b200.utils import profiling
from ep_balance_b200.utils.workload import make_loads


def test_config_validation():
    with pytest.raises(ValueError):
        EPLBConfig(u_min=0)
    assert EPLBConfig(eta_milli=1500).eta == 1.5 and EPLBConfig().device_stage2_iters == 64


def test_topology_and_spec_validation():
    t = Topology.from_nvlink_rdma(2, 4)
    assert t.num_ranks == 8 and t.num_domains == 2 and t.ranks_in_domain(1).tolist() == [4, 5, 6, 7]
    assert int(t.cost[0, 1]) == 1 and int(t.cost[0, 4]) == 8 and int(t.cost[3, 3]) == 0
    bad = Topology(torch.tensor([0, 2]), torch.zeros(2, 2))
    with pytest.raises(ValueError):
        bad.validate()
    with pytest.raises(ValueError):
        Topology(torch.tensor([0, 0]), torch.ones(2, 2)).validate()
    assert Topology(torch.tensor([0, 1]), torch.zeros(2, 2)).sync_free_num_domains == 2
    with pytest.raises(ValueError):
        ProblemSpec.uniform_main_placement(8, 2, 10, 1, 3)
    s = ProblemSpec.contiguous_main_placement(8, 2, 10, 1, 5)
    assert s.main_rank.tolist() == [0, 0, 0, 0, 1, 1, 1, 1]


def test_metrics_and_constraint_violations():
    topo = Topology.from_nvlink_rdma(1, 2, intra_cost=3)
    spec = ProblemSpec.uniform_main_placement(2, 2, 100, 1, 2)
    loads = Loads(torch.tensor([[4, 0], [2, 2]]))
    plan = solve(loads, topo, spec)
    m = compute_metrics(plan, loads, topo, spec, EPLBConfig(alpha=2, beta=1, gamma=1))
    assert m.mean_load == 4.0 and m.theta == int(plan.theta)
    assert m.phi_token == int((plan.q.sum(1) * topo.cost).sum())
    assert m.objective == 2 * m.theta + m.phi_token + m.phi_weight
    # break things one at a time
    q = plan.q.clone(); q[0, 0, 0] += 1
    assert any(v.startswith("C1") for v in check_constraints(Plan(plan.x, q, plan.theta), loads, topo, spec).violations)
    x = plan.x.clone(); x[0, 0] = 0
    rep = check_constraints(Plan(x, plan.q, plan.theta), loads, topo, spec)
    assert any(v.startswith("C7") for v in rep.violations)
    assert any(v.startswith("C3") for v in check_constraints(Plan(plan.x, plan.q, 99), loads, topo, spec).violations)
    tight = ProblemSpec(2, spec.main_rank, spec.weight_bytes, 1, 1)
    full = Plan(torch.ones(2, 2, dtype=torch.int8), plan.q, plan.theta)
    assert any(v.startswith("C4") for v in check_constraints(full, loads, topo, tight).violations)


@pytest.mark.parametrize("seed", range(6))
def test_assign_physical_matches_host_loop(seed):
    R, E, n_slot = 8, 16, 4
    topo = Topology.from_nvlink_rdma(2, 4)
    spec = ProblemSpec.uniform_main_placement(E, R, 1000, 100, n_slot)
    loads = make_loads(R, E, 48, 2, 1.5, 0.25, seed)
    plan = solve(loads, topo, spec)
    table = build_phys_slot_table(plan.x, n_slot)
    g = torch.Generator().manual_seed(seed)
    for src in range(R):
        ue = torch.repeat_interleave(torch.arange(E), loads.omega[src])
        ue = ue[torch.randperm(ue.numel(), generator=g)]
        phys, dst = assign_physical(ue, plan, spec, src)
        left = plan.q[src].clone()
        for u, e in enumerate(ue.tolist()):
            host = int((left[e] > 0).nonzero()[0])
            left[e, host] -= 1
            assert int(dst[u]) == host and int(phys[u]) == int(table[e, host])
        assert int(left.sum()) == 0
        # physical id -> (rank, slot) -> expert inverse
        assert torch.equal(phys // n_slot, dst)


def test_trace_round_trip_and_analysis(tmp_path):
    topo = Topology.from_nvlink_rdma(2, 2)
    spec = ProblemSpec.contiguous_main_placement(8, 4, 1000, 64, 4)
    w = tr.TraceWriter(str(tmp_path / "t.pt"), tr.build_trace_meta(topo, spec), every=2)
    for i in range(5):
        w.add(layer=i % 2, mb=i // 2, omega=make_loads(4, 8, 32, 2, 1.2, 0.25, i).omega)
    w.flush()
    t = tr.load_routing_trace(tmp_path / "t.pt")
    assert t["meta"]["format_version"] == 3 and t["meta"]["n_slot"] == 4
    assert t["meta"]["omega_semantics"] == "source_ep_rank_by_logical_expert_token_assignments"
    layers, cube = tr.expert_count_cube(t)
    assert layers == [0, 1] and tuple(cube.shape) == (2, 2, 8)
    _, per, agg = tr.expert_max_mean_by_layer(t)
    assert per.shape == (2, 2) and bool((agg >= 1).all())
    _, snap = tr.select_expert_count_matrix(t, view="snapshot", occurrence=1)
    _, ag = tr.select_expert_count_matrix(t, view="aggregate")
    assert torch.equal(ag, cube.sum(1)) and torch.equal(snap, cube[:, 1])
    assert torch.allclose(tr.normalize_expert_counts(ag, "share").sum(1), torch.ones(2, dtype=torch.float64))
    rows = tr.metric_rows(label="x", view="aggregate", layers=layers, expert_counts=ag, meta=t["meta"])
    assert rows[0]["total_assignments"] == int(ag[0].sum()) and rows[0]["rank_max_mean"] >= 1
    topo2, spec2 = tr.spec_and_topology_from_meta(t["meta"])
    assert torch.equal(topo2.cost, topo.cost) and torch.equal(spec2.main_rank, spec.main_rank)
    # legacy key
    legacy = {"meta": t["meta"], "samples": [{"layer": 0, "lam": t["samples"][0]["omega"]}]}
    torch.save(legacy, tmp_path / "old.pt")
    assert "omega" in tr.load_routing_trace(tmp_path / "old.pt")["samples"][0]
    torch.save({"meta": t["meta"], "samples": []}, tmp_path / "bad.pt")
    with pytest.raises(ValueError):
        tr.load_routing_trace(tmp_path / "bad.pt")


def _debug_window(monkeypatch):
    monkeypatch.setattr(profiling, "_P", profiling.Profiler(debug=True))
    profiling.begin_debug_window()


def test_debug_timing_line_format(monkeypatch):
    _debug_window(monkeypatch)
    with profiling.record("solve", time_it=True, device="cpu"):
        pass
    for _ in range(2):
        with profiling.record("apply/dispatch", time_it=True, device="cpu", payload_bytes=4 * 1024 * 1024):
            pass
    lines = []
    profiling.maybe_summary(lines.append, context="layer=3 mb=7")
    assert len(lines) == 1 and lines[0].startswith("[EPLB-debug] layer=3 mb=7 ")
    assert "solver=" in lines[0] and "dispatch=" in lines[0] and "ms(x2)" in lines[0]
    assert "/8.00MiB/" in lines[0] and "GB/s" in lines[0]
    assert not profiling.current().window
    with profiling.record("apply/grad_move", time_it=True, device="cpu"):
        pass
    profiling.begin_debug_window()  # backward phases are reported at the next window
    assert any("direction=backward" in l and "expert_grad_reduce=" in l for l in lines)


def test_profile_table_and_rank_reduction(monkeypatch):
    monkeypatch.setattr(profiling, "_P", profiling.Profiler(profile=True, every=2, rank="3"))
    lines = []
    for _ in range(2):
        with profiling.record("apply/expert_gemm", time_it=True, device="cpu", payload_bytes=1 << 20):
            pass
        profiling.maybe_summary(lines.append)
    assert len(lines) == 1 and lines[0].startswith("[EPLB-profile r3] region")
    assert "apply/expert_gemm" in lines[0] and "peak memory" in lines[0]
    assert profiling.stats()["apply/expert_gemm"].count == 2 and profiling.last_ms("apply/expert_gemm") >= 0.0
    mean_max = profiling.reduce_over_ranks()  # no process group: this rank alone
    assert set(mean_max) == {"apply/expert_gemm"} and mean_max["apply/expert_gemm"][0] == mean_max["apply/expert_gemm"][1]
    profiling.reset()
    assert "no samples" in profiling.summary_str()


def test_rebalancer_ring_and_backward():
    topo = Topology.from_nvlink_rdma(1, 4)
    spec = ProblemSpec.uniform_main_placement(8, 4, 1000, 100, 4)
    reb = EPLBRebalancer(topo, spec, ring_size=2)
    plans = {}
    for mb in range(3):
        plans[mb] = reb.rebalance_from_omega(make_loads(4, 8, 32, 2, 1.5, 0.25, mb), 0, mb).plan
    assert reb.backward(0, 2).equals(plans[2]) and reb.backward(0, 1).equals(plans[1])
    with pytest.raises(KeyError):
        reb.backward(0, 0)  # evicted
    off = EPLBRebalancer(topo, spec, ring_size=0)
    off.rebalance_from_omega(make_loads(4, 8, 32, 2, 1.5, 0.25, 0), 0, 0)
    with pytest.raises(KeyError):
        off.backward(0, 0)
    cached = EPLBRebalancer(topo, spec, cache_plans=True)
    p = cached.rebalance_from_omega(make_loads(4, 8, 32, 2, 1.5, 0.25, 9), 1, 1).plan
    assert cached.backward(1, 1) is p
    cached.clear()
    with pytest.raises(KeyError):
        cached.backward(1, 1)
