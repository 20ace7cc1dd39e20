"""Baseline policies, the harness, trace replay and the simulators (reference: tests/test_baselines.py)."""

import json

import pytest
import torch

from ep_balance_b200 import Loads, ProblemSpec, Topology
from ep_balance_b200.baselines import (ShadowCostModel, flexmoe_schedule, rebalance_experts, run_deepseek_eplb,
                                       run_fastermoe, run_flexmoe, run_scale_eplb, select_shadow_experts, slot_budget)
from ep_balance_b200.baselines import benchmark as bm
from ep_balance_b200.baselines.adapters import LPLBBaseline, LPLBUnavailableError, select_lplb_topology
from ep_balance_b200.core import trace as tr
from ep_balance_b200.utils.workload import make_loads


def test_n_slot_counts_only_additional_replicas():
    assert slot_budget(640, 32, 4) == (20, 4, 24)
    with pytest.raises(ValueError):
        slot_budget(10, 4, 1)


def test_deepseek_eplb_published_example():
    weight = torch.tensor([[90, 132, 40, 61, 104, 165, 39, 4, 73, 56, 183, 86],
                           [20, 107, 104, 64, 19, 197, 187, 157, 172, 86, 16, 27]])
    phy2log, log2phy, logcnt = rebalance_experts(weight, 16, 4, 2, 8)
    assert phy2log.tolist() == [[5, 6, 5, 7, 8, 4, 3, 4, 10, 9, 10, 2, 0, 1, 11, 1],
                                [7, 10, 6, 8, 6, 11, 8, 9, 2, 4, 5, 1, 5, 0, 3, 1]]
    assert bool((logcnt >= 1).all()) and bool((log2phy[:, :, 0] >= 0).all()) and int(logcnt.sum()) == 32


def _setup(seed=0, R=8, E=64, extra=2):
    loads = make_loads(R, E, 1024, 4, 1.5, 0.25, seed)
    topo = Topology.from_nvlink_rdma(2, R // 2)
    spec = ProblemSpec.uniform_main_placement(E, R, 3 * 512 * 256 * 2, 1024, E // R + extra)
    return loads, topo, spec


def test_every_strategy_conserves_load_and_respects_the_slot_budget():
    loads, topo, spec = _setup()
    total = float(loads.omega.sum())
    results = [run_scale_eplb(loads, topo, spec),
               run_deepseek_eplb(loads, num_nodes=2, num_gpus=8, n_slot=2, num_groups=8),
               run_fastermoe(loads, spec, num_ranks=8, n_slot=2), run_flexmoe(loads, spec, num_ranks=8, n_slot=2)]
    base = bm.no_balance_result(loads, spec, 8)
    for r in results:
        assert abs(float(r.rank_load.double().sum()) - total) < 1e-6 * total, r.name
        assert r.metadata["replicas"] <= r.metadata["replica_budget"], r.name
        assert r.imbalance <= base.imbalance + 1e-9, r.name
        assert int((r.placement > 0).sum(0).max()) <= r.metadata["physical_slots_per_rank"], r.name
    assert results[1].metadata["replicas"] == 16  # DeepSeek-EPLB always fills every slot


def test_fastermoe_stops_when_the_model_predicts_no_gain():
    loads, _, spec = _setup(seed=2)
    free = ShadowCostModel(bw_net=1e15)  # broadcasting weights is free -> shadow as much as slots allow
    costly = ShadowCostModel(bw_net=1.0, comm_rounds=0)  # only the broadcast pays the slow link -> shadow nothing
    m_free, _ = select_shadow_experts(loads.omega, spec.main_rank, spec.weight_bytes, spec.s_tok, 8, free, 2)
    m_cost, load = select_shadow_experts(loads.omega, spec.main_rank, spec.weight_bytes, spec.s_tok, 8, costly, 2)
    assert 0 < int(m_free.sum()) <= 2 and int(m_cost.sum()) == 0
    assert torch.allclose(load, bm.no_balance_result(loads, spec, 8).rank_load)


def test_flexmoe_expands_hot_experts_only_above_threshold():
    uniform = torch.full((4, 8), 10)
    n, load, x = flexmoe_schedule(uniform, torch.ones(8), 4, 2)
    assert n == [1] * 8 and float(load.max()) == 80.0 and int(x.sum()) == 8
    hot = uniform.clone()
    hot[:, 0] = 200
    n, load, _ = flexmoe_schedule(hot, torch.ones(8), 4, 2)
    assert n[0] > 1 and sum(n) <= 8 + 8


def test_lplb_is_reported_unavailable_and_topology_selection():
    with pytest.raises(LPLBUnavailableError):
        LPLBBaseline(num_experts=64, num_ranks=8, n_slot=2)
    assert select_lplb_topology("auto", 3)[0] == "ring" and select_lplb_topology("auto", 4)[0] == "cube"
    assert select_lplb_topology("cube", 1)[1].shape == (16, 2)


def test_harness_rows_and_json(capsys):
    rows = bm.main(["--nodes", "2", "--gpus-per-node", "4", "--experts", "64", "--n-slot", "2", "--tokens-per-rank", "512",
                    "--iterations", "1", "--warmup", "0", "--include-no-balance", "--details", "--json",
                    "--strategies", "scale,eplb,fastermoe,flexmoe,lplb", "--device", "cpu"])
    parsed = json.loads(capsys.readouterr().out)
    names = [r["strategy"] for r in parsed]
    assert names == ["no-balance", "scale-eplb", "deepseek-eplb", "fastermoe", "flexmoe", "lplb"]
    scale = rows[1]
    assert scale["physical_slots_per_rank"] == 10 and len(scale["rank_load_by_rank"]) == 8 and scale["solve_ms"] > 0
    assert "placement_details" in scale and "unavailable" in rows[-1]
    assert scale["quality_imbalance"] < rows[0]["quality_imbalance"]


def test_trace_dump_then_replay(tmp_path):
    loads, topo, spec = _setup(R=4, E=16, extra=2)
    w = tr.TraceWriter(str(tmp_path / "t.pt"), tr.build_trace_meta(topo, spec))
    for i in range(3):
        w.add(0, i, make_loads(4, 16, 256, 2, 1.5, 0.25, i).omega)
    w.flush()
    rows = bm.main(["--trace", str(tmp_path / "t.pt"), "--strategies", "scale,eplb,flexmoe", "--num-groups", "4"])
    by = {r["strategy"]: r for r in rows}
    assert set(by) == {"no-balance", "scale-eplb", "deepseek-eplb", "flexmoe"}
    assert by["scale-eplb"]["samples"] == 3 and by["scale-eplb"]["replica_slots_per_rank"] == 2
    assert by["scale-eplb"]["imbalance"]["mean"] <= by["no-balance"]["imbalance"]["mean"]
    rows1 = bm.main(["--trace", str(tmp_path / "t.pt"), "--strategies", "scale", "--replica-slots-per-rank", "0"])
    s0 = {r["strategy"]: r for r in rows1}["scale-eplb"]
    assert s0["replica_slots_per_rank"] == 0 and s0["imbalance"]["mean"] >= by["scale-eplb"]["imbalance"]["mean"]


def test_run_sim_and_run_dist():
    from ep_balance_b200.sim import run_dist, run_sim

    out = run_sim.main(["--nodes", "2", "--gpus-per-node", "4", "--experts", "32", "--n-slot", "6", "--tokens-per-rank", "512"])
    assert out["constraints_ok"] and out["after"].imbalance <= out["before"].imbalance
    assert run_dist.main(["--world", "3", "--experts", "12", "--tokens-per-rank", "128", "--port", "6233"])
