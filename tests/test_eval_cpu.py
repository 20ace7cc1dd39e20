"""Log extractors, the skew calibrator and the figure data (reference: tests/test_plot_*.py,
test_trace_analysis.py)."""

import json

import torch

from ep_balance_b200 import ProblemSpec, Topology
from ep_balance_b200.core import trace as tr
from ep_balance_b200.eval import (calibrate_router_skew, extract_eplb_debug, extract_routing_imbalance,
                                  extract_train_metrics, plots)
from ep_balance_b200.utils.workload import make_loads


def _trace(tmp_path, layers=2, occ=3):
    topo = Topology.from_nvlink_rdma(2, 2)
    spec = ProblemSpec.contiguous_main_placement(8, 4, 1000, 64, 4)
    w = tr.TraceWriter(str(tmp_path / "t.pt"), tr.build_trace_meta(topo, spec))
    for o in range(occ):
        for l in range(layers):
            w.add(l, o, make_loads(4, 8, 64, 2, 1.5, 0.25, 10 * o + l).omega)
    w.flush()
    return tmp_path / "t.pt"


def test_debug_extractor_handles_interleaved_ranks(tmp_path):
    log = tmp_path / "run.log"
    log.write_text(
        "noise [EPLB-debug r0] mode=apply layer=0 mb=0 solver=0.050ms dispatch=2.107ms(x2)/64.00MiB/31.86GB/s "
        "expert_gemm=4.936ms combine=1.988ms/64.00MiB/33.75GB/s [EPLB-debug r1] mode=apply layer=0 mb=0 solver=0.060ms "
        "dispatch=2.000ms\n[EPLB-debug r0] mode=apply direction=backward expert_repull=1.791ms/512.00MiB/299.71GB/s "
        "expert_grad_reduce=2.031ms/512.00MiB/264.30GB/s\n[EPLB-debug r0] mode=apply layer=0 mb=1 solver=0.040ms\n")
    summary = extract_eplb_debug.main(["--log", str(log), "--out-dir", str(tmp_path / "out")])
    assert summary["records"] == 3
    assert abs(summary["phases"]["dispatch"]["mean_ms"] - 2.0535) < 1e-6
    assert abs(summary["phases"]["expert_repull"]["mean_gbps"] - 299.71) < 1e-6
    rows = extract_eplb_debug.parse([log])
    assert rows[0]["rank"] == 0 and rows[0]["expert_grad_reduce_ms"] == 2.031 and rows[1]["rank"] == 1
    assert (tmp_path / "out" / "by_rank.csv").exists() and (tmp_path / "out" / "summary.json").exists()


def test_routing_imbalance_join(tmp_path):
    t = _trace(tmp_path)
    log = tmp_path / "eplb.log"
    log.write_text("[EPLB] layer=0 mb=0 theta=70 imbalance=1.050 replicas=10 phi_token=123\n")
    out = extract_routing_imbalance.main(["--trace", str(t), "--log", str(log), "--out-dir", str(tmp_path / "o")])
    first = out["rows"][0]
    assert first["residual"] == 1.05 and 0 <= first["absorbed"] <= 1.0 and first["rank_max_mean"] >= 1.0
    assert out["summary"]["expert_max_mean"]["n"] == 6 and out["summary"]["residual"]["n"] == 1


def test_train_metrics_parser(tmp_path):
    log = tmp_path / "train.log"
    log.write_text(
        "  num_layers ...................................... 16\n  hidden_size ..................................... 2048\n"
        " [2026-01-01 00:00:00] iteration       10/     100 | consumed samples:          320 | elapsed time per iteration (ms): 812.5 |"
        " throughput per GPU (TFLOP/s/GPU): 401.2 | learning rate: 1.000000E-04 | global batch size:    32 | lm loss: 9.123456E+00 |"
        " loss scale: 1.0 | grad norm: 1.234 |\n"
        " iteration       20/     100 | consumed samples:          640 | elapsed time per iteration (ms): 800.0 |"
        " learning rate: 1.0E-04 | global batch size:    32 | lm loss: 8.5E+00 | grad norm: 1.1 |\n"
        "[Rank 0] (after 20 iterations) memory (MB) | allocated: 1.0 | max allocated: 2.0 | reserved: 3.0 | max reserved: 4096.0\n")
    out = extract_train_metrics.main(["--log", str(log), "--out-dir", str(tmp_path / "o")])
    assert out["summary"]["iterations"] == 2 and out["summary"]["ms_mean"] == 806.25
    assert out["summary"]["tflops_per_gpu_mean"] == 401.2 and out["summary"]["max_reserved_mb"] == 4096.0
    assert out["config"] == {"num_layers": "16", "hidden_size": "2048"} and out["iterations"][0]["grad_norm"] == 1.234


def test_skew_calibrator_monotone_and_target():
    out = calibrate_router_skew.main(["--experts", "32", "--topk", "2", "--ranks", "4", "--tokens", "2048", "--draws", "6",
                                      "--stds", "0", "1.0", "--target", "1.5", "--tolerance", "0.15", "--json"])
    flat, skewed = out["sweep"]
    assert flat["rank_max_mean"]["median"] < 1.1 < skewed["expert_max_mean"]["median"]
    sol = out["target"]["solution"]
    assert sol is not None and sol["router_skew"] < 0


def test_plot_commands_write_their_data(tmp_path):
    t = _trace(tmp_path)
    for cmd in ("hotspots", "max-mean-layer", "hotspots-mm"):
        res = plots.main([cmd, "--trace", str(t), "--out", str(tmp_path / f"{cmd}.png")])
        assert (tmp_path / f"{cmd}.png.json").exists() and "figure" in res
    res = plots.main(["max-mean", "--trace", str(t), str(t), "--label", "a", "b", "--out", str(tmp_path / "mm.png")])
    assert [s["label"] for s in res["series"]] == ["a", "b"] and len(res["series"][0]["mean"]) == 2
    (tmp_path / "sweep.json").write_text(json.dumps([{"n_slot": k, "rows": [{"strategy": "scale-eplb", "quality_imbalance": 2.0 / (k + 1)}]} for k in range(3)]))
    res = plots.main(["slot-sweep", "--json", str(tmp_path / "sweep.json"), "--out", str(tmp_path / "s.png")])
    assert res["series"]["scale-eplb"][0] == [0, 2.0] or res["series"]["scale-eplb"][0] == (0, 2.0)
    (tmp_path / "sc.json").write_text(json.dumps([{"sweep": "ranks", "x": 8, "min_us": 30.0}, {"sweep": "experts", "x": 64, "min_us": 25.0}]))
    res = plots.main(["solver-scaling", "--json", str(tmp_path / "sc.json"), "--out", str(tmp_path / "sc.png")])
    assert res["ranks"] == [(8, 30.0)] or res["ranks"] == [[8, 30.0]]
    assert "regions" in plots.main(["transport", "--out", str(tmp_path / "tr.png")])
