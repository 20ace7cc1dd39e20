"""The one-line JSON contract of bench.py (no GPU needed: only the line builder is exercised)."""

import argparse
import importlib.util
import json
import os


def _bench():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    spec = importlib.util.spec_from_file_location("bench_under_test", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_both_arms_emit_the_same_config_and_all_required_keys(capsys):
    bench = _bench()
    args = argparse.Namespace(tokens=8192, steps=20, warmup=5)
    clocks = {"sm_mhz": 1900.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"]}
    quality = {"rank_load_max_over_mean": 1.1, "replicas": 16, "plan_digest": "ab"}
    lines = []
    for impl, launches in (("ours", 300), ("reference", 0)):
        bench.emit(args, 8, impl, 4.0, 4.2, launches, clocks, 8192 * 2048 * 2, 4, quality, {"arm": impl})
        lines.append(json.loads(capsys.readouterr().out.strip().splitlines()[-1]))
    ours, ref = lines
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "impl"):
        assert key in ours, key
    assert ours["config"] == ref["config"]                       # arm-specific prose lives in `notes`, not in `config`
    assert {"model", "global_batch", "seq_len", "parallelism"} <= set(ours["config"])
    assert ours["metric"] == "moe_layer_train_tokens_per_s" and ours["higher_is_better"] is True and ours["scaling"] == "weak"
    assert ours["n_gpus"] == 8 and ours["config"]["global_batch"] == 8 * 8192 and ours["config"]["parallelism"] == "ep8"
    assert abs(ours["value"] - 8 * 8192 / 4.0e-3) < 1e-6          # whole-job tokens/s from the device-timed step
    assert abs(ours["e2e"]["value"] - 8 * 8192 / 4.2e-3) < 1e-6
    assert ours["e2e"]["h2d_bytes_per_step"] == 8192 * 2048 * 2 and ours["e2e"]["d2h_bytes_per_step"] == 4
    assert ours["gpu_launches"] == 300 and ref["impl"] == "reference"
    assert set(ours["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}


def test_defaults_finish_quickly_and_flags_exist(monkeypatch):
    import sys

    bench = _bench()
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    a = bench.parse()
    assert a.gpus == 1 and a.steps <= 50 and a.warmup >= 3 and a.impl == "ours" and a.tokens == 8192
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--gpus", "8", "--steps", "10", "--warmup", "3"])
    a = bench.parse()
    assert (a.impl, a.gpus, a.steps, a.warmup) == ("reference", 8, 10, 3)
