"""Recipes, slot sweep driver (reference: tests/test_model_recipes.py)."""

import pytest

from ep_balance_b200.launch import recipes, slot_sweep


def test_recipes_and_slot_defaults():
    q = recipes.recipe("qwen3_30b_a3b")
    assert (q["experts"], q["top_k"], q["hidden"]) == (128, 8, 2048)
    assert recipes.recipe("glm45_air", num_layers=4)["layers"] == 4
    with pytest.raises(KeyError):
        recipes.recipe("nope")
    assert recipes.expert_param_bytes(2048, 768) == 3 * 2048 * 768 * 2
    assert recipes.default_n_slot(128, 8) == 32 and recipes.default_n_slot(8, 8) == 2
    assert recipes.default_n_slot(128, 8, "20") == 20
    with pytest.raises(ValueError):
        recipes.default_n_slot(128, 8, "0")


def test_slot_sweep_monotone(tmp_path):
    out = slot_sweep.main(["--slots", "0", "2", "--strategies", "scale", "--json", str(tmp_path / "s.json"),
                           "--nodes", "2", "--gpus-per-node", "4", "--experts", "64", "--tokens-per-rank", "512",
                           "--iterations", "1", "--warmup", "0", "--device", "cpu"])
    imb = [[r for r in pt["rows"] if r["strategy"] == "scale-eplb"][0]["quality_imbalance"] for pt in out]
    assert imb[1] <= imb[0] and (tmp_path / "s.json").exists()


def test_env_report_runs_without_a_gpu(capsys):
    from ep_balance_b200.launch import env_check
    from ep_balance_b200.utils.env import describe_environment, problems

    info = describe_environment()
    assert info["torch"] and "cuda_available" in info
    if not info["cuda_available"]:
        assert problems(info) == ["no CUDA device is visible"]
        assert env_check.main(["--json"]) == 1
    out = capsys.readouterr().out
    assert "torch" in out or info["cuda_available"]
