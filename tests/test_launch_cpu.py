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


def test_preflight_accepts_the_defaults_and_names_bad_knobs(tmp_path):
    from ep_balance_b200.launch.preflight import check, main

    ok = check({}, 8)
    assert ok.ok and ok.resolved["n_slot"] == 10 and ok.resolved["replica_slots"] == 2 and ok.resolved["adapter"] == "fused"
    assert check({"GPUS_PER_NODE": "4"}, 8).resolved["domains"] == 2

    def errors(env, nproc=8, **kw):
        return " | ".join(check(env, nproc, **kw).errors)

    assert "EPLB_N_SLOT=4 is below the 8 experts" in errors({"EPLB_N_SLOT": "4"})
    assert "does not divide the 64 experts" in errors({}, nproc=6)
    assert "GPUS_PER_NODE=3 does not divide" in errors({"GPUS_PER_NODE": "3"})
    assert "EPLB_ADAPTER=deepep" in errors({"EPLB_ADAPTER": "deepep"})
    assert "EPLB_MODE='bogus'" in errors({"EPLB_MODE": "bogus"})
    assert "EPLB_GIN_LSA is set" in errors({"EPLB_GIN_LSA": "0"})
    assert "MODEL='nope'" in errors({"MODEL": "nope"})
    assert "ROUTER_BALANCING='sinkhorn'" in errors({"ROUTER_BALANCING": "sinkhorn"})
    assert "is not an integer" in errors({"EPLB_N_SLOT": "ten"})
    shape = dict(layers=2, hidden=2000, heads=8, ffn=1000, experts=64, top_k=2)
    e = errors({}, shape=shape)
    assert "hidden % 64" in e and "ffn % 128" in e
    assert not check({"EPLB_ADAPTER": "alltoall"}, 8, shape=shape).errors       # the portable path has no such rule
    assert "EPLB_CHUNKS=3" in errors({"EPLB_ADAPTER": "alltoall", "EPLB_CHUNKS": "3"})
    assert "needs EPLB_WEIGHT_COMM=broadcast" in errors({"EPLB_ADAPTER": "alltoall", "EPLB_REMATERIALIZE": "1",
                                                          "EPLB_WEIGHT_COMM": "gin"})
    assert "does not exist" in errors({"EPLB_TRACE_OUT": str(tmp_path / "missing" / "t.pt")})
    w = check({"EPLB_N_SLOT": "8", "ROUTER_SKEW": "-0.5", "ROUTER_BALANCING": "aux_loss", "EPLB_CHUNKS": "2"}, 8)
    assert w.ok and len(w.warnings) >= 3 and "[preflight] WARNING" in w.report()
    assert main(["--nproc", "8"]) == 0


def test_aux_loss_switch_changes_the_router_gradient():
    import torch

    from ep_balance_b200.models.moe_layer import FusedMoE, MoEConfig

    # route_tokens needs no device: drive it on a bare object with the attributes it reads
    layer = FusedMoE.__new__(FusedMoE)
    torch.nn.Module.__init__(layer)
    layer.cfg = MoEConfig(hidden=16, ffn=128, num_experts=8, top_k=2, max_tokens=32, aux_loss_coeff=0.5)
    layer.router = torch.nn.Parameter(torch.randn(8, 16))
    layer.router_bias, layer.route_fn, layer.fused_router, layer.aux_loss = None, None, None, None
    x = torch.randn(32, 16)
    idx, prob = layer.route_tokens(x)
    assert idx.shape == (32, 2) and layer.aux_loss is not None and float(layer.aux_loss) > 0
    layer.aux_loss.backward()
    assert layer.router.grad is not None and float(layer.router.grad.abs().sum()) > 0
    with torch.no_grad():
        layer.route_tokens(x)
    assert layer.aux_loss is None


def test_shell_entry_points_parse():
    """The launcher and the machine bootstrap are shell scripts: at least their syntax is checked here."""
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for script in ("run_train.sh", "bootstrap.sh"):
        path = os.path.join(root, "ep_balance_b200", "launch", script)
        assert os.access(path, os.X_OK), script
        assert subprocess.run(["bash", "-n", path], capture_output=True).returncode == 0, script


def test_bring_up_recipe_passes_preflight():
    from ep_balance_b200.launch import recipes
    from ep_balance_b200.launch.preflight import check

    tiny = recipes.recipe("tiny")
    assert (tiny["layers"], tiny["hidden"], tiny["experts"], tiny["top_k"]) == (4, 512, 8, 2)
    for mode in ("observe", "apply"):
        for nproc in (1, 2, 4, 8):
            res = check({"MODEL": "tiny", "EPLB_MODE": mode}, nproc)
            assert res.ok, (mode, nproc, res.errors)


def test_preflight_knows_the_padded_adapter_and_refuses_the_fused_one_across_nodes():
    from ep_balance_b200.launch.preflight import check

    assert "EPLB_PAIR_ROWS" in " ".join(check({"EPLB_ADAPTER": "padded", "EPLB_MODE": "apply"}, 8).errors)
    assert check({"EPLB_ADAPTER": "padded", "EPLB_MODE": "apply", "EPLB_PAIR_ROWS": "4096"}, 8).ok
    assert "one node" in " ".join(check({"NNODES": "4"}, 8).errors)
    assert check({"NNODES": "4", "EPLB_ADAPTER": "alltoall"}, 8).ok
