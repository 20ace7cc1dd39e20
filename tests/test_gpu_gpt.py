"""Tiny GPT-MoE: loss goes down on a fixed batch (single GPU, all experts local)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tiny_gpt_moe_trains():
    from ep_balance_b200.models.gpt_moe import GPTMoE, GPTMoEConfig
    from ep_balance_b200.utils.optim import FusedAdamW

    torch.manual_seed(0)
    cfg = GPTMoEConfig(vocab=512, layers=2, hidden=256, heads=4, ffn=256, experts=8, top_k=2, seq_len=128, micro_batch=2)
    model = GPTMoE(cfg, torch.device("cuda", 0))
    dense = torch.optim.AdamW(model.dense_parameters(), lr=3e-3)
    experts = FusedAdamW(list(model.expert_parameters()), lr=3e-3, weight_decay=0.0)
    ids = torch.randint(0, 512, (2, 129), device="cuda")
    losses = []
    for _ in range(12):
        loss = model(ids[:, :-1], ids[:, 1:])
        loss.backward()
        dense.step()
        experts.step()
        dense.zero_grad(set_to_none=True)
        losses.append(float(loss))
    model.check_status()
    assert losses[-1] < losses[0] - 0.5, losses
    assert all(torch.isfinite(torch.tensor(losses)))


def test_group_limited_routing_and_dsv3_block():
    from ep_balance_b200.models.dsv3 import DSv3Config, DSv3Stack, group_limited_topk

    torch.manual_seed(0)
    logits = torch.randn(64, 32, device="cuda")
    idx, w = group_limited_topk(logits, n_groups=8, topk_groups=4, top_k=4)
    assert idx.shape == (64, 4) and torch.allclose(w.sum(-1), torch.ones(64, device="cuda"), atol=1e-5)
    assert int((idx // 4).unique(dim=1).shape[1]) <= 4 or True
    groups_used = torch.stack([torch.bincount(r // 4, minlength=8).gt(0).sum() for r in idx])
    assert int(groups_used.max()) <= 4  # never more than topk_groups groups per token

    cfg = DSv3Config(layers=2, hidden=256, ffn=256, experts=16, top_k=4, n_groups=4, topk_groups=2, shared_ffn=256,
                     max_tokens=256, num_domains=1)
    model = DSv3Stack(cfg, torch.device("cuda", 0))
    x = torch.randn(256, 256, device="cuda").bfloat16().requires_grad_(True)
    y = model(x)
    y.float().square().mean().backward()
    model.check_status()
    assert torch.isfinite(y.float()).all() and torch.isfinite(x.grad.float()).all()
    with torch.no_grad():
        y2 = model(x[:64].detach().contiguous())  # inference-only forward at a smaller batch
    assert y2.shape == (64, 256) and torch.isfinite(y2.float()).all()


def _run_train(capsys, argv, env=None):
    import os

    from ep_balance_b200.launch import train_gpt_moe

    old = {k: os.environ.get(k) for k in (env or {})}
    os.environ.update(env or {})
    try:
        assert train_gpt_moe.main(argv) == 0
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    out = capsys.readouterr().out
    from ep_balance_b200.eval.extract_train_metrics import ITER_RE

    return {int(m.group("iter")): float(m.group("loss")) for m in ITER_RE.finditer(out)}, out


TINY = ["--layers", "2", "--hidden", "256", "--heads", "4", "--ffn", "256", "--experts", "8", "--top-k", "2",
        "--vocab", "512", "--seq-len", "128", "--micro-batch", "2", "--lr", "1e-3"]


def test_training_resumes_from_a_checkpoint_with_the_same_losses(tmp_path, capsys):
    ck = str(tmp_path / "ck")
    full, _ = _run_train(capsys, TINY + ["--steps", "6", "--num-micro-batches", "2"])
    first, _ = _run_train(capsys, TINY + ["--steps", "3", "--num-micro-batches", "2", "--save", ck])
    second, out = _run_train(capsys, TINY + ["--steps", "6", "--num-micro-batches", "2", "--load", ck])
    assert "resume_step=3" in out
    assert sorted(second) == [4, 5, 6] and sorted(first) == [1, 2, 3]
    for it in (1, 2, 3):
        assert abs(first[it] - full[it]) < 1e-6
    for it in (4, 5, 6):
        assert abs(second[it] - full[it]) < 2e-3 * abs(full[it]), (it, second[it], full[it])


def test_observe_mode_logs_plans_and_writes_a_trace(tmp_path, capsys):
    from ep_balance_b200.core.trace import load_routing_trace

    trace = str(tmp_path / "trace.pt")
    _, out = _run_train(capsys, TINY + ["--steps", "2"], env={"EPLB_MODE": "observe", "EPLB_TRACE_OUT": trace,
                                                             "EPLB_TRACE_EVERY": "1"})
    assert out.count("[EPLB] layer=") == 4      # 2 layers x 2 steps
    t = load_routing_trace(trace)
    assert len(t["samples"]) == 4 and t["meta"]["num_experts"] == 8


def test_frozen_checkpoint_capture_runs_forward_only(tmp_path, capsys):
    from ep_balance_b200.core.trace import load_routing_trace

    ck, trace = str(tmp_path / "ck"), str(tmp_path / "hot.pt")
    _run_train(capsys, TINY + ["--steps", "2", "--save", ck])
    _, out = _run_train(capsys, TINY + ["--load", ck, "--skip-train", "--eval-iters", "3"],
                        env={"EPLB_MODE": "observe", "EPLB_TRACE_OUT": trace, "EPLB_TRACE_EVERY": "1"})
    assert out.count("evaluation iteration") == 3 and "iteration        3/" not in out
    assert len(load_routing_trace(trace)["samples"]) == 6      # 2 layers x 3 forward passes


@pytest.mark.parametrize("E,G,KG,K", [(256, 8, 4, 8), (64, 4, 2, 6), (32, 8, 4, 4)])
def test_fused_router_matches_the_pytorch_formulation(E, G, KG, K):
    from ep_balance_b200.models.dsv3 import group_limited_topk
    from ep_balance_b200.ops.extension import load

    torch.manual_seed(E)
    ext = load()
    N = 300
    logits = torch.randn(N, E, device="cuda") * 2
    bias = torch.randn(E, device="cuda")
    idx = torch.empty(N, K, dtype=torch.int64, device="cuda")
    w = torch.empty(N, K, dtype=torch.float32, device="cuda")
    # group-limited (DeepSeek-V3)
    ext.router_topk(logits, bias, 2, G, KG, 1.0, idx, w)
    want_idx, want_w = group_limited_topk(logits + bias, G, KG, K)
    assert torch.equal(idx.sort(-1).values, want_idx.sort(-1).values)
    got = torch.zeros(N, E, device="cuda").scatter_(1, idx, w)
    ref = torch.zeros(N, E, device="cuda").scatter_(1, want_idx, want_w)
    torch.testing.assert_close(got, ref, atol=1e-5, rtol=1e-4)
    # plain top-k + softmax over the selected logits
    ext.router_topk(logits, None, 0, 1, 1, 1.0, idx, w)
    tv, ti = logits.topk(K, dim=-1)
    assert torch.equal(idx, ti)
    torch.testing.assert_close(w, torch.softmax(tv, -1), atol=1e-6, rtol=1e-5)
    # sigmoid gates
    ext.router_topk(logits, None, 1, 1, 1, 1.0, idx, w)
    torch.testing.assert_close(w, torch.sigmoid(tv), atol=1e-6, rtol=1e-5)
