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
