"""Native AdamW step vs torch.optim.AdamW evaluated in fp32."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,n", [(torch.bfloat16, 1 << 20), (torch.bfloat16, 1000003), (torch.float32, 4099)])
def test_adamw_matches_torch(dtype, n):
    from ep_balance_b200.utils.optim import FusedAdamW

    torch.manual_seed(0)
    p0 = torch.randn(n, device="cuda")
    mine = torch.nn.Parameter(p0.to(dtype).clone())
    ref = torch.nn.Parameter(p0.to(dtype).float().clone())
    opt_m = FusedAdamW([mine], lr=1e-2, weight_decay=0.1)
    opt_r = torch.optim.AdamW([ref], lr=1e-2, weight_decay=0.1)
    for step in range(4):
        g = torch.randn(n, device="cuda").to(dtype)
        mine.grad = g.clone()
        ref.grad = g.float()
        opt_m.step()
        opt_r.step()
    err = float((mine.float() - ref).norm() / ref.norm())
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5  # bf16 parameter and moment rounding
    assert err < tol, err
    # the step moved the parameters by far more than the tolerance
    assert float((ref - p0.to(dtype).float()).norm() / ref.norm()) > 2 * tol


def test_adamw_reads_an_fp32_main_grad_for_bf16_parameters():
    from ep_balance_b200.utils.optim import FusedAdamW

    torch.manual_seed(1)
    n = 262147  # not a multiple of 8: exercises the scalar tail too
    p0 = torch.randn(n, device="cuda")
    mine = torch.nn.Parameter(p0.bfloat16().clone())
    ref = torch.nn.Parameter(p0.bfloat16().float().clone())
    opt_m = FusedAdamW([mine], lr=1e-2, weight_decay=0.1)
    opt_r = torch.optim.AdamW([ref], lr=1e-2, weight_decay=0.1)
    for step in range(3):
        g = torch.randn(n, device="cuda")
        mine.main_grad = g.clone()
        ref.grad = g.clone()
        opt_m.step()
        opt_r.step()
    assert float((mine.float() - ref).norm() / ref.norm()) < 1e-2


def test_capturable_adamw_replays_from_a_graph_like_eager_steps():
    """Whole training step of the fused layer captured once and replayed: parameters after three replays equal
    three eager steps from the same start (same inputs), including the device-side step counter."""
    from ep_balance_b200.models.emulated import EmulatedCluster
    from ep_balance_b200.models.moe_layer import MoEConfig
    from ep_balance_b200.utils.graphs import GraphedStep
    from ep_balance_b200.utils.optim import FusedAdamW

    def build():
        torch.manual_seed(0)
        cfg = MoEConfig(hidden=256, ffn=256, num_experts=8, top_k=2, max_tokens=256)
        layer = EmulatedCluster(cfg, world=1).layers[0]
        opt = FusedAdamW(layer.parameters(), lr=1e-3, capturable=True)

        def step(x):
            loss = layer(x.detach().requires_grad_(True)).float().square().mean()
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            return loss

        return layer, step

    xs = [torch.randn(256, 256, device="cuda", generator=torch.Generator(device="cuda").manual_seed(i)).bfloat16()
          for i in range(6)]
    eager_layer, eager_step = build()
    eager_losses = [float(eager_step(x)) for x in xs]
    graph_layer, graph_step = build()
    g = GraphedStep(graph_step, xs[0], warmup=3)        # three warm-up steps on xs[0] inside
    # bring the eager twin to the same state: three steps on xs[0]
    twin_layer, twin_step = build()
    for _ in range(3):
        twin_step(xs[0])
    losses = []
    for x in xs[:3]:
        losses.append(float(g(x)))
        twin_step(x)
    torch.cuda.synchronize()
    graph_layer.check_status()
    err = float((graph_layer.w1.float() - twin_layer.w1.float()).norm() / twin_layer.w1.float().norm())
    assert err < 2e-3, err
    assert float((graph_layer.w1.float() - eager_layer.w1.float()).abs().max()) > 0      # it did train
    assert all(l == l and l > 0 for l in losses)


def test_guarded_adamw_skips_the_update_while_a_status_word_is_set():
    from ep_balance_b200.utils.optim import FusedAdamW

    guard = torch.zeros((3, 4), dtype=torch.int32, device="cuda")
    p = torch.nn.Parameter(torch.randn(4099, device="cuda").bfloat16())
    p.grad = torch.randn_like(p)
    opt = FusedAdamW([p], lr=1e-2, guard=guard)
    before = p.detach().clone()
    guard[2, 0] = 4                       # some layer reported a row overflow
    opt.step()
    torch.cuda.synchronize()
    assert torch.equal(p.detach(), before)
    assert float(opt.state[p]["exp_avg"].float().abs().sum()) == 0.0   # moments untouched too
    guard.zero_()
    opt.step()
    torch.cuda.synchronize()
    assert not torch.equal(p.detach(), before)
