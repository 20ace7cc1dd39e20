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
