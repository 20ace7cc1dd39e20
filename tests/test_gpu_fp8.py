"""Block-scaled fp8 grouped GEMM and its quantisers vs plain PyTorch in fp32."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def test_quantisers_round_trip_within_fp8_precision():
    from ep_balance_b200.ops import fp8

    torch.manual_seed(0)
    x = (torch.randn(256, 1408, device="cuda") * torch.logspace(-3, 2, 1408, device="cuda")).bfloat16()
    x[5] = 0
    q, sfa = fp8.quantize_rows(x)
    back = fp8.dequantize_rows(q, sfa)
    assert _rel(back, x) < 0.04
    assert float(back[5].abs().sum()) == 0.0
    # every block uses the full range: its largest magnitude lands in (224, 448] after scaling
    e = fp8.row_scale_exponents(sfa, 256, 1408).float() - 127
    amax = x.float().view(256, 11, 128).abs().amax(-1)
    scaled = amax / torch.exp2(e)
    ok = (amax == 0) | ((scaled > 224) & (scaled <= 448))
    assert bool(ok.all())

    w = (torch.randn(3, 256, 640, device="cuda") * 0.02).bfloat16()
    qw, sfb = fp8.quantize_weights(w)
    assert _rel(fp8.dequantize_weights(qw, sfb), w) < 0.04


@pytest.mark.parametrize("ctas", [1, 2])
@pytest.mark.parametrize("K,N", [(512, 256), (640, 384), (1408, 2048), (2048, 2816)])
def test_fp8_grouped_gemm_matches_dequantised_fp32(K, N, ctas):
    from ep_balance_b200.ops import fp8

    torch.manual_seed(1)
    rows = [300, 0, 128, 77]
    slots = [2, 0, 1, 3]
    offs, total = [], 0
    tile = 128 * ctas
    for r in rows:
        offs.append(total)
        total += (r + tile - 1) // tile * tile
    T = total + tile
    x = torch.zeros(T, K, device="cuda", dtype=torch.bfloat16)
    for o, r in zip(offs, rows):
        x[o:o + r] = (torch.randn(r, K, device="cuda") * (1 + 3 * torch.rand(r, 1, device="cuda"))).bfloat16()
    w = (torch.randn(4, N, K, device="cuda") * 0.05).bfloat16()
    aq, sfa = fp8.quantize_rows(x)
    bq, sfb = fp8.quantize_weights(w)
    out = torch.full((T, N), 7.0, device="cuda", dtype=torch.bfloat16)
    i32 = dict(dtype=torch.int32, device="cuda")
    goff = torch.tensor(offs + [total], **i32)
    grows = torch.tensor(rows, **i32)
    gws = torch.tensor(slots, **i32)
    totals = torch.tensor([total, len(rows)], **i32)
    status = torch.zeros(4, **i32)
    fp8.grouped_gemm_fp8(aq, sfa, bq, sfb, out, goff, grows, gws, totals, status, ctas=ctas)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    xd, wd = fp8.dequantize_rows(aq, sfa), fp8.dequantize_weights(bq, sfb)
    for o, r, s in zip(offs, rows, slots):
        if r == 0:
            continue
        want = xd[o:o + r] @ wd[s].t()
        assert _rel(out[o:o + r], want) < 6e-3, (o, r, s)
        # and against the unquantised product: fp8 rounding of both operands
        assert _rel(out[o:o + r], x[o:o + r].float() @ w[s].float().t()) < 0.06
        # rows past the group's end were not touched
        pad_end = o + (r + tile - 1) // tile * tile
        assert bool((out[o + r:pad_end] == 7.0).all())


@pytest.mark.parametrize("world", [1, 4])
def test_fp8_inference_forward_matches_bf16_oracle(world):
    """Whole layer forward with fp8 expert GEMMs (single rank; four emulated ranks with fp8 replica pulls)."""
    from ep_balance_b200.models.emulated import EmulatedCluster
    from ep_balance_b200.models.moe_layer import MoEConfig
    from ep_balance_b200.models.reference_moe import moe_reference

    torch.manual_seed(2)
    E, K, N, H, Fd = 16, 2, 256, 256, 384
    cfg = MoEConfig(hidden=H, ffn=Fd, num_experts=E, top_k=K, max_tokens=N, extra_slots=2, num_domains=1,
                    capacity_factor=float(world), fp8_inference=True)
    cl = EmulatedCluster(cfg, world=world)
    bias = torch.zeros(E, device="cuda")
    bias[:3] = 3.0
    for l in cl.layers:
        l.router_bias = bias
        l.quantize_weights()
    tokens = [torch.randn(N, H, device="cuda").bfloat16() for _ in range(world)]
    outs, routing = cl.forward_fp8(tokens)
    torch.cuda.synchronize()
    for l in cl.layers:
        l.check_status()
    if world > 1:
        assert int(cl.layers[0].last_plan().x.sum()) > E   # replicas exist, so fp8 weights crossed ranks
    w1, w2 = cl.full_weights()
    for r in range(world):
        idx, prob = routing[r]
        want = moe_reference(tokens[r].float(), idx, prob, w1.float(), w2.float())
        assert _rel(outs[r], want) < 0.08, r
        assert _rel(outs[r], want) > 1e-4   # it really is the quantised path
