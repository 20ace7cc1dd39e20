"""tcgen05 grouped GEMM vs a plain fp32 PyTorch loop over groups, every mode."""

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

MODE = dict(fwd1=0, fwd2=1, dgrad2=2, dgrad1=3, wgrad=4, plain=5)


CTAS = [1, 2]


def _groups(rows, device, ctas=1):
    """Group table with starts aligned to the GEMM M tile: returns tensors + padded total."""
    off, acc = [], 0
    tile = 128 * ctas
    for r in rows:
        off.append(acc)
        acc += (r + tile - 1) // tile * tile
    off.append(acc)
    i32 = dict(dtype=torch.int32, device=device)
    return (torch.tensor(off, **i32), torch.tensor(rows, **i32), torch.tensor([acc, len(rows)], **i32), acc)


def _ext():
    from ep_balance_b200.ops.extension import load

    return load()


def _run(mode, a, b, out0, out1, rows, wslot, ctas=1):
    ext = _ext()
    dev = a.device
    goff, grows, totals, _ = _groups(rows, dev, ctas)
    gws = torch.tensor(wslot, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    ext.grouped_gemm(MODE[mode], a, b, out0, out1, goff, grows, gws, totals, status, sms, ctas)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    return goff.tolist()


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


ROWS = [300, 0, 128, 1, 517]
WSLOT = [2, 0, 4, 1, 3]


@pytest.mark.parametrize("ctas", CTAS)
@pytest.mark.parametrize("N,K", [(512, 256), (2048, 1408), (320, 192)])
def test_plain_k_major(N, K, ctas):
    dev = "cuda"
    torch.manual_seed(0)
    _, _, _, T = _groups(ROWS, dev, ctas)
    a = torch.randn(T, K, device=dev).bfloat16()
    w = (torch.randn(5, N, K, device=dev) * 0.05).bfloat16()
    out = torch.full((T, N), 7.0, device=dev).bfloat16()
    off = _run("plain", a, w, out, None, ROWS, WSLOT, ctas)
    for g, r in enumerate(ROWS):
        if r == 0:
            continue
        want = a[off[g]:off[g] + r].float() @ w[WSLOT[g]].float().t()
        assert _rel(out[off[g]:off[g] + r], want) < 1e-2
        # rows past the group's end are never written
        pad = out[off[g] + r: off[g + 1]]
        assert bool((pad == 7.0).all())


@pytest.mark.parametrize("ctas", CTAS)
def test_fwd1_swiglu_and_zeroed_padding(ctas):
    dev = "cuda"
    torch.manual_seed(1)
    K, Fd = 512, 384
    _, _, _, T = _groups(ROWS, dev, ctas)
    a = torch.randn(T, K, device=dev).bfloat16()
    w = (torch.randn(5, 2 * Fd, K, device=dev) * 0.05).bfloat16()
    h = torch.full((T, 2 * Fd), 3.0, device=dev).bfloat16()
    act = torch.full((T, Fd), 3.0, device=dev).bfloat16()
    off = _run("fwd1", a, w, h, act, ROWS, WSLOT, ctas)
    for g, r in enumerate(ROWS):
        sl = slice(off[g], off[g] + r)
        if r:
            hh = a[sl].float() @ w[WSLOT[g]].float().t()
            assert _rel(h[sl], hh) < 1e-2
            gate, up = h[sl].float().chunk(2, dim=-1)
            assert _rel(act[sl], F.silu(gate) * up) < 1e-2
        assert bool((h[off[g] + r: off[g + 1]] == 0).all())
        assert bool((act[off[g] + r: off[g + 1]] == 0).all())


@pytest.mark.parametrize("ctas", CTAS)
@pytest.mark.parametrize("N,K", [(512, 256), (2048, 2816), (1408, 2048)])
def test_dgrad1_mn_major_weights(N, K, ctas):
    dev = "cuda"
    torch.manual_seed(2)
    _, _, _, T = _groups(ROWS, dev, ctas)
    a = torch.randn(T, K, device=dev).bfloat16()
    w = (torch.randn(5, K, N, device=dev) * 0.05).bfloat16()
    out = torch.zeros(T, N, device=dev).bfloat16()
    off = _run("dgrad1", a, w, out, None, ROWS, WSLOT, ctas)
    for g, r in enumerate(ROWS):
        if r:
            want = a[off[g]:off[g] + r].float() @ w[WSLOT[g]].float()
            assert _rel(out[off[g]:off[g] + r], want) < 1e-2


@pytest.mark.parametrize("ctas", CTAS)
def test_dgrad2_activation_gradient_in_place(ctas):
    dev = "cuda"
    torch.manual_seed(3)
    Hd, Fd = 256, 384
    _, _, _, T = _groups(ROWS, dev, ctas)
    dy = torch.randn(T, Hd, device=dev).bfloat16()
    w2 = (torch.randn(5, Hd, Fd, device=dev) * 0.05).bfloat16()
    h = torch.randn(T, 2 * Fd, device=dev).bfloat16()
    h0 = h.clone()
    off = _run("dgrad2", dy, w2, h, None, ROWS, WSLOT, ctas)
    for g, r in enumerate(ROWS):
        sl = slice(off[g], off[g] + r)
        if r:
            hh = h0[sl].float().requires_grad_(True)
            gate, up = hh.chunk(2, dim=-1)
            a = F.silu(gate) * up
            da = dy[sl].float() @ w2[WSLOT[g]].float()
            (dh,) = torch.autograd.grad(a, hh, da)
            assert _rel(h[sl], dh) < 2e-2
        assert bool((h[off[g] + r: off[g + 1]] == 0).all())


@pytest.mark.parametrize("ctas", CTAS)
@pytest.mark.parametrize("M,N", [(256, 512), (2048, 1408), (2816, 2048)])
def test_wgrad_ragged_contraction(M, N, ctas):
    dev = "cuda"
    torch.manual_seed(4)
    goff, grows, totals, T = _groups(ROWS, dev, ctas)
    p = torch.randn(T, M, device=dev).bfloat16()
    q = torch.randn(T, N, device=dev).bfloat16()
    off = goff.tolist()
    for g, r in enumerate(ROWS):  # padding rows must be zero in at least one operand (here: both)
        p[off[g] + r: off[g + 1]] = 0
        q[off[g] + r: off[g + 1]] = 0
    out = torch.full((5, M, N), 5.0, device=dev).bfloat16()
    _run("wgrad", p, q, out, None, ROWS, WSLOT, ctas)
    for g, r in enumerate(ROWS):
        want = p[off[g]:off[g] + r].float().t() @ q[off[g]:off[g] + r].float()
        if r == 0:
            assert bool((out[WSLOT[g]] == 0).all())
        else:
            assert _rel(out[WSLOT[g]], want) < 1e-2
