"""Fused MoE layer (native kernels) vs the plain PyTorch oracle.

Single rank, and R logical ranks emulated on one GPU (reference strategy: logical ranks on one
device for the solver, gloo ranks for the apply path -- tests/test_sync_free.py:177-232).
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def _oracle(tokens, idx, prob, w1, w2, dout):
    from ep_balance_b200.models.reference_moe import moe_reference

    x = tokens.float().requires_grad_(True)
    p = prob.clone().requires_grad_(True)
    a = w1.float().requires_grad_(True)
    b = w2.float().requires_grad_(True)
    out = moe_reference(x, idx, p, a, b)
    out.backward(dout.float())
    return out.detach(), x.grad, p.grad, a.grad, b.grad


@pytest.mark.parametrize("ctas,fused_comm", [(1, True), (2, True), (2, False)])
def test_single_rank_forward_backward(ctas, fused_comm):
    from ep_balance_b200.models.emulated import EmulatedCluster
    from ep_balance_b200.models.moe_layer import MoEConfig

    torch.manual_seed(0)
    cfg = MoEConfig(hidden=256, ffn=384, num_experts=8, top_k=2, max_tokens=512, gemm_ctas=ctas,
                    fused_comm=fused_comm)
    cl = EmulatedCluster(cfg, world=1)
    layer = cl.layers[0]
    tokens = torch.randn(512, 256, device="cuda").bfloat16()
    layer.router_bias = torch.linspace(0, 2.0, 8, device="cuda")  # skewed routing, some experts rare
    tok = tokens.clone().requires_grad_(True)
    out = layer(tok)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    layer.check_status()
    idx, prob = layer.route_tokens(tokens)
    w1, w2 = cl.full_weights()
    o, dx, dp, dw1, dw2 = _oracle(tokens, idx, prob.detach(), w1, w2, dout)
    assert _rel(out, o) < 2e-2
    assert _rel(layer.w1.grad, dw1) < 3e-2
    assert _rel(layer.w2.grad, dw2) < 3e-2
    # token gradient = expert path + router path; compare the expert path via the emulated step
    res = cl.step([tokens], [dout])[0]
    assert _rel(res[0], o) < 2e-2
    assert _rel(res[1], dx) < 3e-2
    assert _rel(res[2], dp) < 3e-2


@pytest.mark.parametrize("world,domains", [(4, 2), (8, 2), (2, 1)])
def test_emulated_ranks_match_oracle(world, domains):
    from ep_balance_b200 import Loads, check_constraints
    from ep_balance_b200.models.emulated import EmulatedCluster
    from ep_balance_b200.models.moe_layer import MoEConfig
    from ep_balance_b200.solver import solve_device_semantics

    torch.manual_seed(1)
    E, K, N, H, Fd = 16, 2, 256, 256, 256
    cfg = MoEConfig(hidden=H, ffn=Fd, num_experts=E, top_k=K, max_tokens=N, extra_slots=2, num_domains=domains,
                    capacity_factor=float(world))
    cl = EmulatedCluster(cfg, world=world)
    bias = torch.zeros(E, device="cuda")
    bias[:3] = 3.0  # three hot experts -> replicas are worth it
    for l in cl.layers:
        l.router_bias = bias
    tokens = [torch.randn(N, H, device="cuda").bfloat16() for _ in range(world)]
    douts = [torch.randn(N, H, device="cuda").bfloat16() for _ in range(world)]
    res = cl.step(tokens, douts)
    torch.cuda.synchronize()
    for l in cl.layers:
        l.check_status()

    # every rank solved the same plan, and it is the plan of the host restatement
    omega = cl.heap.tensor("omega", 0).to(torch.int64).cpu()
    plan0 = cl.layers[0].last_plan().to("cpu")
    for l in cl.layers[1:]:
        assert plan0.equals(l.last_plan().to("cpu"))
    want = solve_device_semantics(Loads(omega), cl.layers[0].topo, cl.layers[0].spec, cl.layers[0].solver_cfg)
    assert plan0.equals(want)
    assert check_constraints(plan0, Loads(omega), cl.layers[0].topo, cl.layers[0].spec).ok
    assert int(plan0.x.sum()) > E  # replicas were placed

    w1, w2 = cl.full_weights()
    gw1, gw2 = cl.full_grads()
    dw1_sum = torch.zeros_like(w1, dtype=torch.float32)
    dw2_sum = torch.zeros_like(w2, dtype=torch.float32)
    for r in range(world):
        out, dtok, dprob, idx, prob = res[r]
        o, dx, dp, dw1, dw2 = _oracle(tokens[r], idx, prob, w1, w2, douts[r])
        assert _rel(out, o) < 2e-2, r
        assert _rel(dtok, dx) < 3e-2, r
        assert _rel(dprob, dp) < 3e-2, r
        dw1_sum += dw1
        dw2_sum += dw2
    # owners hold the sum of all replicas' weight gradients
    assert _rel(gw1, dw1_sum) < 3e-2
    assert _rel(gw2, dw2_sum) < 3e-2


def test_bounded_wait_reports_status_and_context_survives():
    from ep_balance_b200.ops.extension import load

    ext = load()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ext.wait_probe(flag, 1, 50_000_000, status)  # nobody sets the flag; budget 50 ms
    torch.cuda.synchronize()
    assert status.tolist()[0] == 2
    assert float(torch.ones(4, device="cuda").sum()) == 4.0  # the context is still usable


@pytest.mark.parametrize("acc_dtype", [torch.bfloat16, torch.float32])
def test_weight_gradients_accumulate_over_micro_batches(acc_dtype):
    """Two micro-batches through one layer: the accumulation buffer holds the sum of both weight
    gradients (fp32 oracle), for a single rank and for four emulated ranks with replicas."""
    from ep_balance_b200.models.emulated import EmulatedCluster
    from ep_balance_b200.models.moe_layer import MoEConfig

    torch.manual_seed(3)
    for world in (1, 4):
        E, N, H, Fd = 8, 256, 256, 256
        cfg = MoEConfig(hidden=H, ffn=Fd, num_experts=E, top_k=2, max_tokens=N, extra_slots=2,
                        capacity_factor=float(world), grad_accum_dtype=acc_dtype)
        cl = EmulatedCluster(cfg, world=world)
        bias = torch.zeros(E, device="cuda")
        bias[:2] = 3.0
        for l in cl.layers:
            l.router_bias = bias
            l.zero_grad_accum()
        w1, w2 = cl.full_weights()
        want1 = torch.zeros_like(w1, dtype=torch.float32)
        want2 = torch.zeros_like(w2, dtype=torch.float32)
        for mb in range(2):
            tokens = [torch.randn(N, H, device="cuda").bfloat16() for _ in range(world)]
            douts = [torch.randn(N, H, device="cuda").bfloat16() for _ in range(world)]
            res = cl.step(tokens, douts)
            for r in range(world):
                _, _, _, idx, prob = res[r]
                _, _, _, dw1, dw2 = _oracle(tokens[r], idx, prob, w1, w2, douts[r])
                want1 += dw1
                want2 += dw2
        torch.cuda.synchronize()
        for l in cl.layers:
            l.check_status()
        if acc_dtype == torch.float32:
            got1 = torch.cat([l.w1.main_grad for l in cl.layers])
            got2 = torch.cat([l.w2.main_grad for l in cl.layers])
        else:
            got1, got2 = cl.full_grads()
        assert got1.dtype == acc_dtype
        assert _rel(got1, want1) < 3e-2, world
        assert _rel(got2, want2) < 3e-2, world
        for l in cl.layers:
            l.zero_grad_accum()
        assert float(torch.cat([l._acc_gw1.flatten() for l in cl.layers]).abs().sum()) == 0.0


def test_router_logits_from_bf16_tokens_match_fp32_matmul():
    from ep_balance_b200.models.moe_layer import _RouterLinear

    torch.manual_seed(5)
    x = torch.randn(1024, 512, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(64, 512, device="cuda") * 0.02).requires_grad_(True)
    out = _RouterLinear.apply(x, w)
    g = torch.randn_like(out)
    out.backward(g)
    xr = x.detach().double().requires_grad_(True)
    wr = w.detach().double().requires_grad_(True)
    ref = xr @ wr.t()
    ref.backward(g.double())
    assert out.dtype == torch.float32
    assert _rel(out, ref) < 2e-6            # fp32-grade, far below bf16's 4e-3
    assert _rel(w.grad, wr.grad) < 2e-6
    assert _rel(x.grad, xr.grad) < 1e-2     # token gradient is bf16


def test_no_kernel_writes_past_a_symmetric_region():
    """Canary bytes behind every symmetric region survive a full step of four emulated ranks (and the check
    itself notices a deliberate host-side overwrite)."""
    from ep_balance_b200.models.emulated import EmulatedCluster
    from ep_balance_b200.models.moe_layer import MoEConfig

    torch.manual_seed(4)
    cfg = MoEConfig(hidden=256, ffn=256, num_experts=8, top_k=2, max_tokens=256, extra_slots=2, capacity_factor=4.0,
                    fp8_inference=True)
    cl = EmulatedCluster(cfg, world=4)
    for l in cl.layers:
        l.quantize_weights()
    tokens = [torch.randn(256, 256, device="cuda").bfloat16() for _ in range(4)]
    cl.step(tokens, [torch.randn_like(t) for t in tokens])
    cl.forward_fp8(tokens)
    torch.cuda.synchronize()
    for r in range(4):
        assert cl.heap.damaged_guards(r) == []
    flat = cl.heap._flat[2]
    off = cl.heap.layout.guards["ybuf"]
    flat[off + 3] = 0                                        # host-side: simulate an overrun of `ybuf`
    assert cl.heap.damaged_guards(2) == ["ybuf"]


def _one_layer(**kw):
    from ep_balance_b200.models.emulated import EmulatedCluster
    from ep_balance_b200.models.moe_layer import MoEConfig

    cfg = MoEConfig(hidden=256, ffn=256, num_experts=8, top_k=2, max_tokens=256, **kw)
    return EmulatedCluster(cfg, world=1).layers[0]


def test_warm_forward_backward_has_no_host_sync():
    """The hot path never reads device data on the host (reference: tests/test_gin_weights.py:423-436,
    tests/test_gpu_solver.py:149-171): a warmed step passes under the synchronisation detector."""
    layer = _one_layer()
    x = torch.randn(256, 256, device="cuda").bfloat16()
    dout = torch.randn_like(x)
    for _ in range(2):  # warm-up: lazy initialisation may synchronise
        y = layer(x.clone().requires_grad_(True))
        y.backward(dout)
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        tok = x.clone().requires_grad_(True)
        y = layer(tok)
        y.backward(dout)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()
    layer.check_status()
    assert torch.isfinite(tok.grad.float()).all()


@pytest.mark.parametrize("fused_comm", [True, False])
def test_launch_order_of_a_step(fused_comm):
    """The step is a fixed launch sequence (reference: the backward collective issue order pinned in
    tests/test_sync_free.py:61-82, 152-157): transport inside (or right before) the GEMM that consumes it,
    Dgrad2 before the weight-gradient GEMMs, Dgrad1 last so that the gradient return can run beside it."""
    layer = _one_layer(fused_comm=fused_comm)
    x = torch.randn(256, 256, device="cuda").bfloat16().requires_grad_(True)
    layer.rt.trace_launches(True)
    layer(x).backward(torch.randn(256, 256, device="cuda").bfloat16())
    torch.cuda.synchronize()
    log = layer.rt.launch_log()
    layer.rt.trace_launches(False)
    gemm1 = ["grouped_gemm+transport"] if fused_comm else ["dispatch", "grouped_gemm"]
    dgrad2 = ["grouped_gemm+transport"] if fused_comm else ["dispatch_grads", "grouped_gemm"]
    want = (["count_publish", "solver", "route_assign"] + gemm1 + ["grouped_gemm", "unit_reduce"]            # forward
            + dgrad2 + ["swiglu_backward", "grouped_gemm", "grouped_gemm", "grouped_gemm", "unit_reduce(bwd)"])  # backward
    assert log == want, log


def test_capacity_overflow_is_detected_and_contained():
    """Rows beyond the receive buffers are dropped by the kernels (never written out of bounds).  Such a step must
    not reach the weights and must surface on the host: the optimizer kernel skips its update while a status
    word is set, and the late monitor raises within two steps; afterwards the context is still usable."""
    from ep_balance_b200.models.emulated import EmulatedCluster
    from ep_balance_b200.models.moe_layer import MoEConfig
    from ep_balance_b200.utils.optim import FusedAdamW
    from ep_balance_b200.utils.status import MoEStatusError, StatusMonitor

    torch.manual_seed(3)
    world, E, K, N, H = 4, 8, 2, 512, 256
    # no replica slots and buffers for exactly the mean load: one hot expert overflows its owner
    cfg = MoEConfig(hidden=H, ffn=256, num_experts=E, top_k=K, max_tokens=N, extra_slots=0, capacity_factor=1.0)
    cl = EmulatedCluster(cfg, world=world)
    bias = torch.zeros(E, device="cuda")
    bias[0] = 8.0
    for l in cl.layers:
        l.router_bias = bias
    params = [p for l in cl.layers for p in (l.w1, l.w2)]
    opt = FusedAdamW(params, lr=1e-2, guard=cl.status.words)
    before = [p.detach().clone() for p in params]
    tokens = [torch.randn(N, H, device="cuda").bfloat16() for _ in range(world)]
    douts = [torch.randn(N, H, device="cuda").bfloat16() for _ in range(world)]
    monitor = StatusMonitor(cl.status.words)
    raised_at = None
    for step in range(3):
        cl.step(tokens, douts)
        opt.step()
        try:
            monitor.poll()
        except MoEStatusError as err:
            raised_at, seen = step, err
            break
    assert raised_at is not None and raised_at <= 2, "the overflow never reached the host"
    assert seen.code == 4 and "row overflow" in str(seen)
    torch.cuda.synchronize()
    for p, b in zip(params, before):
        assert torch.equal(p.detach(), b), "a damaged step changed the weights"
    assert cl.heap.damaged_guards() == []            # nothing was written past a buffer
    # the context survives: with the status cleared and a balanced router the same cluster trains again
    cl.status.clear()
    for l in cl.layers:
        l.router_bias = None
    cl.step(tokens, douts)
    opt.step()
    torch.cuda.synchronize()
    cl.status.check_now()
    assert any(not torch.equal(p.detach(), b) for p, b in zip(params, before))


def test_backward_after_another_forward_is_refused():
    """Backward reads the layer's buffers: a second autograd forward in between must raise, not corrupt gradients."""
    from ep_balance_b200.models.emulated import EmulatedCluster
    from ep_balance_b200.models.moe_layer import MoEConfig

    torch.manual_seed(0)
    cfg = MoEConfig(hidden=256, ffn=384, num_experts=8, top_k=2, max_tokens=256)
    layer = EmulatedCluster(cfg, world=1).layers[0]
    a = torch.randn(256, 256, device="cuda").bfloat16().requires_grad_(True)
    b = torch.randn(256, 256, device="cuda").bfloat16().requires_grad_(True)
    out_a = layer(a)
    out_b = layer(b)                      # replaces what out_a's backward would read
    with pytest.raises(RuntimeError, match="another forward"):
        out_a.sum().backward()
    out_b.sum().backward()                # the latest forward's backward is fine
    torch.cuda.synchronize()
    layer.check_status()
    assert b.grad is not None and torch.isfinite(b.grad.float()).all()


def test_device_routing_tables_equal_the_host_model():
    """row_base / send_off / tiles_of built by the solver kernel on 8 emulated ranks vs parallel/transport_model.py."""
    from ep_balance_b200.models.emulated import EmulatedCluster
    from ep_balance_b200.models.moe_layer import MoEConfig
    from ep_balance_b200.parallel.transport_model import sender_tables

    torch.manual_seed(1)
    world, E, N, H = 8, 16, 256, 256
    cfg = MoEConfig(hidden=H, ffn=256, num_experts=E, top_k=2, max_tokens=N, extra_slots=2, num_domains=2,
                    capacity_factor=float(world))
    cl = EmulatedCluster(cfg, world=world)
    bias = torch.zeros(E, device="cuda")
    bias[:3] = 3.0
    for l in cl.layers:
        l.router_bias = bias
    cl.step([torch.randn(N, H, device="cuda").bfloat16() for _ in range(world)],
            [torch.randn(N, H, device="cuda").bfloat16() for _ in range(world)])
    torch.cuda.synchronize()
    plan = cl.layers[0].last_plan().to("cpu")
    x, q = plan.x.to(torch.int64), plan.q.to(torch.int64)
    assert int(x.sum()) > E
    for r, layer in enumerate(cl.layers):
        want = sender_tables(x, q, layer.spec.main_rank.cpu(), r, 128 * cfg.gemm_ctas)
        for name in ("row_base", "send_off", "tiles_of"):
            assert torch.equal(layer.loc[name].cpu().to(torch.int64), want[name]), (r, name)
