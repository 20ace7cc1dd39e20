"""Megatron bindings driven by stand-in objects (reference strategy: tests/test_sync_free.py:279-372)."""

from collections import OrderedDict
from types import SimpleNamespace

import pytest
import torch
import torch.nn as nn

from ep_balance_b200 import EPLBRebalancer, ProblemSpec, Topology
from ep_balance_b200.core.trace import load_routing_trace
from ep_balance_b200.integration import (MegatronEPLBHook, assert_plan_replicated, attach_router_observers,
                                         bind_eplb_to_moe_layer, bind_native_moe_timing, build_spec_for_megatron,
                                         find_moe_layers, setup_eplb_observer)
from ep_balance_b200.integration.megatron_moe import _routing_to_units
from ep_balance_b200.models.reference_moe import expert_mlp
from ep_balance_b200.utils import profiling

E, H, F, K = 4, 8, 16, 2


class TopKRouter(nn.Module):
    def __init__(self):
        super().__init__()
        self.w = nn.Parameter(torch.randn(E, H) * 0.5)

    def forward(self, x):
        logits = x.reshape(-1, H) @ self.w.t()
        top = logits.topk(K, dim=-1)
        rmap = torch.zeros_like(logits, dtype=torch.bool).scatter_(1, top.indices, True)
        probs = torch.zeros_like(logits).scatter_(1, top.indices, torch.softmax(top.values, -1))
        return probs, rmap


class _FC(nn.Module):
    def __init__(self, o, i):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(o, i) * 0.2)


class _Expert(nn.Module):
    def __init__(self):
        super().__init__()
        self.linear_fc1, self.linear_fc2 = _FC(2 * F, H), _FC(H, F)


class _Experts(nn.Module):
    def __init__(self):
        super().__init__()
        self.local_experts = nn.ModuleList([_Expert() for _ in range(E)])

    def forward(self, x):
        return x


class MoELayer(nn.Module):
    def __init__(self, shared=False):
        super().__init__()
        self.router, self.experts = TopKRouter(), _Experts()
        self.config = SimpleNamespace(moe_router_topk=K, gated_linear_unit=True, activation_func=torch.nn.functional.silu)
        self.use_shared_expert = shared

    def shared_experts_compute(self, x):
        return 0.5 * x

    def dispatch(self, x):
        return x

    def combine(self, x):
        return x

    def forward(self, x):
        probs, rmap = self.router(x)
        return self.combine(self.experts(self.dispatch(x))), None


def _truth(layer, x):
    probs, rmap = layer.router(x)
    out = torch.zeros_like(x.reshape(-1, H))
    for t in range(out.shape[0]):
        for e in rmap[t].nonzero().flatten().tolist():
            ex = layer.experts.local_experts[e]
            out[t] += probs[t, e] * expert_mlp(x.reshape(-1, H)[t:t + 1], ex.linear_fc1.weight, ex.linear_fc2.weight)[0]
    return out.reshape(x.shape)


def test_observer_logs_and_writes_trace(tmp_path):
    model = nn.Sequential(MoELayer(), MoELayer())
    lines = []
    hook, handles = setup_eplb_observer(model, num_experts=E, weight_bytes_each=100, s_tok=16, n_slot=E + 1,
                                        logger=lines.append, trace_out=str(tmp_path / "trace.pt"), trace_every=1,
                                        ep_group=None, ep_size=1)
    assert len(handles) == 2
    model.eval()
    x = torch.randn(5, H)
    for layer in model:
        layer(x)
    model[0](x)
    assert len(lines) == 3 and lines[0].startswith("[EPLB] layer=0 mb=0 theta=") and "layer=0 mb=1" in lines[2]
    assert "imbalance=" in lines[0] and "replicas=" in lines[0] and "phi_token=" in lines[0]
    hook.flush_trace()
    tr = load_routing_trace(tmp_path / "trace.pt")
    assert len(tr["samples"]) == 3 and tr["meta"]["num_ranks"] == 1
    assert int(tr["samples"][0]["omega"].sum()) == 5 * K
    assert assert_plan_replicated(hook.last_plan)
    for h in handles:
        h.remove()


def test_observer_skips_no_grad_pass_of_reentrant_checkpoint():
    model = nn.Sequential(MoELayer())
    seen = []
    hook = SimpleNamespace(step=lambda counts, layer_id, micro_batch_id: seen.append((layer_id, micro_batch_id)))
    attach_router_observers(model, hook, E)
    model.train()
    x = torch.randn(3, H)
    with torch.no_grad():
        model[0](x)
    assert seen == []
    model[0](x)
    assert seen == [(0, 0)]
    seen.clear()
    model2 = nn.Sequential(MoELayer())
    attach_router_observers(model2, hook, E, prefer_initial_forward=True)
    model2.train()
    with torch.no_grad():
        model2[0](x)
    model2[0](x)  # the recompute is skipped
    assert seen == [(0, 0)]


@pytest.mark.parametrize("shared", [False, True])
def test_bound_layer_matches_per_token_truth(shared):
    torch.manual_seed(0)
    layer = MoELayer(shared=shared)
    spec = build_spec_for_megatron(E, 1, 100, 16, E)
    reb = EPLBRebalancer(Topology.from_nvlink_rdma(1, 1), spec, ring_size=0)
    x = torch.randn(2, 3, H)
    want = _truth(layer, x) + (0.5 * x if shared else 0)
    bind_eplb_to_moe_layer(layer, reb, None, layer_id=3)
    assert find_moe_layers(nn.Sequential(layer)) == [layer]
    got, bias = layer(x)
    assert bias is None and torch.allclose(got, want, atol=1e-5, rtol=1e-4)
    got.sum().backward()
    assert layer.experts.local_experts[0].linear_fc1.weight.grad is not None
    assert layer._eplb["mb"] == 1


class _FakeFusedLayer:
    """Stands in for FusedMoE on CPU: same attributes the binding touches, expert math by the plain oracle."""

    def __init__(self):
        self.cfg = SimpleNamespace(num_experts=E)
        self.w1 = torch.zeros(E, 2 * F, H)
        self.w2 = torch.zeros(E, H, F)
        self.calls = []

    def apply_routed(self, tokens, top_idx, prob):
        from ep_balance_b200.models.reference_moe import moe_reference

        self.calls.append((tuple(top_idx.shape), tuple(prob.shape), top_idx.dtype))
        return moe_reference(tokens, top_idx, prob, self.w1, self.w2)


@pytest.mark.parametrize("shared", [False, True])
def test_fused_binding_rehomes_weights_and_matches_truth(shared):
    from ep_balance_b200.integration.megatron_moe import bind_fused_moe_layer

    torch.manual_seed(2)
    layer = MoELayer(shared=shared)
    x = torch.randn(2, 3, H)
    want = _truth(layer, x) + (layer.shared_experts_compute(x) if shared else 0)
    fused = _FakeFusedLayer()
    bind_fused_moe_layer(layer, fused)
    # the local experts were copied into the fused layer's owned slots, in order
    for i, ex in enumerate(layer.experts.local_experts):
        assert torch.equal(fused.w1[i], ex.linear_fc1.weight) and torch.equal(fused.w2[i], ex.linear_fc2.weight)
    got, bias = layer(x)
    assert bias is None and got.shape == x.shape and torch.allclose(got, want, atol=1e-5, rtol=1e-4)
    # one call with the router's decision as fixed-width [tokens, top-k] tensors (no data-dependent shapes)
    assert fused.calls == [((6, K), (6, K), torch.int64)]


def test_bind_rejects_unsupported_configurations(monkeypatch):
    layer = MoELayer(shared=True)
    layer.shared_expert_overlap = True
    reb = EPLBRebalancer(Topology.from_nvlink_rdma(1, 1), build_spec_for_megatron(E, 1, 100, 16, E))
    with pytest.raises(NotImplementedError):
        bind_eplb_to_moe_layer(layer, reb, None)
    monkeypatch.setenv("EPLB_ADAPTER", "deepep")
    with pytest.raises(ValueError):
        bind_eplb_to_moe_layer(MoELayer(), reb, None)
    monkeypatch.setenv("EPLB_ADAPTER", "bogus")
    with pytest.raises(ValueError):
        bind_eplb_to_moe_layer(MoELayer(), reb, None)


def test_routing_to_units_fixed_topk_equals_nonzero_path():
    probs, rmap = TopKRouter()(torch.randn(7, H))
    a = _routing_to_units(probs, rmap, 7, E, topk=K)
    b = _routing_to_units(probs, rmap, 7, E, topk=None)
    for u, v in zip(a, b):
        assert torch.equal(u, v)


def test_native_timing_wraps_and_restores(monkeypatch):
    monkeypatch.setattr(profiling, "_P", profiling.Profiler(debug=True))
    layer = MoELayer()
    model = nn.Sequential(layer)
    original = layer.forward
    lines = []
    (binding,) = bind_native_moe_timing(model, mode="off", logger=lines.append)
    layer(torch.randn(3, H))
    assert len(lines) == 1 and "mode=off layer=0 mb=0" in lines[0]
    for field in ("router=", "dispatch=", "expert_gemm=", "combine=", "solver=n/a", "expert_transfer=n/a"):
        assert field in lines[0], lines[0]
    with pytest.raises(RuntimeError):
        bind_native_moe_timing(model, mode="off")
    binding.remove()
    assert layer.forward.__func__ is original.__func__ and not hasattr(layer, "_eplb_native_timing")
    assert "forward" not in vars(layer.router) and "dispatch" not in vars(layer)
    # a layer without a required call: nothing stays installed
    broken = MoELayer()
    broken.combine = None
    with pytest.raises(RuntimeError):
        bind_native_moe_timing(nn.Sequential(broken), mode="off")
    assert "forward" not in vars(broken.router) and not hasattr(broken, "_eplb_native_timing")
