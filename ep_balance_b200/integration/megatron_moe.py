"""Apply mode for Megatron-Core: replace ``MoELayer.forward`` with the balanced dispatcher.

Three transports are selectable with ``EPLB_ADAPTER``:
  ``alltoall`` (default)  the portable path over NCCL (:mod:`ep_balance_b200.parallel.library_path`); reads
                          the split sizes to the host once per chunk,
  ``padded``              the portable path with fixed-size blocks per rank pair (``EPLB_PAIR_ROWS``): no
                          host read at all, padding travels instead,
  ``fused``               the native B200 layer; the layer's experts are re-homed into symmetric
                          memory once, at bind time (:func:`bind_fused_moe_layer`).
``deepep`` is rejected: DeepEP's ElasticBuffer is not available in this build; its role (zero-sync
token transport) is what ``padded`` (library collectives) and ``fused`` (device-initiated) provide.  Reference: eplb/integration/megatron_moe.py:19-260.
"""

from __future__ import annotations

import os
import types
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..parallel.grouped_mlp import make_batched_gated_mlp, make_grouped_gated_mlp
from ..parallel.library_path import AllToAllAdapter, PaddedAllToAllAdapter, sync_free_moe_forward
from ..parallel.omega import local_counts_from_routing
from ..utils import profiling


def _env_flag(name: str) -> bool:
    return os.environ.get(name, "0").strip().lower() not in ("0", "", "false", "no")


def _env_positive(name: str) -> Optional[int]:
    v = int(os.environ.get(name, "0") or "0")
    return v if v > 0 else None


def _make_adapter():
    name = os.environ.get("EPLB_ADAPTER", "alltoall").strip().lower()
    if name in ("", "alltoall", "all_to_all", "a2a"):
        return AllToAllAdapter()
    if name == "fused":
        return "fused"
    if name == "padded":
        rows = _env_positive("EPLB_PAIR_ROWS")
        if rows is None:
            raise ValueError("EPLB_ADAPTER=padded needs EPLB_PAIR_ROWS (rows every pair of ranks exchanges per chunk)")
        return PaddedAllToAllAdapter(rows)
    if name in ("deepep", "deep_ep"):
        raise ValueError("EPLB_ADAPTER=deepep: DeepEP is not part of this build; use EPLB_ADAPTER=fused for the "
                         "zero-sync device-initiated transport, or EPLB_ADAPTER=padded for the zero-sync transport on "
                         "library collectives")
    raise ValueError(f"unknown EPLB_ADAPTER={name!r} (expected 'alltoall' | 'padded' | 'fused')")


def find_moe_layers(model, class_name: str = "MoELayer") -> List:
    return [m for _, m in model.named_modules() if type(m).__name__ == class_name]


def extract_local_expert_weights(experts_module) -> Tuple[List[Tuple[torch.Tensor, ...]], List[torch.Size]]:
    """``[(fc1.weight, fc2.weight), ...]`` per local expert of a ``SequentialMLP`` + their shapes."""
    local = getattr(experts_module, "local_experts", None)
    if local is None:
        raise NotImplementedError("apply mode supports SequentialMLP experts (``.local_experts``) only; run "
                                  "without --moe-grouped-gemm")
    tuples = [(m.linear_fc1.weight, m.linear_fc2.weight) for m in local]
    return tuples, [t.shape for t in tuples[0]]


def _routing_to_units(probs: torch.Tensor, routing_map: torch.Tensor, num_tokens: int, num_experts: int,
                      topk: Optional[int] = None):
    """Flatten a router's selection into units ``(token idx, expert, gate weight)``.

    With a fixed ``topk`` no data-dependent shape appears: a stable sort of the negated mask lists
    each token's selected experts first, in ascending id.  Without it ``nonzero`` is used (syncs).
    """
    rmap = routing_map.bool().reshape(num_tokens, num_experts)
    p = probs.reshape(num_tokens, num_experts)
    if topk is None:
        nz = rmap.nonzero(as_tuple=False)
        t, e = nz[:, 0].contiguous(), nz[:, 1].contiguous()
        return t, e, p[t, e].contiguous()
    k = int(topk)
    sel = torch.argsort((~rmap).to(torch.int8), dim=1, stable=True)[:, :k].contiguous()
    t = torch.arange(num_tokens, device=rmap.device).view(-1, 1).expand(-1, k).reshape(-1).contiguous()
    return t, sel.reshape(-1).contiguous(), p.gather(1, sel).reshape(-1).contiguous()


def eplb_moe_forward(self, hidden_states, *args, **kwargs):
    """Drop-in ``MoELayer.forward`` (bound by :func:`bind_eplb_to_moe_layer`)."""
    st = self._eplb
    reb, group = st["reb"], st["group"]
    spec = reb.spec
    profiling.begin_debug_window()
    shape = hidden_states.shape
    tokens = hidden_states.reshape(-1, shape[-1])

    shared_out = None
    if getattr(self, "use_shared_expert", False):
        with profiling.record("apply/shared_expert", time_it=True, device=tokens.device):
            shared_out = self.shared_experts_compute(hidden_states)

    with profiling.record("apply/route", time_it=True, device=tokens.device):
        probs, routing_map = self.router(hidden_states)
        ut, ue, up = _routing_to_units(probs, routing_map, tokens.shape[0], spec.num_experts,
                                       topk=getattr(self.config, "moe_router_topk", None))
        local_row = local_counts_from_routing(ue, spec.num_experts)

    mb = st["mb"]
    st["mb"] = mb + 1
    plan = reb.rebalance(local_row, st["layer_id"], mb, group=group).plan

    ep_rank = dist.get_rank(group) if dist.is_initialized() else 0
    tuples, shapes = extract_local_expert_weights(self.experts)
    weights_local: Dict[int, Tuple[torch.Tensor, ...]] = {ep_rank * len(tuples) + i: t for i, t in enumerate(tuples)}
    out = sync_free_moe_forward(
        tokens=tokens, unit_token_idx=ut, unit_expert=ue, unit_prob=up.to(tokens.dtype), plan=plan, spec=spec,
        weights_local=weights_local, weight_shapes=shapes, batched_mlp_fn=st["batched_mlp_fn"],
        grouped_mlp_fn=st["grouped_mlp_fn"], cap=_env_positive("EPLB_CAP"),
        max_recv_rows=_env_positive("EPLB_MAX_RECV_ROWS"), group=group, adapter=st["adapter"],
        rematerialize=st["rematerialize"], overlap=st["overlap"], gated=st["gated"], act=st["act"], transpose_w=True)
    if profiling.enabled():
        profiling.maybe_summary(print if (ep_rank == 0 or profiling.all_ranks()) else None,
                                context=f"mode=apply layer={st['layer_id']} mb={mb}")
    out = out.reshape(shape)
    if shared_out is not None:
        out = out + shared_out
    return out, None


def bind_eplb_to_moe_layer(moe_layer, rebalancer, ep_group, layer_id: int = 0) -> None:
    """Patch one ``MoELayer`` so that its forward dispatches through the balancer."""
    cfg = moe_layer.config
    if getattr(moe_layer, "use_shared_expert", False):
        if getattr(moe_layer, "shared_expert_overlap", False):
            raise NotImplementedError("apply mode supports shared experts only with moe_shared_expert_overlap=False")
        if not callable(getattr(moe_layer, "shared_experts_compute", None)):
            raise NotImplementedError("this MoELayer exposes shared experts but no shared_experts_compute method")
    adapter = _make_adapter()
    if adapter == "fused":
        raise ValueError("EPLB_ADAPTER=fused is bound with bind_fused_moe_layer (it re-homes the expert weights)")
    gated = bool(getattr(cfg, "gated_linear_unit", False))
    act = getattr(cfg, "activation_func", torch.nn.functional.gelu)
    moe_layer._eplb = {
        "reb": rebalancer, "group": ep_group, "layer_id": int(layer_id), "mb": 0, "gated": gated, "act": act,
        "batched_mlp_fn": make_batched_gated_mlp(gated, act), "grouped_mlp_fn": make_grouped_gated_mlp(gated, act),
        "adapter": adapter, "rematerialize": _env_flag("EPLB_REMATERIALIZE"), "overlap": _env_flag("EPLB_OVERLAP"),
    }
    moe_layer.forward = types.MethodType(eplb_moe_forward, moe_layer)


def bind_fused_moe_layer(moe_layer, fused_layer) -> None:
    """Route a Megatron ``MoELayer`` through a :class:`~ep_balance_b200.models.moe_layer.FusedMoE`.

    The local experts' ``linear_fc1/linear_fc2`` weights are copied into the fused layer's owned
    slots (symmetric memory) once; from then on the fused layer's parameters are the trainable ones.
    The Megatron router keeps producing ``(probs, routing_map)``.
    """
    tuples, _ = extract_local_expert_weights(moe_layer.experts)
    with torch.no_grad():
        for i, (w1, w2) in enumerate(tuples):
            fused_layer.w1[i].copy_(w1.to(fused_layer.w1.dtype))
            fused_layer.w2[i].copy_(w2.to(fused_layer.w2.dtype))

    def forward(self, hidden_states, *args, **kwargs):
        shape = hidden_states.shape
        tokens = hidden_states.reshape(-1, shape[-1]).contiguous()
        probs, routing_map = self.router(hidden_states)
        k = int(self.config.moe_router_topk)
        _, ue, up = _routing_to_units(probs, routing_map, tokens.shape[0], fused_layer.cfg.num_experts, topk=k)
        out = fused_layer.apply_routed(tokens, ue.view(-1, k), up.view(-1, k))
        out = out.reshape(shape)
        if getattr(self, "use_shared_expert", False):
            out = out + self.shared_experts_compute(hidden_states)
        return out, None

    moe_layer.forward = types.MethodType(forward, moe_layer)
