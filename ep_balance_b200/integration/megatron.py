"""Observe mode for Megatron-Core models: capture routing into omega, solve, log, dump traces.

Nothing here imports Megatron at module import time; routers and layers are matched by class name
and driven by duck typing, so the whole module is testable with stand-in objects.
Reference: eplb/integration/megatron.py:16-404.
"""

from __future__ import annotations

import atexit
from typing import Callable, List, Optional

import torch

from ..core.config import EPLBConfig
from ..core.loads import Loads
from ..core.metrics import compute_metrics
from ..core.problem import ProblemSpec
from ..core.topology import Topology
from ..core.trace import TraceWriter, build_trace_meta
from ..parallel.rebalancer import EPLBRebalancer
from ..utils import profiling


def omega_row_from_routing_map(routing_map: torch.Tensor) -> torch.Tensor:
    """``routing_map`` [tokens, E] (bool/int) -> int64 [E] counts."""
    return routing_map.to(torch.int64).sum(0)


def omega_row_from_topk_indices(topk_indices: torch.Tensor, num_experts: int) -> torch.Tensor:
    flat = topk_indices.to(torch.int64).reshape(-1)
    return torch.zeros(int(num_experts), dtype=torch.int64, device=flat.device).scatter_add_(0, flat, torch.ones_like(flat))


def reduce_router_counts_tp_cp(local_counts: torch.Tensor, router) -> torch.Tensor:
    """Sum counts over the router's TP x CP group: those ranks hold shards of ONE source rank's
    tokens, whereas expert-parallel ranks must stay separate rows of omega."""
    group = getattr(router, "tp_cp_group", None)
    dist = torch.distributed
    if group is None or not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) <= 1:
        return local_counts
    out = local_counts.contiguous().clone()
    dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
    return out


def build_spec_for_megatron(num_experts: int, ep_size: int, weight_bytes_each: int, s_tok: int, n_slot: int,
                            device="cpu") -> ProblemSpec:
    """Megatron's contiguous split: expert ``e`` is owned by rank ``e // (E / ep)``."""
    return ProblemSpec.contiguous_main_placement(num_experts, ep_size, weight_bytes_each, s_tok, n_slot, device)


class MegatronEPLBHook:
    """Per-layer hook: gather omega, solve, log one ``[EPLB] ...`` line, optionally record a trace."""

    def __init__(self, rebalancer: EPLBRebalancer, mode: str = "observe", ep_group=None,
                 logger: Optional[Callable[[str], None]] = None, *, trace_out: Optional[str] = None,
                 trace_max: int = 0, trace_every: int = 25, counts_reduced_over_tp_cp: bool = False,
                 owns_timing_window: bool = True) -> None:
        if mode not in ("observe", "apply"):
            raise ValueError("mode must be 'observe' or 'apply'")
        self.reb, self.mode, self.ep_group, self.logger = rebalancer, mode, ep_group, logger
        self.last_plan = None
        self.owns_timing_window = bool(owns_timing_window)
        self.counts_reduced_over_tp_cp = bool(counts_reduced_over_tp_cp)
        self.trace: Optional[TraceWriter] = None
        if trace_out is not None:
            meta = build_trace_meta(rebalancer.topo, rebalancer.spec,
                                    counts_reduced_over_tp_cp=self.counts_reduced_over_tp_cp)
            self.trace = TraceWriter(trace_out, meta, max_samples=trace_max, every=trace_every)
            atexit.register(self.flush_trace)

    def step(self, local_counts: torch.Tensor, layer_id: int, micro_batch_id: int):
        if self.owns_timing_window:
            profiling.begin_debug_window()
        res = self.reb.rebalance(local_counts, layer_id, micro_batch_id, group=self.ep_group)
        self.last_plan = res.plan
        omega = self.reb.omega_of(layer_id, micro_batch_id)
        if self.logger is not None and omega is not None:
            self._log(res.plan, omega, layer_id, micro_batch_id)
        if self.trace is not None and omega is not None:
            self.trace.add(layer_id, micro_batch_id, omega)
        return res.plan

    def backward(self, layer_id: int, micro_batch_id: int):
        return self.reb.backward(layer_id, micro_batch_id)

    def _log(self, plan, omega, layer_id: int, micro_batch_id: int) -> None:
        m = compute_metrics(plan, Loads(omega), self.reb.topo, self.reb.spec, self.reb.cfg)
        extra = f" solve_ms={profiling.last_ms('solve'):.3f}" if profiling.enabled() else ""
        self.logger(f"[EPLB] layer={layer_id} mb={micro_batch_id} theta={m.theta} imbalance={m.imbalance:.3f} "
                    f"replicas={m.total_replicas} phi_token={m.phi_token}{extra}")
        if self.owns_timing_window:
            profiling.maybe_summary(self.logger, context=f"mode=observe layer={layer_id} mb={micro_batch_id}")

    def flush_trace(self) -> None:
        if self.trace is not None:
            self.trace.flush()


def _extract_routing_map(output, num_experts: int) -> torch.Tensor:
    """Find the [tokens, E] selection mask (or top-k index tensor) in a router's output."""
    cands = output if isinstance(output, (tuple, list)) else (output,)
    ints = [t for t in cands if isinstance(t, torch.Tensor) and (t.dtype == torch.bool or not t.is_floating_point())]
    for t in ints:
        if t.dim() >= 2 and t.shape[-1] == num_experts:
            return t.reshape(-1, num_experts)
    for t in ints:
        return torch.nn.functional.one_hot(t.to(torch.int64).reshape(-1), num_classes=num_experts)
    raise TypeError("could not locate a routing_map / index tensor in router output")


def attach_router_observers(model, hook: MegatronEPLBHook, num_experts: int, micro_batch_id_fn=None,
                            router_class_name: str = "TopKRouter", reduce_tp_cp: bool = True,
                            prefer_initial_forward: bool = False) -> List:
    """Forward hooks on every router.  Under re-entrant activation checkpointing a training forward
    runs twice (no-grad, then recompute); exactly one of the two is observed: the recompute by
    default, the initial pass with ``prefer_initial_forward``."""
    handles, calls, pending = [], {}, {}

    def make(layer_id: int):
        def cb(module, _inputs, output):
            if getattr(module, "training", False):
                if not torch.is_grad_enabled():
                    if not prefer_initial_forward:
                        return output
                    pending[layer_id] = pending.get(layer_id, 0) + 1
                elif prefer_initial_forward and pending.get(layer_id, 0):
                    pending[layer_id] -= 1
                    return output
            counts = omega_row_from_routing_map(_extract_routing_map(output, num_experts))
            if reduce_tp_cp:
                counts = reduce_router_counts_tp_cp(counts, module)
            if micro_batch_id_fn is not None:
                mb = micro_batch_id_fn()
            else:  # n-th forward of this layer (stable across layers without pipeline parallelism)
                mb = calls.get(layer_id, 0)
                calls[layer_id] = mb + 1
            hook.step(counts, layer_id=layer_id, micro_batch_id=mb)
            return output

        return cb

    layer = 0
    for _name, module in model.named_modules():
        if type(module).__name__ == router_class_name:
            handles.append(module.register_forward_hook(make(layer)))
            layer += 1
    return handles


def setup_eplb_observer(model, *, num_experts: int, weight_bytes_each: int, s_tok: int, n_slot: int,
                        gpus_per_node: Optional[int] = None, intra_cost: int = 1, inter_cost: int = 8,
                        cfg: Optional[EPLBConfig] = None, logger=print, micro_batch_id_fn=None,
                        router_class_name: str = "TopKRouter", trace_out: Optional[str] = None, trace_max: int = 0,
                        trace_every: int = 25, reduce_tp_cp: bool = True, native_timing: bool = False,
                        ep_group=None, ep_size: Optional[int] = None):
    """One-call observe-mode set-up.  The expert-parallel group and size come from Megatron's
    ``parallel_state`` unless passed in (``ep_group``/``ep_size``), which also makes this usable
    without Megatron installed.  Returns ``(hook, handles)``."""
    if ep_size is None:
        from megatron.core import parallel_state as mpu  # only needed on a Megatron cluster

        ep_group = mpu.get_expert_model_parallel_group()
        ep_size = mpu.get_expert_model_parallel_world_size()
    device = next(model.parameters()).device
    gpn = gpus_per_node or ep_size
    if gpn <= 0 or ep_size % gpn:
        gpn = ep_size
    topo = Topology.from_nvlink_rdma(ep_size // gpn, gpn, intra_cost, inter_cost, device)
    spec = build_spec_for_megatron(num_experts, ep_size, weight_bytes_each, s_tok, n_slot, device)
    hook = MegatronEPLBHook(EPLBRebalancer(topo, spec, cfg or EPLBConfig()), mode="observe", ep_group=ep_group,
                            logger=logger, trace_out=trace_out, trace_max=trace_max, trace_every=trace_every,
                            counts_reduced_over_tp_cp=reduce_tp_cp, owns_timing_window=not native_timing)
    handles = attach_router_observers(model, hook, num_experts, micro_batch_id_fn, router_class_name,
                                      reduce_tp_cp=reduce_tp_cp, prefer_initial_forward=native_timing)
    return hook, handles


def assert_plan_replicated(plan, group=None) -> bool:
    """True when every rank of ``group`` holds the same plan (trivially true when not distributed)."""
    dist = torch.distributed
    if not dist.is_available() or not dist.is_initialized():
        return True
    flat = torch.cat([torch.tensor([int(plan.theta)], dtype=torch.int64, device=plan.x.device),
                      plan.x.reshape(-1).to(torch.int64), plan.q.reshape(-1).to(torch.int64)])
    got = [torch.empty_like(flat) for _ in range(dist.get_world_size(group))]
    dist.all_gather(got, flat, group=group)
    return all(torch.equal(g, flat) for g in got)
