"""Expert-parallel MoE feed-forward layer with per-step load balancing, on native kernels.

One forward does, entirely on the device and without any host read:

  router (PyTorch)  ->  count + publish omega  ->  solve plan  ->  route units  ->  dispatch
  token rows into the hosts' buffers  ->  pull replica weights  ->  grouped GEMM1 + SwiGLU  ->
  grouped GEMM2 with rows scattered back to their source rank  ->  gate-weighted reduce.

and the backward mirrors it (gradient dispatch with fused gate gradients, Wgrad/Dgrad grouped
GEMMs, the activation gradient as one coalesced pass or fused into the Dgrad2 epilogue, owner-side
reduction of replica weight gradients).  A unit's gate weight travels with its token row and is folded
into the activation by GEMM1's epilogue, so GEMM2 produces weighted rows, the combine is a plain sum and
the backward pass sends the output gradient unscaled; the hosts apply the weight and compute the
gate-weight gradients in their SwiGLU-gradient pass and store them back to the units' source ranks.  Forwards that run without autograd can use block-scaled fp8
expert GEMMs (``MoEConfig.fp8_inference``) and select experts with one fused router kernel.
This is the B200 counterpart of the reference's apply mode
(eplb/integration/eplb_manager.py:905-1167 ``sync_free_moe_forward``, megatron_moe.py:156-215).

Weight layout: every rank holds ``w_slots`` expert slots in symmetric memory.  Slots
``[0, home_cap)`` are the experts this rank owns -- those *are* the parameters, the optimizer
updates them in place -- and the remaining slots receive replicas chosen by the plan each step.
Weights use the ``[out, in]`` layout: ``w1[slot]`` is ``[2F, H]`` (gate rows then up rows) and
``w2[slot]`` is ``[H, F]`` (reference: eplb/integration/grouped_mlp.py:117-137).

Weight gradients are written straight into ``param.grad`` (a view of the symmetric gradient
slots), overwriting the previous content; replicas' contributions are added by the owner.  With
``MoEConfig.grad_accum_dtype`` they are accumulated over micro-batches instead.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..core.config import EPLBConfig
from ..core.problem import ProblemSpec
from ..core.topology import Topology
from ..ops.extension import load
from ..parallel.symm import HeapLayout, SymmetricHeap
from ..utils import profiling

from ..utils.status import STATUS_NAMES  # noqa: E402,F401  (re-exported)


@dataclass
class MoEConfig:
    hidden: int
    ffn: int
    num_experts: int
    top_k: int
    max_tokens: int  # tokens per rank per step
    extra_slots: int = 2  # replica slots per rank on top of the owned experts
    capacity_factor: float = 2.0  # receive-buffer rows as a multiple of this rank's units
    num_domains: int = 1
    intra_cost: int = 1
    inter_cost: int = 8
    router_dtype: torch.dtype = torch.float32
    normalize_topk: bool = True
    gemm_ctas: int = 2  # 2: CTA-pair grouped GEMM (256-row tiles); 1: single-CTA kernel (128-row tiles)
    # None: every backward overwrites ``param.grad``.  torch.bfloat16 / torch.float32: every backward ADDS the
    # expert weight gradients into an accumulation buffer of that dtype (``param.grad`` for bf16,
    # ``param.main_grad`` for fp32), for steps made of several micro-batches; clear it with
    # ``FusedMoE.zero_grad_accum()`` (or ``optimizer.zero_grad(set_to_none=False)`` in the bf16 case).
    grad_accum_dtype: Optional[torch.dtype] = None
    # True: forwards that run without autograd (inference) use block-scaled fp8 expert GEMMs (e4m3, 1 x 128
    # activation scales, 128 x 128 weight scales, power-of-two scale factors).  Call
    # ``FusedMoE.quantize_weights()`` after the weights change; replicas then pull the fp8 copies.
    fp8_inference: bool = False
    # > 0: switch-style auxiliary load-balancing loss  coeff * E * sum_e f_e * P_e  (f_e: share of routed units,
    # P_e: mean router probability) is left in ``FusedMoE.aux_loss`` by every forward that runs with autograd.
    # 0 (default): no balancing pressure on the router, the routing skew reaches the dispatcher intact.
    aux_loss_coeff: float = 0.0
    # True: the token transport of a pass (dispatch + replica weight pull in forward, gradient dispatch in
    # backward) runs on spare warps of the GEMM kernel that consumes the rows, so transfer and tensor-core
    # tiles overlap.  False: a stand-alone transport kernel runs first.  ``EPLB_FUSED_COMM=0`` overrides.
    fused_comm: bool = True
    # Budget of every cross-rank wait inside this layer's kernels, in milliseconds (always bounded; on expiry
    # the kernel records a status and returns).  ``EPLB_WAIT_MS`` overrides.
    wait_ms: int = 1500


# Regions that only live inside one layer's forward or backward pass: a model keeps ONE copy of them for
# all its layers (``heap_layout(..., layers=n)``).  Reuse across layers is safe without extra barriers: a
# peer writes layer L+1's rows into this rank's scratch only after its solver has seen this rank's
# publish for L+1 (forward), or after this rank's gradient rows for that layer reached it (backward), and
# both follow, in this rank's stream, the kernels that read the previous layer's contents.
SHARED_SYMM = ("ybuf", "dybuf", "dxbuf", "dprob", "xq", "sfx")
SHARED_LOCAL = ("dact", "actq", "sfact")


def region_name(name: str, layer: Optional[int]) -> str:
    """Heap region of ``name`` for layer ``layer`` of a model heap (None: a single-layer heap, plain names)."""
    if layer is None:
        return name
    return f"S.{name}" if name in SHARED_SYMM else f"L{layer}.{name}"


def heap_layout(cfg: MoEConfig, world: int, layers: Optional[int] = None) -> HeapLayout:
    """Symmetric regions (identical on every rank) of one layer, or -- with ``layers`` -- of a whole model:
    per-layer state under ``L<i>.`` and one set of per-step scratch buffers under ``S.``; one allocation and
    one handle exchange per model."""
    E, H, F = cfg.num_experts, cfg.hidden, cfg.ffn
    home_cap = -(-E // world)
    w_slots = home_cap + (cfg.extra_slots if world > 1 else 0)
    U = cfg.max_tokens * cfg.top_k
    cap = row_capacity(cfg, world)
    lay = HeapLayout()
    per_layer = [
        ("omega", (world, E), torch.int32),
        ("signals", (16,), torch.int32),
        # arrival counters per GEMM M-tile of the receive buffers (forward, backward) + replica pull counters
        ("arrive", (2 * (cap // (128 * cfg.gemm_ctas)) + 2 * max(w_slots - home_cap, 0) + 4,), torch.int32),
        ("xbuf", (cap, H), torch.bfloat16),
        ("meta", (cap, 2), torch.int32),
        ("rowp", (cap,), torch.float32),      # gate weight of every received row (stored by its sender)
        ("w1", (w_slots, 2 * F, H), torch.bfloat16),
        ("w2", (w_slots, H, F), torch.bfloat16),
        ("gw1", (w_slots, 2 * F, H), torch.bfloat16),
        ("gw2", (w_slots, H, F), torch.bfloat16),
    ]
    scratch = [
        ("dprob", (U,), torch.float32),       # gate-weight gradients of this rank's units (stored by their hosts)
        ("ybuf", (U, H), torch.bfloat16),
        ("dybuf", (cap, H), torch.bfloat16),
        ("dxbuf", (U, H), torch.bfloat16),
    ]
    if cfg.fp8_inference:
        per_layer += [
            ("w1q", (w_slots, 2 * F, H), torch.uint8),
            ("w2q", (w_slots, H, F), torch.uint8),
            ("sfb1", (w_slots, _sf_bytes(2 * F, H)), torch.uint8),
            ("sfb2", (w_slots, _sf_bytes(H, F)), torch.uint8),
        ]
        scratch += [
            ("xq", (cap, H), torch.uint8),                      # received rows, quantised by the sender
            ("sfx", (cap // 128 * _sf_bytes(128, H),), torch.uint8),
        ]
    if layers is None:
        for name, shape, dtype in per_layer + scratch:
            lay.add(name, shape, dtype)
        return lay
    for i in range(int(layers)):
        for name, shape, dtype in per_layer:
            lay.add(region_name(name, i), shape, dtype)
    for name, shape, dtype in scratch:
        lay.add(region_name(name, 0), shape, dtype)
    return lay


def _sf_bytes(n: int, k: int) -> int:
    """Bytes of the scale-factor chunks of an ``[n, k]`` operand (512 per 128 rows and four 128-wide k-blocks)."""
    return (n // 128) * ((k // 128 + 3) // 4) * 512


def row_capacity(cfg: MoEConfig, world: int) -> int:
    U = cfg.max_tokens * cfg.top_k
    home_cap = -(-cfg.num_experts // world)
    w_slots = home_cap + (cfg.extra_slots if world > 1 else 0)
    tile = 128 * cfg.gemm_ctas  # every group starts on a GEMM M-tile boundary
    rows = int(U * (cfg.capacity_factor if world > 1 else 1.0)) + tile * w_slots
    return (rows + tile - 1) // tile * tile


def _split3(w: torch.Tensor) -> torch.Tensor:
    """fp32 ``[A, B]`` -> bf16 ``[3A, B]`` whose three row blocks sum to ``w`` to 24 mantissa bits."""
    hi = w.to(torch.bfloat16)
    r1 = w - hi.float()
    mid = r1.to(torch.bfloat16)
    lo = (r1 - mid.float()).to(torch.bfloat16)
    return torch.cat([hi, mid, lo], 0)


class _RouterLinear(torch.autograd.Function):
    """fp32 router logits ``x @ W^T`` from bf16 tokens on the tensor cores, without an fp32 copy of ``x``.

    ``W`` (fp32) is split into three bf16 terms; bf16 x bf16 products are exact in the fp32 accumulator,
    so one bf16 GEMM against the stacked terms reproduces the fp32 product to fp32 rounding.  The weight
    gradient splits the (fp32) logit gradient the same way.  Library GEMMs (the router is not one of the
    fused expert paths)."""

    @staticmethod
    def forward(ctx, x, w):
        E = w.shape[0]
        stacked = torch.mm(x, _split3(w).t(), out_dtype=torch.float32)      # [N, 3E]
        ctx.save_for_backward(x, w)
        return stacked.view(x.shape[0], 3, E).sum(1)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        E = w.shape[0]
        g = g.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[1]:
            g3 = _split3(g.t().contiguous())                                  # [3E, N] bf16
            dw = torch.mm(g3, x, out_dtype=torch.float32).view(3, E, -1).sum(0)
        if ctx.needs_input_grad[0]:
            dx = torch.mm(g.to(torch.bfloat16), w.to(torch.bfloat16))
        return dx, dw


class _FusedMoEFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, topk_idx, topk_prob, layer):
        n = tokens.shape[0]
        out = torch.empty_like(tokens)
        layer.rt.forward(tokens.data_ptr(), topk_idx.data_ptr(), topk_prob.data_ptr(), out.data_ptr(), n)
        # Backward reads what this forward left in the layer's buffers (received rows, pre-activations, routing
        # tables): one forward, then its backward.  A second forward in between would silently replace them, so
        # the forward is numbered and backward checks the number.
        layer._forward_generation += 1
        ctx.generation = layer._forward_generation
        ctx.layer = layer
        ctx.save_for_backward(topk_prob)
        ctx.n = n
        ctx.keep = (tokens, topk_idx)  # inputs stay alive until the enqueued kernels have read them
        return out

    @staticmethod
    def backward(ctx, dout):
        layer = ctx.layer
        if ctx.generation != layer._forward_generation:
            raise RuntimeError("FusedMoE.backward: the layer ran another forward (generation "
                               f"{layer._forward_generation}) after the one this backward belongs to ({ctx.generation}); "
                               "its saved activations live in the layer's buffers, so every forward must be followed "
                               "by its backward before the next forward with autograd enabled")
        (topk_prob,) = ctx.saved_tensors
        dout = dout.contiguous()
        dtokens = torch.empty_like(dout)
        dprob = torch.empty_like(topk_prob)
        layer.rt.backward(dout.data_ptr(), dtokens.data_ptr(), dprob.data_ptr(), ctx.n)
        layer.bind_grads()
        return dtokens, None, dprob, None


class FusedMoE(nn.Module):
    """One MoE FFN layer of an expert-parallel group (``world`` ranks; this object is rank ``rank``).

    ``heap`` is a :class:`SymmetricHeap` built from :func:`heap_layout`; with the ``local`` backend
    several ``FusedMoE`` objects (one per logical rank) can share one heap in a single process.
    """

    def __init__(self, cfg: MoEConfig, heap: SymmetricHeap, rank: int, world: int, *,
                 solver_cfg: Optional[EPLBConfig] = None, multi_rank_sync: bool = True, seed: int = 0,
                 layer_index: Optional[int] = None, scratch: Optional[Dict[str, torch.Tensor]] = None,
                 status: Optional[torch.Tensor] = None) -> None:
        """``layer_index``: this layer's position in a model heap built with ``heap_layout(cfg, world, layers=n)``
        (None: ``heap`` holds this layer alone).  ``scratch``: a dict shared by the layers of a model in which the
        per-step local buffers are created once.  ``status``: an int32 ``[4]`` view to use as this layer's status
        word (a row of a :class:`~ep_balance_b200.utils.status.StatusBoard`)."""
        super().__init__()
        self.cfg, self.heap, self.rank, self.world = cfg, heap, int(rank), int(world)
        self.layer_index = layer_index
        self._forward_generation = 0   # forwards that went through autograd (see _FusedMoEFunction)
        sym = lambda name: region_name(name, layer_index)  # noqa: E731
        self.solver_cfg = solver_cfg or EPLBConfig()
        dev = heap.device
        self.device = dev
        E, H, F, K = cfg.num_experts, cfg.hidden, cfg.ffn, cfg.top_k
        if E % world:
            raise ValueError("num_experts must be divisible by the expert-parallel world size")
        self.home_cap = E // world
        self.w_slots = self.home_cap + (cfg.extra_slots if world > 1 else 0)
        self.n_slot_plan = self.w_slots
        self.row_capacity = row_capacity(cfg, world)
        self.max_units = cfg.max_tokens * K
        self.topo = Topology.logical(world, cfg.num_domains, cfg.intra_cost, cfg.inter_cost)
        wbytes = 3 * H * F * 2
        self.spec = ProblemSpec.contiguous_main_placement(E, world, wbytes, H * 2, self.n_slot_plan)

        # ---- parameters: router + the owned expert slots (views of symmetric memory)
        g = torch.Generator(device="cpu").manual_seed(1234 + seed)
        self.router = nn.Parameter((torch.randn(E, H, generator=g) * 0.02).to(dev, cfg.router_dtype))
        w1_all, w2_all = heap.tensor(sym("w1"), rank), heap.tensor(sym("w2"), rank)
        ge = torch.Generator(device=dev)
        for i in range(self.home_cap):
            e = rank * self.home_cap + i
            ge.manual_seed(10_000 + 7919 * seed + e)  # weights depend on the expert id only, not on the world size
            w1_all[i].copy_((torch.randn(2 * F, H, generator=ge, device=dev) * 0.02).to(torch.bfloat16))
            w2_all[i].copy_((torch.randn(H, F, generator=ge, device=dev) * 0.02).to(torch.bfloat16))
        self.w1 = nn.Parameter(w1_all[: self.home_cap])
        self.w2 = nn.Parameter(w2_all[: self.home_cap])
        self._gw1 = heap.tensor(sym("gw1"), rank)[: self.home_cap]
        self._gw2 = heap.tensor(sym("gw2"), rank)[: self.home_cap]
        self.router_bias: Optional[torch.Tensor] = None  # additive logit skew (synthetic workloads)
        self.aux_loss: Optional[torch.Tensor] = None     # auxiliary balancing loss of the last forward (aux_loss_coeff > 0)
        self.route_fn = None  # optional ``logits [N, E] -> (top_idx int64 [N, K], prob fp32 [N, K])``
        # Inference (no autograd) selects experts with one fused kernel.  ``None``: the default top-k + softmax
        # (or sigmoid) router; a model with its own ``route_fn`` sets ``dict(mode=2, n_groups=, topk_groups=, scale=)``
        # to get the fused group-limited variant, or ``False`` to always use ``route_fn``.
        self.fused_router = None

        # ---- local state
        i32 = dict(dtype=torch.int32, device=dev)
        R = world
        self.loc: Dict[str, torch.Tensor] = {
            "dom": self.topo.domain_of_rank.to(**i32), "cost": self.topo.cost.to(**i32).contiguous(),
            "main_rank": self.spec.main_rank.to(**i32), "weight_bytes": self.spec.weight_bytes.to(dev),
            "home_index": (torch.arange(E) % self.home_cap).to(**i32),
            "x": torch.zeros((E, R), dtype=torch.int8, device=dev), "q": torch.zeros((R, E, R), **i32),
            "erl": torch.zeros((E, R), **i32), "rank_load": torch.zeros(R, **i32),
            "slot_used": torch.zeros(R, **i32), "stuck": torch.zeros(R, dtype=torch.uint8, device=dev),
            "theta": torch.zeros(1, dtype=torch.int64, device=dev),
            "control": torch.zeros(3, dtype=torch.int64, device=dev), "sync": torch.zeros(2, **i32),
            "status": status if status is not None else torch.zeros(4, **i32), "epochs": torch.zeros(8, **i32),
            "slot_of": torch.full((E, R), -1, **i32), "row_base": torch.full((E, R), -1, **i32),
            "group_expert": torch.full((self.w_slots,), -1, **i32), "group_wslot": torch.zeros(self.w_slots, **i32),
            "group_off": torch.zeros(self.w_slots + 1, **i32), "group_rows": torch.zeros(self.w_slots, **i32),
            "totals": torch.zeros(2, **i32),
            "send_off": torch.zeros((E, R), **i32), "tiles_of": torch.zeros(R, **i32),
            "chunk_hist": torch.zeros((-(-self.max_units // 256), E), **i32), "hist_acc": torch.zeros(E + 1, **i32),
            "exp_prefix": torch.zeros(E + 1, **i32), "sorted_units": torch.zeros(self.max_units, **i32),
            "done_ctr": torch.zeros(4, **i32),
            "unit_dst": torch.zeros(self.max_units, **i32), "unit_row": torch.zeros(self.max_units, **i32),
            "unit_pos": torch.zeros(self.max_units, **i32),
            "hbuf": torch.zeros((self.row_capacity, 2 * F), dtype=torch.bfloat16, device=dev),
            "act": torch.zeros((self.row_capacity, F), dtype=torch.bfloat16, device=dev),
        }
        if status is not None and (status.shape != (4,) or status.dtype != torch.int32 or status.device != torch.device(dev)
                                   or not status.is_contiguous()):
            raise ValueError("status must be a contiguous int32 [4] tensor on the layer's device")

        def local_scratch(name, shape, dtype):
            pool = scratch if scratch is not None else {}
            t = pool.get(name)
            if t is None or t.shape != tuple(shape) or t.dtype != dtype:
                t = pool[name] = torch.zeros(shape, dtype=dtype, device=dev)
            return t

        self.loc["dact"] = local_scratch("dact", (self.row_capacity, F), torch.bfloat16)
        if os.environ.get("EPLB_TRACE_FUSED", "0") not in ("", "0"):
            # profiling aid: the fused transport+GEMM kernels leave four timestamps each (see fused_trace())
            self.loc["gemm_trace"] = torch.zeros(24, dtype=torch.int64, device=dev)
        ptrs = {k: v.data_ptr() for k, v in self.loc.items()}
        self._acc_gw1 = self._acc_gw2 = None
        if cfg.grad_accum_dtype is not None:
            if cfg.grad_accum_dtype not in (torch.bfloat16, torch.float32):
                raise ValueError("grad_accum_dtype must be None, torch.bfloat16 or torch.float32")
            self._acc_gw1 = torch.zeros((self.home_cap, 2 * F, H), dtype=cfg.grad_accum_dtype, device=dev)
            self._acc_gw2 = torch.zeros((self.home_cap, H, F), dtype=cfg.grad_accum_dtype, device=dev)
            ptrs["acc_gw1"], ptrs["acc_gw2"] = self._acc_gw1.data_ptr(), self._acc_gw2.data_ptr()
        symm_names = ["omega", "signals", "arrive", "xbuf", "meta", "rowp", "dprob", "ybuf", "dybuf", "dxbuf", "w1", "w2", "gw1", "gw2"]
        table_names = [("omega", "omega_ptrs"), ("signals", "signal_ptrs"), ("arrive", "arrive_ptrs"), ("xbuf", "xbuf_ptrs"),
                       ("meta", "meta_ptrs"), ("rowp", "rowp_ptrs"), ("dprob", "dprob_ptrs"), ("ybuf", "ybuf_ptrs"), ("dybuf", "dybuf_ptrs"),
                       ("dxbuf", "dxbuf_ptrs"), ("w1", "w1_ptrs"), ("w2", "w2_ptrs"), ("gw1", "gw1_ptrs"),
                       ("gw2", "gw2_ptrs")]
        self._fp8_ready = False
        if cfg.fp8_inference:
            if H % 128 or F % 128:
                raise ValueError("fp8_inference needs hidden and ffn to be multiples of 128")
            symm_names += ["w1q", "w2q", "sfb1", "sfb2", "xq", "sfx"]
            table_names += [(n, n + "_ptrs") for n in ("w1q", "w2q", "sfb1", "sfb2", "xq", "sfx")]
            cap = self.row_capacity
            self._fp8_local = {"actq": local_scratch("actq", (cap, F), torch.uint8),
                               "sfact": local_scratch("sfact", (cap // 128 * _sf_bytes(128, F),), torch.uint8)}
            ptrs.update({k: v.data_ptr() for k, v in self._fp8_local.items()})
        for name in symm_names:
            ptrs[name] = heap.address(sym(name), rank)
        self._tables: List[torch.Tensor] = []
        for name, key in table_names:
            t = heap.peer_ptrs(sym(name))
            self._tables.append(t)
            ptrs[key] = t.data_ptr()
        sc = self.solver_cfg
        iters = sc.device_stage2_iters
        props = torch.cuda.get_device_properties(dev)
        rt_cfg = dict(R=R, me=rank, E=E, H=H, F=F, topk=K, w_slots=self.w_slots, home_cap=self.home_cap,
                      n_slot_plan=self.n_slot_plan, row_capacity=self.row_capacity, max_units=self.max_units,
                      D=cfg.num_domains, u_min=sc.u_min, iters=iters, patience=sc.stage2_stagnation_patience,
                      allow_cross=int(sc.allow_cross_domain),
                      probe=int(sc.stage2_patience_all_scales and iters > sc.stage2_stagnation_patience + 1),
                      s_tok=H * 2, num_sms=props.multi_processor_count, multi_rank_sync=int(multi_rank_sync),
                      gemm_ctas=cfg.gemm_ctas, accum_fp32=int(cfg.grad_accum_dtype == torch.float32),
                      fused_comm=int(os.environ.get("EPLB_FUSED_COMM", int(cfg.fused_comm))),
                      wait_ms=int(os.environ.get("EPLB_WAIT_MS", cfg.wait_ms)))
        self.rt_config = rt_cfg
        self.rt = load().MoeRuntime(rt_cfg, ptrs)
        self.bind_grads()

    # ---- gradients ---------------------------------------------------------
    def bind_grads(self) -> None:
        """Point ``.grad`` of the expert parameters at the symmetric gradient slots, or at the
        accumulation buffers when ``grad_accum_dtype`` is set (fp32: ``.main_grad``, ``.grad`` stays None)."""
        if self._acc_gw1 is not None:
            if self._acc_gw1.dtype == torch.float32:
                self.w1.main_grad, self.w2.main_grad = self._acc_gw1, self._acc_gw2
                return
            if self.w1.grad is None or self.w1.grad.data_ptr() != self._acc_gw1.data_ptr():
                self.w1.grad = self._acc_gw1
            if self.w2.grad is None or self.w2.grad.data_ptr() != self._acc_gw2.data_ptr():
                self.w2.grad = self._acc_gw2
            return
        if self.w1.grad is None or self.w1.grad.data_ptr() != self._gw1.data_ptr():
            self.w1.grad = self._gw1
        if self.w2.grad is None or self.w2.grad.data_ptr() != self._gw2.data_ptr():
            self.w2.grad = self._gw2

    def quantize_weights(self) -> None:
        """Refresh the fp8 copies (and scale factors) of this rank's own experts from the bf16 parameters.
        In a multi-rank group, call it on every rank and synchronise (e.g. ``dist.barrier`` after a stream
        sync) before the next fp8 forward: replicas read the owners' fp8 slots."""
        if not self.cfg.fp8_inference:
            raise RuntimeError("MoEConfig.fp8_inference is off")
        self.rt.quantize_own_weights()
        self._fp8_ready = True

    def zero_grad_accum(self) -> None:
        """Clear the gradient accumulation buffers (start of a step made of several micro-batches)."""
        if self._acc_gw1 is not None:
            self._acc_gw1.zero_()
            self._acc_gw2.zero_()

    # ---- routing -----------------------------------------------------------
    def route_tokens(self, tokens: torch.Tensor):
        """fp32 router: logits = x . W_r^T (+ bias), top-k, softmax over the selected logits."""
        with profiling.record("apply/route", time_it=True, device=tokens.device):
            if tokens.is_cuda and tokens.dtype == torch.bfloat16 and self.router.dtype == torch.float32:
                logits = _RouterLinear.apply(tokens, self.router)
            else:
                logits = tokens.to(self.router.dtype) @ self.router.t()
            if tokens.is_cuda and not torch.is_grad_enabled() and logits.dtype == torch.float32 and (
                    self.fused_router or (self.fused_router is None and self.route_fn is None)):
                fr = self.fused_router or dict(mode=0 if self.cfg.normalize_topk else 1, n_groups=1, topk_groups=1, scale=1.0)
                top_idx = torch.empty((tokens.shape[0], self.cfg.top_k), dtype=torch.int64, device=tokens.device)
                prob = torch.empty((tokens.shape[0], self.cfg.top_k), dtype=torch.float32, device=tokens.device)
                load().router_topk(logits.contiguous(), self.router_bias, fr["mode"], fr["n_groups"], fr["topk_groups"],
                                   fr["scale"], top_idx, prob)
                return top_idx, prob
            if self.router_bias is not None:
                logits = logits + self.router_bias
            if self.route_fn is not None:
                top_idx, prob = self.route_fn(logits)
                return top_idx.contiguous(), prob.float().contiguous()
            top_val, top_idx = torch.topk(logits, self.cfg.top_k, dim=-1)
            prob = torch.softmax(top_val.float(), dim=-1) if self.cfg.normalize_topk else torch.sigmoid(top_val.float())
            self.aux_loss = None
            if self.cfg.aux_loss_coeff > 0 and torch.is_grad_enabled():
                E = self.cfg.num_experts
                share = torch.zeros(E, dtype=torch.float32, device=logits.device).scatter_add_(
                    0, top_idx.reshape(-1), torch.ones(top_idx.numel(), dtype=torch.float32, device=logits.device))
                share = share / max(top_idx.numel(), 1)
                self.aux_loss = self.cfg.aux_loss_coeff * E * (share * torch.softmax(logits.float(), dim=-1).mean(0)).sum()
        return top_idx.contiguous(), prob.contiguous()

    def apply_routed(self, tokens: torch.Tensor, top_idx: torch.Tensor, prob: torch.Tensor) -> torch.Tensor:
        """Expert computation for an externally made routing decision (``top_idx`` int64 ``[N, K]``, ``prob``
        fp32 ``[N, K]``): what a framework binding calls after running its own router."""
        return _FusedMoEFunction.apply(tokens.contiguous(), top_idx.contiguous(), prob.float().contiguous(), self)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        if tokens.dtype != torch.bfloat16 or tokens.dim() != 2 or tokens.shape[1] != self.cfg.hidden:
            raise ValueError("tokens must be bf16 [num_tokens, hidden]")
        if tokens.shape[0] > self.cfg.max_tokens:
            raise ValueError("more tokens than MoEConfig.max_tokens")
        tokens = tokens.contiguous()
        top_idx, prob = self.route_tokens(tokens)
        if self.cfg.fp8_inference and self._fp8_ready and not torch.is_grad_enabled():
            out = torch.empty_like(tokens)
            self.rt.forward_fp8(tokens.data_ptr(), top_idx.data_ptr(), prob.data_ptr(), out.data_ptr(), tokens.shape[0])
            self._keep = (tokens, top_idx, prob)  # alive until the enqueued kernels have read them
            return out
        return _FusedMoEFunction.apply(tokens, top_idx, prob, self)

    def fused_trace_reset(self) -> None:
        if "gemm_trace" in self.loc:
            one = [-1, 0, 0, -1, 0, 0, 0, 0, 0, 0, 0, 0]
            self.loc["gemm_trace"].copy_(torch.tensor(one + one, dtype=torch.int64), non_blocking=True)

    def fused_trace(self) -> Dict[str, float]:
        """With ``EPLB_TRACE_FUSED=1``: microseconds, from the first transport warp's start, until the last transport
        warp finished / the last MMA was issued / the first tile had its operands, for the forward (dispatch +
        GEMM1) and the backward (gradient dispatch + Dgrad2) kernel of the last step.  Call ``fused_trace_reset()``
        before the step; reads device memory."""
        if "gemm_trace" not in self.loc:
            return {}
        t = self.loc["gemm_trace"].tolist()
        out = {}
        warps = 2 * self.rt_config["num_sms"]  # transport warps of a fused launch
        for name, o in (("fwd", 0), ("bwd", 12)):
            if t[o + 1] > 0:
                out[f"{name}_transport_us"] = (t[o + 1] - t[o]) / 1e3
                out[f"{name}_mma_end_us"] = (t[o + 2] - t[o]) / 1e3
                out[f"{name}_first_tile_us"] = (t[o + 3] - t[o]) / 1e3
                # per transport warp: time waiting for loads / for ring slots / in drains, and segments moved
                out[f"{name}_warp_load_wait_us"] = t[o + 8] / warps / 1e3
                out[f"{name}_warp_slot_wait_us"] = t[o + 9] / warps / 1e3
                out[f"{name}_warp_drain_us"] = t[o + 10] / warps / 1e3
                out[f"{name}_warp_segments"] = t[o + 11] / warps * 1e3
        return out

    def omega(self) -> torch.Tensor:
        """This rank's gathered load matrix ``[R, E]`` (int32 view of symmetric memory)."""
        return self.heap.tensor(region_name("omega", self.layer_index), self.rank)

    # ---- introspection (these read device memory: debugging / tests only) ---
    def check_status(self) -> None:
        """Synchronous read of this layer's status word; raises :class:`MoEStatusError` when it is set."""
        from ..utils.status import raise_if_set

        rows = [[0, 0, 0, 0]] * (self.layer_index or 0) + [self.loc["status"].tolist()]
        raise_if_set(rows)

    def last_plan(self):
        from ..core.plan import Plan

        return Plan(self.loc["x"].clone(), self.loc["q"].to(torch.int64), self.loc["theta"][0].clone())

    def rank_loads(self) -> torch.Tensor:
        return self.loc["rank_load"].clone()
