"""Replica weight channel over one-sided transfers (``EPLB_WEIGHT_COMM=symm``).

The portable library path moves replica weights with one ``dist.broadcast`` per replicated expert
and returns their gradients with one ``dist.reduce`` each (:class:`BroadcastReplicaTransport`).
This module is the device-initiated alternative, the counterpart of the reference's
``GinWeightReplicator`` / ``GinReplicaTransport`` (eplb/integration/gin_weights.py:78-377):

* every rank keeps, per weight tensor ``j``, a symmetric ``home[j]`` window of ``home_cap`` rows
  (its own experts, row ``local_slot(e)`` = position of ``e`` among the experts with the same owner,
  ascending id) and a symmetric ``inbox[j]`` window of ``home_cap * world + 1`` rows (gradient
  inbox; row ``local_slot(e) * world + src_rank``; the last row absorbs nothing and exists so that
  an all-empty schedule still has a valid target);
* forward: owners publish their parameters into ``home`` -> fence -> every host *gets* the rows of
  the experts in its slots straight into a fresh ``[n_slot, ...]`` stack (local experts go through
  the same kernel with ``peer == me``) -> fence;
* backward: every rank clears its inbox -> fence -> every host *puts* the gradient of each slot
  into the owner's inbox column -> fence -> the owner sums the ``world`` columns of each row.

The schedule (who to pull from, where to push to) is computed on the device from ``plan.x``, so no
host read sits on this path.  Replica weights are not kept between forward and backward by this
module: the stack is an ordinary tensor owned by autograd.

Differences from the reference's layout: it stages pulled rows in a third symmetric window
(``slot``) and merges local rows with ``where``; here a get may target any local tensor, so the
stack is filled in place and the staging window does not exist.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..utils import profiling
from .onesided import SymmetricWorld

_SYMM_NAMES = ("symm", "gin", "nccl_gin", "devnccl")


def symm_weights_enabled() -> bool:
    """``EPLB_WEIGHT_COMM`` selects the device-initiated channel; the reference's spellings
    (``gin``, ``nccl_gin``, ``devnccl``; gin_weights.py:47-49) are accepted as aliases."""
    return os.environ.get("EPLB_WEIGHT_COMM", "").strip().lower() in _SYMM_NAMES


def local_slot_table(main_rank: torch.Tensor, world: int) -> Tuple[torch.Tensor, int]:
    """``local_slot_of_e[E]`` (rank of ``e`` among the experts with the same owner) and ``home_cap``."""
    main = main_rank.to(torch.int64)
    E = int(main.numel())
    onehot = torch.zeros((E, world), dtype=torch.int64, device=main.device)
    onehot.scatter_(1, main.view(-1, 1), 1)
    before = onehot.cumsum(0) - onehot                       # experts with the same owner and a smaller id
    local_slot = before.gather(1, main.view(-1, 1)).flatten()
    return local_slot, int(onehot.sum(0).max())


def replica_schedule(x: torch.Tensor, main_rank: torch.Tensor, local_slot_of_e: torch.Tensor, me: int, n_slot: int,
                     world: int) -> Dict[str, torch.Tensor]:
    """Per physical slot of rank ``me``: hosted expert (-1 empty), its owner, the owner's home row and
    the inbox row that this rank's gradient of it goes to.  Pure tensor code, no host read."""
    col = x[:, me].to(torch.int64)
    E = int(col.numel())
    pos = torch.cumsum(col, 0) - 1                             # slot of hosted expert e (ascending id)
    slot_to_e = torch.full((n_slot + 1,), -1, dtype=torch.int64, device=x.device)
    tgt = torch.where((col > 0) & (pos < n_slot), pos, torch.full_like(pos, n_slot))
    slot_to_e.scatter_(0, tgt, torch.where(col > 0, torch.arange(E, device=x.device), torch.full_like(pos, -1)))
    slot_to_e = slot_to_e[:n_slot]
    hosted = slot_to_e >= 0
    e_safe = slot_to_e.clamp_min(0)
    owner = torch.where(hosted, main_rank.to(torch.int64)[e_safe], torch.full_like(e_safe, -1))
    home_row = torch.where(hosted, local_slot_of_e[e_safe], torch.zeros_like(e_safe))
    inbox_row = home_row * world + me
    remote = hosted & (owner != me)
    return {"slot_to_e": slot_to_e, "owner": owner, "home_row": home_row, "inbox_row": inbox_row, "remote": remote}


class SymmWeightReplicator:
    """Static part: symmetric windows for every weight tensor of one expert-parallel group."""

    def __init__(self, world: SymmetricWorld, main_rank: torch.Tensor, weight_shapes: Sequence[Sequence[int]],
                 dtype: torch.dtype) -> None:
        self.world = world
        self.dtype = dtype
        self.weight_shapes = [tuple(int(s) for s in shp) for shp in weight_shapes]
        self.main_rank = main_rank.to(world.device)
        self.local_slot_of_e, self.home_cap = local_slot_table(self.main_rank, world.world)
        es = torch.empty((), dtype=dtype).element_size()
        self.wb = [int(torch.Size(s).numel()) * es for s in self.weight_shapes]
        for b in self.wb:
            if b % 16:
                raise ValueError("expert weight tensors must be a multiple of 16 bytes")
        self.home = [world.create_tensor((self.home_cap,) + s, dtype) for s in self.weight_shapes]
        self.inbox = [world.create_tensor((self.home_cap * world.world + 1,) + s, dtype) for s in self.weight_shapes]
        self.home_off = [world.offset_of(t) for t in self.home]
        self.inbox_off = [world.offset_of(t) for t in self.inbox]
        self._gslot: Dict[int, List[torch.Tensor]] = {}      # n_slot -> per-tensor symmetric gradient staging

    def gslot(self, n_slot: int) -> List[torch.Tensor]:
        """Symmetric ``[n_slot, ...]`` windows where every host stages its slot gradients for the owners
        to read (collective on first use per ``n_slot``)."""
        g = self._gslot.get(int(n_slot))
        if g is None:
            g = [self.world.create_tensor((int(n_slot),) + s, self.dtype) for s in self.weight_shapes]
            self._gslot[int(n_slot)] = g
        return g

    @staticmethod
    def arena_bytes(num_experts: int, world_size: int, weight_shapes, dtype, home_cap: Optional[int] = None,
                    n_slot: int = 0) -> int:
        """Arena size for the home and inbox windows plus one gradient staging window of ``n_slot`` rows."""
        es = torch.empty((), dtype=dtype).element_size()
        cap = home_cap if home_cap is not None else -(-num_experts // world_size)
        total = 0
        for s in weight_shapes:
            wb = int(torch.Size(tuple(s)).numel()) * es
            total += (cap + cap * world_size + 1 + int(n_slot)) * wb + 2048
        return total


class SymmReplicaTransport:
    """Per-plan part: materialises the ``[n_slot, ...]`` stacks and returns their gradients."""

    def __init__(self, rep: SymmWeightReplicator, x: torch.Tensor, n_slot: int,
                 weights_local: Dict[int, Tuple[torch.Tensor, ...]]) -> None:
        self.rep = rep
        self.n_slot = int(n_slot)
        self.weights_local = weights_local
        w = rep.world
        self._x = x.to(w.device)
        self._rt = None
        self._home_has_holes = len(weights_local) < rep.home_cap
        self.sched = replica_schedule(x.to(w.device), rep.main_rank, rep.local_slot_of_e, w.rank, self.n_slot, w.world)
        s = self.sched
        slots = torch.arange(self.n_slot, dtype=torch.int64, device=w.device)
        self._get_desc, self._put_desc = [], []
        for j, wb in enumerate(rep.wb):
            peer = s["owner"]                                   # -1 on empty slots: skipped by the kernel
            self._get_desc.append(torch.stack([peer, rep.home_off[j] + s["home_row"] * wb, slots * wb,
                                               torch.full_like(slots, wb)], 1).contiguous())
            self._put_desc.append(torch.stack([peer, rep.inbox_off[j] + s["inbox_row"] * wb, slots * wb,
                                               torch.full_like(slots, wb)], 1).contiguous())
        self.owned = sorted(weights_local)
        self._owned_rows = rep.local_slot_of_e[torch.tensor(self.owned, dtype=torch.int64, device=w.device)] \
            if self.owned else torch.zeros(0, dtype=torch.int64, device=w.device)

    # ---- forward pieces
    def publish(self, owner_params: Optional[Sequence[torch.Tensor]] = None) -> None:
        """Copy this rank's expert parameters into its ``home`` windows."""
        rep, n_w = self.rep, len(self.rep.weight_shapes)
        if not self.owned:
            return
        params = list(owner_params) if owner_params is not None else \
            [w for e in self.owned for w in self.weights_local[e]]
        for j in range(n_w):
            rows = torch.stack([params[i * n_w + j].detach().to(rep.dtype) for i in range(len(self.owned))], 0)
            rep.home[j].index_copy_(0, self._owned_rows, rows)

    def pull(self) -> List[torch.Tensor]:
        rep, w = self.rep, self.rep.world
        stacks = []
        for j, shp in enumerate(rep.weight_shapes):
            st = torch.zeros((self.n_slot,) + shp, dtype=rep.dtype, device=w.device)
            w.get_batched(st, self._get_desc[j])
            stacks.append(st)
        return stacks

    def materialize_replicas(self, owner_params: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
        """publish -> fence -> pull -> fence (reference: gin_weights.py:305-341)."""
        w = self.rep.world
        nbytes = self.sched["remote"].sum().view(1) * sum(self.rep.wb)   # device tensor, read only when drained
        with profiling.record("apply/weight_move", time_it=True, device=w.device, payload_bytes=nbytes):
            self.publish(owner_params)
            w.world_fence(0)
            stacks = self.pull()
            w.world_fence(1)
        return stacks

    # ---- backward pieces
    def clear_inbox(self) -> None:
        for t in self.rep.inbox:
            t.zero_()

    def push(self, grad_stacks: Sequence[Optional[torch.Tensor]]) -> None:
        rep, w = self.rep, self.rep.world
        for j, g in enumerate(grad_stacks):
            if g is None:
                continue
            w.put_batched(g.to(rep.dtype).contiguous(), self._put_desc[j])

    def collect(self) -> List[torch.Tensor]:
        """Sum the ``world`` inbox columns of every home row: ``[home_cap, ...]`` per weight tensor."""
        rep, w = self.rep, self.rep.world
        out = []
        for j, shp in enumerate(rep.weight_shapes):
            box = rep.inbox[j][: rep.home_cap * w.world].view((rep.home_cap, w.world) + shp)
            out.append(box.sum(1, dtype=torch.float32).to(rep.dtype))
        return out

    # ---- owner-side reduce (bf16): hosts stage, owners read their replicas' rows and sum in registers
    def owner_reduce_available(self) -> bool:
        rep = self.rep
        return rep.dtype == torch.bfloat16 and rep.world.world <= 64 and all(b % 16 == 0 for b in rep.wb)

    def _reduce_tables(self):
        if getattr(self, "_rt", None) is None:
            rep, w = self.rep, self.rep.world
            x = self._x.to(torch.int64)
            slot_of = torch.where(x > 0, torch.cumsum(x, 0) - 1, torch.full_like(x, -1))
            slot_of = torch.where(slot_of < self.n_slot, slot_of, torch.full_like(slot_of, -1)).to(torch.int32).contiguous()
            gs = rep.gslot(self.n_slot)
            ptrs = [torch.tensor([w.heap.address("arena", r) + w.offset_of(t) for r in range(w.world)],
                                 dtype=torch.int64, device=w.device) for t in gs]
            self._rt = (slot_of, rep.main_rank.to(torch.int32).contiguous(),
                        rep.local_slot_of_e.to(torch.int32).contiguous(), gs, ptrs)
        return self._rt

    def stage(self, grad_stacks: Sequence[Optional[torch.Tensor]]) -> None:
        _, _, _, gs, _ = self._reduce_tables()
        for j, g in enumerate(grad_stacks):
            if g is None:
                gs[j].zero_()
            else:
                gs[j].copy_(g)

    def owner_sum(self) -> List[torch.Tensor]:
        """``[home_cap, ...]`` per weight tensor: sum over every host's staged row (peer loads, fp32 accumulate)."""
        rep, w = self.rep, self.rep.world
        slot_of, main32, home32, _, ptrs = self._reduce_tables()
        out = []
        for j, shp in enumerate(rep.weight_shapes):
            # rows of home slots that hold no expert are never written: start from zeros only then
            acc = (torch.zeros if self._home_has_holes else torch.empty)((rep.home_cap,) + shp, dtype=rep.dtype,
                                                                         device=w.device)
            w.ext.grad_reduce(ptrs[j], rep.wb[j] // 2, slot_of, main32, home32, w.rank, rep.home_cap, acc, True, True)
            out.append(acc)
        return out

    def reduce_grads(self, grad_stacks: Sequence[Optional[torch.Tensor]]) -> List[torch.Tensor]:
        """Returns one gradient per owned expert and weight tensor, in ``sorted(weights_local)`` order.

        bf16 weights: stage -> fence -> owners sum their replicas' rows with peer loads -> fence (the
        gradient crosses NVLink once and nothing is zeroed or re-read).  Other dtypes take the
        reference's inbox protocol: clear -> fence -> push -> fence -> sum (gin_weights.py:343-377)."""
        w = self.rep.world
        n_w = len(self.rep.weight_shapes)
        if self.owner_reduce_available():
            with profiling.record("apply/grad_move", time_it=True, device=w.device):
                self.stage(grad_stacks)
                w.world_fence(2)
                rows = self.owner_sum()
                w.world_fence(3)
            mine = [rows[j].index_select(0, self._owned_rows) for j in range(n_w)]
            return [mine[j][i] for i in range(len(self.owned)) for j in range(n_w)]
        with profiling.record("apply/grad_move", time_it=True, device=w.device):
            self.clear_inbox()
            w.world_fence(2)
            self.push(grad_stacks)
            w.world_fence(3)
            rows = self.collect()
        n_w = len(self.rep.weight_shapes)
        mine = [rows[j].index_select(0, self._owned_rows) for j in range(n_w)]
        return [mine[j][i] for i in range(len(self.owned)) for j in range(n_w)]

    # ---- the two halves without autograd (what a WeightLease calls)
    def acquire(self, owner_params: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
        return self.materialize_replicas(owner_params)

    def give_back(self, grad_stacks: Sequence[Optional[torch.Tensor]]) -> List[torch.Tensor]:
        return self.reduce_grads(grad_stacks)

    # ---- protocol used by the library path
    def materialize(self, rows: Sequence[torch.Tensor] = ()):
        params = [w for e in self.owned for w in self.weights_local[e]]
        out = _SymmMaterialize.apply(self, len(rows), *rows, *params)
        if not rows:
            return tuple(out)
        return tuple(out[: len(rows)]), tuple(out[len(rows):])


class _SymmMaterialize(torch.autograd.Function):
    """Forward = :meth:`SymmReplicaTransport.materialize_replicas`; backward =
    :meth:`SymmReplicaTransport.reduce_grads`.  The received token rows are passed through the node
    unchanged so that, on every rank, the gradient fences of this node run before the reverse token
    all-to-alls (device fences and collectives share one stream, so their order must not depend on
    how autograd schedules each rank's graph)."""

    @staticmethod
    def forward(ctx, tr: SymmReplicaTransport, n_rows: int, *tensors):
        rows, params = tensors[:n_rows], tensors[n_rows:]
        ctx.tr, ctx.n_rows = tr, n_rows
        stacks = tr.materialize_replicas(params)
        return (*[r.view_as(r) for r in rows], *stacks)

    @staticmethod
    def backward(ctx, *grad_all):
        grad_rows, grad_stacks = grad_all[: ctx.n_rows], grad_all[ctx.n_rows:]
        grads = ctx.tr.reduce_grads(grad_stacks)
        return (None, None, *grad_rows, *grads)


# ---------------------------------------------------------------------- cache used by the library path
_REPLICATORS: Dict[tuple, SymmWeightReplicator] = {}


def replicator_for(group, main_rank: torch.Tensor, weight_shapes, dtype, device) -> SymmWeightReplicator:
    """One replicator (and one symmetric arena) per (group, shapes, dtype); created collectively on
    first use, as the reference caches its replicators per layer shape (eplb_manager.py:67-83)."""
    import torch.distributed as dist

    shapes = tuple(tuple(int(s) for s in shp) for shp in weight_shapes)
    key = (id(group), shapes, dtype, int(main_rank.numel()))
    rep = _REPLICATORS.get(key)
    if rep is None:
        world_size = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        _, cap = local_slot_table(main_rank, world_size)
        arena = SymmWeightReplicator.arena_bytes(int(main_rank.numel()), world_size, shapes, dtype, home_cap=cap,
                                                 n_slot=2 * cap + 8)
        world = SymmetricWorld(arena, device, group=group)
        rep = SymmWeightReplicator(world, main_rank, shapes, dtype)
        _REPLICATORS[key] = rep
    return rep


def clear_replicators() -> None:
    for rep in _REPLICATORS.values():
        rep.world.destroy()
    _REPLICATORS.clear()
