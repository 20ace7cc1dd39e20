"""Replication-aware MoE forward on library collectives (gloo on CPU, NCCL on GPUs).

This is the portable statement of apply mode: it is the oracle of the multi-process CPU tests and the
NCCL baseline that the fused layer (:mod:`ep_balance_b200.models.moe_layer`) is measured against.
Pipeline per call (reference: eplb/integration/eplb_manager.py:905-1167):

    plan tables -> unit -> (physical slot, dst) -> sort by dst -> all-to-all dispatch (rows + slot ids)
    -> replica weights from their owners -> grouped expert MLP -> all-to-all combine -> un-sort
    -> gate-weighted index_add.

Two concerns stay separate, as in the reference: the *token transport* sits behind a
:class:`CommAdapter`; *replication* (weights out from ``main(e)``, gradients back) sits behind a
:class:`ReplicaTransport`.  Differences from the reference's implementation: slot ids travel as their
own int64 all-to-all instead of a float column glued to the payload, and the "weights are not held
across forward->backward" modes re-acquire the weights and re-run the expert function under autograd
instead of hand-writing the two-GEMM backward.
"""

from __future__ import annotations

import os
from typing import Callable, Dict, List, Optional, Protocol, Sequence, Tuple

import torch
import torch.distributed as dist
from torch.utils.checkpoint import checkpoint

from ..core.plan import Plan
from ..core.problem import ProblemSpec
from ..utils import profiling
from .comm import a2a_raw, all_to_all_single, broadcast_from_main, global_rank
from .grouped_mlp import grouped_expert_mlp
from .overlap import (BackwardKick, LeasedExperts, WeightLease, forked, side_stream, side_streams_enabled,
                      weight_channel)
from .physical import assign_physical
from .symm_weights import SymmReplicaTransport, replicator_for, symm_weights_enabled


def _env_truthy(name: str, default: str = "0") -> bool:
    return os.environ.get(name, default).strip().lower() not in ("0", "", "false", "no")


# ====================================================================== tables derived from the plan (reference: eplb_manager.py:482-536)
def split_sizes(plan: Plan, my_rank: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(sent_per_dst[R], recv_per_src[R], recv_per_expert[E])`` for this rank, on the plan's device."""
    q = plan.q.to(torch.int64)
    return q[my_rank].sum(0), q[:, :, my_rank].sum(1), q[:, :, my_rank].sum(0)


def slot_tables(x: torch.Tensor, my_rank: int, n_slot: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(slot_to_e[n_slot] (-1 empty), slot_of_e[E], hosted[E])``; local slots in ascending expert id."""
    col = x[:, my_rank].to(torch.int64)
    hosted = col.bool()
    slot_of_e = (col.cumsum(0) - 1).clamp_(min=0)
    ids = torch.arange(col.numel(), device=x.device, dtype=torch.int64)
    target = torch.where(hosted, slot_of_e, torch.full_like(slot_of_e, int(n_slot)))
    ext = torch.full((int(n_slot) + 1,), -1, dtype=torch.int64, device=x.device).scatter_(0, target, ids)
    return ext[: int(n_slot)].clone(), slot_of_e, hosted


def group_sizes_by_slot(slot_to_e: torch.Tensor, recv_per_expert: torch.Tensor) -> torch.Tensor:
    picked = recv_per_expert[slot_to_e.clamp(min=0)]
    return torch.where(slot_to_e >= 0, picked, torch.zeros_like(picked))


# ====================================================================== token transport
class CommAdapter(Protocol):
    def dispatch_chunk(self, payload, sent_per_dst, recv_per_src, group, *, tag: int = 0): ...

    def combine_chunk(self, payload, sent_per_dst, recv_per_src, group, *, tag: int = 0): ...

    def uses_padded_layout(self) -> bool: ...


class AllToAllAdapter:
    """``all_to_all_single`` with split sizes read to the host once per chunk (the only D2H here)."""

    def __init__(self) -> None:
        self._splits: Dict[int, Tuple[List[int], List[int]]] = {}

    def uses_padded_layout(self) -> bool:
        return False

    def host_splits(self, sent_per_dst, recv_per_src, tag: int) -> Tuple[List[int], List[int]]:
        flat = torch.cat([sent_per_dst, recv_per_src]).tolist()
        n = sent_per_dst.numel()
        self._splits[tag] = (flat[:n], flat[n:])
        return self._splits[tag]

    def dispatch_chunk(self, payload, sent_per_dst, recv_per_src, group, *, tag: int = 0):
        send, recv = self.host_splits(sent_per_dst, recv_per_src, tag)
        return all_to_all_single(payload, recv, send, group)

    def dispatch_ids(self, ids: torch.Tensor, group, *, tag: int = 0) -> torch.Tensor:
        send, recv = self._splits[tag]
        return a2a_raw(ids, recv, send, group)

    def combine_chunk(self, payload, sent_per_dst, recv_per_src, group, *, tag: int = 0):
        send, recv = self._splits[tag]
        return all_to_all_single(payload, send, recv, group)

    def chunk_state(self, tag: int):
        return self._splits.pop(tag, None)


class PaddedAllToAllAdapter:
    """Zero-sync token transport on library collectives: every (source, destination) pair exchanges a block of
    ``rows_per_pair`` rows, so every split size is a host constant and nothing is read back from the device.

    The price is padding: ``R * rows_per_pair`` rows travel and are computed on, whatever the routing.  Rows of
    a pair beyond the block are dropped and recorded in the row-budget status word (site 21), like every other
    row budget of the portable path.  This is the contract the reference's DeepEP adapter fulfils with its
    fixed-size buffers (eplb_manager.py ``CommAdapter.uses_padded_layout``; tests/test_sync_free.py:485-606 pin it
    with a fake backend): received rows come as ``R`` aligned blocks with a validity mask instead of a ragged list.
    """

    ALIGN = 8  # rows per block are rounded up so that every block starts on a 16-byte multiple for any dtype

    def __init__(self, rows_per_pair: int) -> None:
        if int(rows_per_pair) <= 0:
            raise ValueError("rows_per_pair must be positive")
        self.cap = -(-int(rows_per_pair) // self.ALIGN) * self.ALIGN
        self._state: Dict[int, dict] = {}

    def uses_padded_layout(self) -> bool:
        return True

    def _splits(self, world: int) -> List[int]:
        return [self.cap] * world

    def dispatch_chunk(self, payload, sent_per_dst, recv_per_src, group, *, tag: int = 0):
        from .grouped_mlp import _record_overflow

        R, cap, n = int(sent_per_dst.numel()), self.cap, int(payload.shape[0])
        ends = sent_per_dst.cumsum(0)
        rows = torch.arange(n, device=payload.device)
        dst = torch.searchsorted(ends, rows, right=True).clamp_(max=R - 1)      # payload is sorted by destination
        pos = rows - (ends - sent_per_dst)[dst]
        keep = pos < cap
        flat = torch.where(keep, dst * cap + pos, torch.full_like(pos, R * cap))  # overflow rows go to a spare row
        _record_overflow(sent_per_dst.max(), cap, site=21)
        block = payload.new_zeros((R * cap + 1,) + tuple(payload.shape[1:])).index_copy(0, flat, payload)[:-1]
        valid = (torch.arange(cap, device=payload.device)[None, :] < recv_per_src.clamp(max=cap)[:, None]).reshape(-1)
        self._state[tag] = {"flat": flat, "keep": keep, "valid": valid, "R": R}
        if R == 1 and not (dist.is_available() and dist.is_initialized()):
            return block
        return all_to_all_single(block, self._splits(R), self._splits(R), group)

    def dispatch_ids(self, ids: torch.Tensor, group, *, tag: int = 0) -> torch.Tensor:
        st = self._state[tag]
        R, cap = st["R"], self.cap
        block = ids.new_zeros(R * cap + 1).index_copy(0, st["flat"], ids)[:-1]
        if R == 1 and not (dist.is_available() and dist.is_initialized()):
            return block
        return a2a_raw(block, self._splits(R), self._splits(R), group)

    def valid_mask(self, tag: int = 0) -> torch.Tensor:
        """Which of the ``R * cap`` received rows are real (block of source s holds ``recv_per_src[s]`` of them)."""
        return self._state[tag]["valid"]

    def combine_chunk(self, payload, sent_per_dst, recv_per_src, group, *, tag: int = 0):
        st = self._state[tag]
        R = st["R"]
        back = payload if (R == 1 and not (dist.is_available() and dist.is_initialized())) else \
            all_to_all_single(payload, self._splits(R), self._splits(R), group)
        back = torch.cat([back, back.new_zeros((1,) + tuple(back.shape[1:]))])          # the spare row reads as zeros
        return back.index_select(0, st["flat"])

    def chunk_state(self, tag: int):
        return self._state.pop(tag, None)


class LocalAdapter(AllToAllAdapter):
    """World of one process without a process group: the all-to-all is the identity."""

    def dispatch_chunk(self, payload, sent_per_dst, recv_per_src, group, *, tag: int = 0):
        self._splits[tag] = ([payload.shape[0]], [payload.shape[0]])
        return payload

    def dispatch_ids(self, ids, group, *, tag: int = 0):
        return ids

    def combine_chunk(self, payload, sent_per_dst, recv_per_src, group, *, tag: int = 0):
        return payload


# ====================================================================== replication
class ReplicaTransport(Protocol):
    """Brings replica weights onto this rank and returns their gradients to the owners."""

    def materialize(self) -> Tuple[torch.Tensor, ...]: ...


class BroadcastReplicaTransport:
    """One ``dist.broadcast`` per replicated expert and weight tensor; backward is ``dist.reduce`` to
    the owner (reference: eplb/integration/overlap.py:113-232, comm.py:65-113)."""

    def __init__(self, *, plan: Plan, spec: ProblemSpec, weights_local, weight_shapes, my_rank: int, n_slot: int,
                 dtype, device, group) -> None:
        self.plan, self.spec = plan, spec
        self.weights_local, self.weight_shapes = weights_local, [tuple(s) for s in weight_shapes]
        self.my_rank, self.n_slot, self.dtype, self.device, self.group = my_rank, n_slot, dtype, device, group
        # Control plane: which experts are replicated and who owns them.  dist.broadcast needs host
        # integers, so this is one consolidated device->host read of ~E numbers per call.
        rep = (plan.num_replicas() > 1).nonzero(as_tuple=False).flatten()
        flat = torch.cat([rep, spec.main_rank.index_select(0, rep).to(torch.int64)]).tolist()
        self.replicated, self.replicated_main = flat[: len(flat) // 2], flat[len(flat) // 2:]
        _, self.slot_of_e, self.hosted = slot_tables(plan.x, my_rank, n_slot)
        self._slot_of_e, self._hosted = self.slot_of_e.tolist(), self.hosted.tolist()

    def materialize(self, rows: Sequence[torch.Tensor] = ()):
        """Stacked ``[n_slot, *shape]`` weights, differentiable w.r.t. the owners' parameters.

        ``rows`` (the received token rows of every chunk) are passed through unchanged.  Routing them
        through the same autograd node makes the gradient reductions of this node run strictly
        before the reverse token all-to-alls on every rank; without that dependency the autograd
        engine may order the two kinds of collectives differently on different ranks (which matters
        when both use one communicator).
        Returns ``stacks`` when ``rows`` is empty, else ``(rows_out, stacks)``.
        """
        out = _MaterializeStacks.apply(self, len(rows), *rows, *_owner_params(self))
        if not rows:
            return tuple(out)
        return tuple(out[: len(rows)]), tuple(out[len(rows):])

    # ---- the two halves without autograd (used by the node above and by a WeightLease)
    def acquire(self, owner_params: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
        """Owned experts are copied into their slots; every replicated expert is broadcast from its owner
        in a fixed order (expert id, then weight index) in which every rank takes part."""
        params = list(owner_params) if owner_params is not None else _owner_params(self)
        n_w = len(self.weight_shapes)
        owned = sorted(self.weights_local)
        slot_of_e, hosted = self._slot_of_e, self._hosted
        stacks = [torch.zeros((self.n_slot,) + self.weight_shapes[j], dtype=self.dtype, device=self.device)
                  for j in range(n_w)]
        for i, e in enumerate(owned):
            if hosted[e]:
                for j in range(n_w):
                    stacks[j][slot_of_e[e]] = params[i * n_w + j].detach().to(self.dtype)
        with profiling.record("apply/weight_move", time_it=True, device=self.device):
            for e, owner in zip(self.replicated, self.replicated_main):
                root = global_rank(self.group, owner)
                for j in range(n_w):
                    if owner == self.my_rank:
                        buf = params[owned.index(e) * n_w + j].detach().to(self.dtype).contiguous().clone()
                    else:
                        buf = torch.empty(self.weight_shapes[j], dtype=self.dtype, device=self.device)
                    if dist.is_available() and dist.is_initialized():
                        dist.broadcast(buf, src=root, group=self.group)
                    if hosted[e] and owner != self.my_rank:
                        stacks[j][slot_of_e[e]] = buf
        return stacks

    def give_back(self, grad_stacks: Sequence[Optional[torch.Tensor]]) -> List[torch.Tensor]:
        """One gradient per owned expert and weight tensor (``sorted(weights_local)`` order): the owner's
        own slot plus, for replicated experts, a ``dist.reduce`` over every rank in the same fixed order."""
        n_w = len(self.weight_shapes)
        owned = sorted(self.weights_local)
        slot_of_e, hosted = self._slot_of_e, self._hosted
        grads: Dict[Tuple[int, int], torch.Tensor] = {}
        for e in owned:  # the owner's own instance
            for j in range(n_w):
                g = grad_stacks[j]
                grads[(e, j)] = (g[slot_of_e[e]].clone(memory_format=torch.contiguous_format) if g is not None and hosted[e]
                                 else torch.zeros(self.weight_shapes[j], dtype=self.dtype, device=self.device))
        with profiling.record("apply/grad_move", time_it=True, device=self.device):
            for e, owner in zip(self.replicated, self.replicated_main):
                root = global_rank(self.group, owner)
                for j in range(n_w):
                    g = grad_stacks[j]
                    if owner == self.my_rank:
                        buf = grads[(e, j)]
                    elif hosted[e] and g is not None:
                        buf = g[slot_of_e[e]].clone(memory_format=torch.contiguous_format)
                    else:
                        buf = torch.zeros(self.weight_shapes[j], dtype=self.dtype, device=self.device)
                    reduce_to_root(buf, root, self.group)
                    if owner == self.my_rank:
                        grads[(e, j)] = buf
        return [grads[(e, j)] for e in owned for j in range(n_w)]


def reduce_to_root(buf: torch.Tensor, root: int, group) -> None:
    """Sum ``buf`` over the group into ``root`` (in place there).  ``buf`` must be contiguous:
    collectives address the storage as a flat array, so a transposed gradient slice (which
    ``Tensor.clone()`` keeps transposed) would be summed with the wrong element order."""
    if not (dist.is_available() and dist.is_initialized()):
        return
    if not buf.is_contiguous():
        raise ValueError("reduce_to_root needs a contiguous buffer")
    dist.reduce(buf, dst=root, op=dist.ReduceOp.SUM, group=group)


class _MaterializeStacks(torch.autograd.Function):
    """All replica broadcasts of a layer in ONE autograd node.

    Forward issues the broadcasts in a fixed order (expert id, then weight index) and every rank
    takes part in each of them; backward issues the matching ``dist.reduce`` calls in the same fixed
    order.  Keeping the collectives inside one node makes their order independent of how the
    autograd engine schedules the rest of the graph, which differs between ranks that host a
    replica and ranks that do not.
    """

    @staticmethod
    def forward(ctx, tr: "BroadcastReplicaTransport", n_rows: int, *tensors):
        rows, owner_params = tensors[:n_rows], tensors[n_rows:]
        ctx.n_rows, ctx.tr = n_rows, tr
        stacks = tr.acquire(owner_params)
        return (*[r.view_as(r) for r in rows], *stacks)

    @staticmethod
    def backward(ctx, *grad_all):
        grad_rows, grad_stacks = grad_all[: ctx.n_rows], grad_all[ctx.n_rows:]
        return (None, None, *grad_rows, *ctx.tr.give_back(grad_stacks))


def _owner_params(transport) -> List[torch.Tensor]:
    return [w for e in sorted(transport.weights_local) for w in transport.weights_local[e]]


# ====================================================================== public forward
def sync_free_moe_forward(tokens: torch.Tensor, unit_token_idx: torch.Tensor, unit_expert: torch.Tensor,
                          unit_prob: torch.Tensor, plan: Plan, spec: ProblemSpec,
                          weights_local: Dict[int, Tuple[torch.Tensor, ...]], weight_shapes: Sequence[torch.Size],
                          batched_mlp_fn: Callable, cap: Optional[int] = None,
                          grouped_mlp_fn: Optional[Callable] = None, max_recv_rows: Optional[int] = None,
                          group=None, adapter: Optional[CommAdapter] = None, rematerialize: bool = False,
                          overlap: bool = False, gated: bool = False, act: Callable = torch.relu,
                          transpose_w: bool = False, num_chunks: Optional[int] = None) -> torch.Tensor:
    """MoE output ``[Ntok, H]`` for this rank's tokens under ``plan`` (see module docstring).

    ``weights_local`` maps each expert owned by this rank to its parameter tuple.  ``rematerialize``
    checkpoints replication + compute; ``overlap`` holds no replica between forward and backward: one
    :class:`~ep_balance_b200.parallel.overlap.WeightLease` per call, re-started by the first backward node.  ``num_chunks``
    (default: ``EPLB_CHUNKS``) splits the units into that many dispatch/compute/combine rounds that
    share one weight acquisition.  ``gated``/``act``/``transpose_w`` are accepted for signature
    compatibility; the expert math is whatever ``batched_mlp_fn``/``grouped_mlp_fn`` compute.
    """
    distributed = dist.is_available() and dist.is_initialized()
    my_rank = dist.get_rank(group) if distributed else 0
    adapter = adapter or (AllToAllAdapter() if distributed else LocalAdapter())
    if not distributed and not isinstance(adapter, (LocalAdapter, PaddedAllToAllAdapter)):
        adapter = LocalAdapter()  # no process group: every transport degenerates to the identity
    device, dtype = tokens.device, tokens.dtype
    n_slot = int(spec.n_slot)
    chunks = int(num_chunks if num_chunks is not None else (os.environ.get("EPLB_CHUNKS", "1") or "1"))
    # three lanes on CUDA: this stream computes, ``comm`` carries the token all-to-alls, ``weight`` (with a
    # communicator of its own) carries the replica weights and their gradients
    lanes = side_streams_enabled(device)
    comm_lane = side_stream(device, "comm") if lanes else None
    weight_lane = side_stream(device, "weight") if lanes else None

    _, _, recv_per_expert = split_sizes(plan, my_rank)
    slot_to_e, _, _ = slot_tables(plan.x, my_rank, n_slot)
    group_sizes = group_sizes_by_slot(slot_to_e, recv_per_expert)
    if cap is None and os.environ.get("EPLB_CAP"):
        cap = int(os.environ["EPLB_CAP"])
    ragged = grouped_mlp_fn is not None
    if cap is None and not ragged:
        cap = max(int(group_sizes.max()), 1)  # padded path only: one host read

    if distributed and device.type == "cuda" and symm_weights_enabled():
        # device-initiated weight channel: one-sided gets/puts over the symmetric heap
        rep = replicator_for(group, spec.main_rank, weight_shapes, dtype, device)
        transport = SymmReplicaTransport(rep, plan.x, n_slot, weights_local)
    else:
        transport = BroadcastReplicaTransport(plan=plan, spec=spec, weights_local=weights_local,
                                              weight_shapes=weight_shapes, my_rank=my_rank, n_slot=n_slot,
                                              dtype=dtype, device=device, group=weight_channel(group, device)) \
            if distributed or weights_local else None

    with profiling.record("apply/route", time_it=True, device=device):
        phys_id, dst_rank = assign_physical(unit_expert, plan, spec, my_rank)

    U = int(unit_expert.shape[0])
    n_chunks = max(chunks, 1)
    bounds = [U * k // n_chunks for k in range(n_chunks + 1)]
    R = int(plan.q.shape[0])

    # ---- weights first: the acquisition is enqueued before any token traffic and joined before the first GEMM
    lease = stacks = None
    join_weights = lambda: None  # noqa: E731
    if overlap:
        lease = WeightLease(transport, n_chunks, device)
        lease.start()
    elif not rematerialize and lanes:
        with forked(weight_lane) as join:
            stacks = transport.materialize()
        join_weights = join[0]

    # ---- all dispatches next (their reverse legs then run last in backward, after the reductions)
    sent_l, recv_l, perm_l, rows_l, slot_l, valid_l, arrived = [], [], [], [], [], [], []
    for k in range(n_chunks):
        lo, hi = bounds[k], bounds[k + 1]
        c_dst, c_phys = dst_rank[lo:hi], phys_id[lo:hi]
        perm = torch.argsort(c_dst, stable=True)
        sent = torch.zeros(R, dtype=torch.int64, device=device).scatter_add_(0, c_dst, torch.ones_like(c_dst))
        payload = tokens[unit_token_idx[lo:hi]][perm]
        ids = c_phys[perm].contiguous()
        with forked(comm_lane) as join:
            if distributed:
                recv = torch.empty_like(sent)
                dist.all_to_all_single(recv, sent, group=group)
            else:
                recv = sent
            # bytes this rank puts on the wire for the chunk (rows + ids); shows as MiB and GB/s in the debug line
            with profiling.record("apply/dispatch", time_it=True, device=device,
                                  payload_bytes=payload.numel() * payload.element_size() + ids.numel() * ids.element_size()):
                rows = adapter.dispatch_chunk(payload, sent, recv, group, tag=k)
                recv_phys = adapter.dispatch_ids(ids, group, tag=k)
            # still on the comm lane: the received ids may be read only after their all-to-all
            recv_slot = recv_phys - my_rank * n_slot
            valid = adapter.valid_mask(k) if adapter.uses_padded_layout() else None
            if valid is not None:
                recv_slot = torch.where(valid, recv_slot, torch.zeros_like(recv_slot))
        _shared_between(comm_lane, device, payload, ids, sent, recv, rows, recv_phys, recv_slot, valid)
        valid_l.append(valid)
        arrived.append(join[0])
        sent_l.append(sent)
        recv_l.append(recv)
        perm_l.append(perm)
        rows_l.append(rows)
        slot_l.append(recv_slot)

    def compute_chunk(k: int):
        ones = torch.ones_like(slot_l[k]) if valid_l[k] is None else valid_l[k].to(slot_l[k].dtype)
        sizes = torch.zeros(n_slot, dtype=torch.int64, device=device).scatter_add_(0, slot_l[k], ones)

        def compute(x, stacks):
            return grouped_expert_mlp(x, slot_l[k], sizes, stacks, batched_mlp_fn, cap=cap, valid_mask=valid_l[k],
                                      grouped_mlp_fn=grouped_mlp_fn, max_recv_rows=max_recv_rows)

        return compute

    if not lanes:
        if not overlap and not rematerialize:
            # one communicator, one stream: the rows pass through the weight node to pin the backward order
            rows_l, stacks = transport.materialize(rows_l)
            rows_l = list(rows_l)
    else:
        for k in range(n_chunks):
            arrived[k]()            # nothing received on the comm lane was touched on this stream before this point
    if stacks is not None:
        join_weights()
        _shared_between(weight_lane, device, *stacks)

    # ---- per chunk: GEMMs here, the combine on the comm lane (so that it runs under the next chunk's GEMMs)
    backs, combined = [], []
    for k in range(n_chunks):
        compute = compute_chunk(k)
        with profiling.record("apply/expert_compute", time_it=True, device=device):
            if overlap:
                y = LeasedExperts.apply(rows_l[k], lease, compute, *_owner_params(transport))
            elif rematerialize:
                y = checkpoint(lambda x, c=compute: c(x, transport.materialize()), rows_l[k], use_reentrant=False,
                               preserve_rng_state=False)
            else:
                y = compute(rows_l[k], stacks)
        with forked(comm_lane) as join:
            with profiling.record("apply/combine", time_it=True, device=device,
                                  payload_bytes=y.numel() * y.element_size()):
                back = adapter.combine_chunk(y, sent_l[k], recv_l[k], group, tag=k)
        _shared_between(comm_lane, device, y, back)
        adapter.chunk_state(k)
        backs.append(back)
        combined.append(join[0])

    result = torch.zeros((tokens.shape[0], tokens.shape[1]), dtype=dtype, device=device)
    for k in range(n_chunks):
        lo, hi = bounds[k], bounds[k + 1]
        combined[k]()
        per_unit = backs[k][torch.argsort(perm_l[k])]
        result = result.index_add(0, unit_token_idx[lo:hi], unit_prob[lo:hi].unsqueeze(1).to(dtype) * per_unit)
    if lease is not None:
        result = BackwardKick.apply(result, lease)
    return result


def _shared_between(lane, device, *tensors) -> None:
    """Tensors that cross between this stream and ``lane``: tell the caching allocator about both users."""
    if lane is None:
        return
    here = torch.cuda.current_stream(device)
    for t in tensors:
        if isinstance(t, torch.Tensor) and t.is_cuda:
            t.record_stream(lane)
            t.record_stream(here)
