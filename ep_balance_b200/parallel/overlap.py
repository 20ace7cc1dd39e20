"""Side channels of the portable apply path: replica weights move beside the token traffic.

The portable path (:mod:`ep_balance_b200.parallel.library_path`) has three kinds of work per layer call:
token all-to-alls, expert GEMMs, and the replica weight traffic (weights out from their owners, gradients
back).  Run on one stream and one communicator they queue behind one another.  This module gives the
weight traffic its own lane:

* :func:`weight_channel` -- a second communicator over the same ranks (NCCL keeps one stream per
  communicator, so collectives of the two run side by side) and :func:`side_stream`, a per-device CUDA
  stream on which the weight collectives are enqueued.  On CPU both collapse to the caller's group and
  "no stream": the code path is the same, only nothing runs concurrently.
* :class:`WeightLease` -- ONE acquisition of a layer call's replica stacks, started before the token
  dispatches are enqueued, shared by every chunk of the call, and dropped after the last chunk's
  forward so that no replica stays alive between forward and backward.  In backward the lease is
  started again (:class:`BackwardKick`, the first node of the layer's backward, so that the re-pull
  runs under the reverse combine), every chunk replays its expert function on the leased stacks, the
  weight gradients of all chunks are summed locally and returned to the owners ONCE.
* :func:`forked` -- context manager that runs a block on a side stream after everything the caller has
  enqueued so far, and hands back a join callable.

Reference: eplb/integration/overlap.py:57-110 (pool, side streams), :257-328 (lease, prefetch on
backward), eplb/integration/manual_block.py:127-367 (issue order).  The design here differs: a separate
communicator instead of stream juggling on one, a lease that also owns the gradient accumulation, and
autograd's own stream bookkeeping for the held-weights mode (a node runs its backward on the stream its
forward ran on).
"""

from __future__ import annotations

import contextlib
import os
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

_STREAMS: Dict[Tuple[int, str], "torch.cuda.Stream"] = {}
_CHANNELS: Dict[int, object] = {}


def side_streams_enabled(device) -> bool:
    """``EPLB_SIDE_STREAMS`` (default on) and a CUDA device."""
    if torch.device(device).type != "cuda":
        return False
    return os.environ.get("EPLB_SIDE_STREAMS", "1").strip().lower() not in ("0", "", "false", "no")


def side_stream(device, name: str = "weight") -> Optional["torch.cuda.Stream"]:
    """The process-wide side stream ``name`` of ``device`` (``None`` off CUDA)."""
    device = torch.device(device)
    if device.type != "cuda":
        return None
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, name)
    if key not in _STREAMS:
        _STREAMS[key] = torch.cuda.Stream(device=index)
    return _STREAMS[key]


def weight_channel(group, device):
    """Communicator for the replica weight traffic.  On CUDA with side streams on: a second process group
    over the ranks of ``group``, created collectively on first use (every rank of ``group`` must reach
    this call, which holds for a layer call that all ranks make together).  Otherwise ``group`` itself."""
    if not (dist.is_available() and dist.is_initialized()) or not side_streams_enabled(device):
        return group
    key = id(group) if group is not None else 0
    if key not in _CHANNELS:
        ranks = dist.get_process_group_ranks(group if group is not None else dist.group.WORLD)
        _CHANNELS[key] = dist.new_group(ranks=ranks)
    return _CHANNELS[key]


def close_channels() -> None:
    _CHANNELS.clear()
    _STREAMS.clear()


@contextlib.contextmanager
def forked(stream: Optional["torch.cuda.Stream"]):
    """Run the block on ``stream`` once the caller's stream has reached this point.  Yields a list that
    receives one callable, ``join()``: the caller's stream waits for the block."""
    if stream is None:
        yield [lambda: None]
        return
    stream.wait_stream(torch.cuda.current_stream(stream.device))
    done = torch.cuda.Event()
    with torch.cuda.stream(stream):
        holder: List[Callable[[], None]] = [lambda: torch.cuda.current_stream(stream.device).wait_event(done)]
        yield holder
        done.record(stream)


def _keep_alive_on(tensors: Sequence[torch.Tensor], stream) -> None:
    if stream is None:
        return
    for t in tensors:
        if t is not None and t.is_cuda:
            t.record_stream(stream)


class WeightLease:
    """One acquisition of the replica stacks per pass, shared by ``consumers`` chunks.

    ``transport`` needs two calls without autograd: ``acquire() -> list of [n_slot, ...] stacks`` (every
    rank takes part) and ``give_back(grad_stacks) -> [gradient per owned expert and weight tensor]``.
    """

    def __init__(self, transport, consumers: int, device) -> None:
        self.transport, self.consumers, self.device = transport, int(consumers), torch.device(device)
        self.stream = side_stream(device, "weight") if side_streams_enabled(device) else None
        self._stacks: Optional[List[torch.Tensor]] = None
        self._join: Callable[[], None] = lambda: None
        self._left = 0
        self._grad_sum: Optional[List[Optional[torch.Tensor]]] = None
        self.acquisitions = 0               # how many times the stacks were brought over (tests read this)
        self.returns = 0

    # ---- acquisition
    def start(self) -> None:
        """Enqueue the acquisition (on the weight stream when there is one); returns at once."""
        if self._stacks is not None:
            return
        with forked(self.stream) as join, torch.no_grad():
            self._stacks = list(self.transport.acquire())
        self._join = join[0]
        self._left = self.consumers
        self._grad_sum = None
        self.acquisitions += 1

    def stacks(self) -> List[torch.Tensor]:
        """The leased stacks, ordered after the acquisition on the caller's stream."""
        if self._stacks is None:
            self.start()
        self._join()
        self._join = lambda: None
        if self.stream is not None:
            _keep_alive_on(self._stacks, torch.cuda.current_stream(self.device))
        return self._stacks

    def consumer_done(self) -> None:
        """A forward consumer is finished; the last one drops the stacks."""
        self._left -= 1
        if self._left <= 0:
            self._stacks = None

    # ---- gradient return
    def return_grads(self, grad_stacks: Sequence[Optional[torch.Tensor]]) -> Optional[List[torch.Tensor]]:
        """Add one chunk's stack gradients.  The last chunk returns the owners' gradients (one reduction
        per layer call); the others return ``None``."""
        if self._grad_sum is None:
            self._grad_sum = [None if g is None else g.clone() for g in grad_stacks]
        else:
            for j, g in enumerate(grad_stacks):
                if g is None:
                    continue
                self._grad_sum[j] = g.clone() if self._grad_sum[j] is None else self._grad_sum[j].add_(g)
        self._left -= 1
        if self._left > 0:
            return None
        total, self._grad_sum, self._stacks = self._grad_sum, None, None
        self.returns += 1
        with torch.no_grad():
            return list(self.transport.give_back(total))


class BackwardKick(torch.autograd.Function):
    """Identity on the layer's output.  It is the last node of the forward graph, so its backward runs
    first: it starts the lease's re-acquisition, which then proceeds under the reverse combine."""

    @staticmethod
    def forward(ctx, out: torch.Tensor, lease: WeightLease) -> torch.Tensor:
        ctx.lease = lease
        return out.view_as(out)

    @staticmethod
    def backward(ctx, grad_out):
        ctx.lease.start()
        return grad_out, None


class LeasedExperts(torch.autograd.Function):
    """Expert compute of one chunk on leased stacks.  Forward keeps only the received rows; backward
    replays ``compute`` on the re-acquired stacks and hands the weight gradients to the lease."""

    @staticmethod
    def forward(ctx, rows: torch.Tensor, lease: WeightLease, compute: Callable, *owner_params):
        with torch.no_grad():
            out = compute(rows, tuple(lease.stacks()))
        lease.consumer_done()
        ctx.lease, ctx.compute, ctx.n_params = lease, compute, len(owner_params)
        ctx.save_for_backward(rows)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (rows,) = ctx.saved_tensors
        lease = ctx.lease
        stacks = [s.detach().requires_grad_(True) for s in lease.stacks()]
        with torch.enable_grad():
            x = rows.detach().requires_grad_(True)
            out = ctx.compute(x, tuple(stacks))
            grads = torch.autograd.grad(out, [x] + stacks, grad_out, allow_unused=True)
        owner = lease.return_grads(grads[1:])
        if owner is None:
            owner = [None] * ctx.n_params
        return (grads[0], None, None, *owner)
