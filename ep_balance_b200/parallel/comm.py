"""Differentiable collectives for the library (NCCL/gloo) MoE path.

These back the portable implementation in :mod:`ep_balance_b200.parallel.library_path`, which is
the correctness oracle on CPU ranks and the NCCL baseline on GPUs.  Reference:
eplb/integration/comm.py:11-113.
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def global_rank(group, local_rank: int) -> int:
    return int(local_rank) if group is None else int(dist.get_global_rank(group, int(local_rank)))


def a2a_raw(inp: torch.Tensor, out_splits: List[int], in_splits: List[int], group=None) -> torch.Tensor:
    """All-to-all of rows without an autograd node (caller schedules the transposed leg itself)."""
    out = inp.new_empty((int(sum(out_splits)),) + tuple(inp.shape[1:]))
    dist.all_to_all_single(out, inp.contiguous(), list(out_splits), list(in_splits), group=group)
    return out


class _A2A(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, out_splits, in_splits, group):
        ctx.meta = (list(out_splits), list(in_splits), group)
        return a2a_raw(inp, out_splits, in_splits, group)

    @staticmethod
    def backward(ctx, grad):
        out_splits, in_splits, group = ctx.meta
        return a2a_raw(grad, in_splits, out_splits, group), None, None, None


def all_to_all_single(inp, out_splits, in_splits, group=None):
    """Row all-to-all whose backward is the transposed all-to-all."""
    return _A2A.apply(inp, out_splits, in_splits, group)


class _Bcast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, root, group):
        ctx.meta = (root, group)
        out = tensor.detach().clone()
        dist.broadcast(out, src=root, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        root, group = ctx.meta
        g = grad.detach().clone(memory_format=torch.contiguous_format)
        dist.reduce(g, dst=root, op=dist.ReduceOp.SUM, group=group)
        return g, None, None


def broadcast_from_main(weight: Optional[torch.Tensor], shape, dtype, device, main_local_rank: int,
                        group=None) -> torch.Tensor:
    """Value of an expert weight on every rank; backward sums all ranks' grads into the owner.

    Non-owners pass ``weight=None``; their placeholder's gradient is meaningless and dropped.
    """
    root = global_rank(group, main_local_rank)
    me = dist.get_rank() if group is None else global_rank(group, dist.get_rank(group))
    src = weight if me == root else torch.zeros(tuple(shape), dtype=dtype, device=device, requires_grad=True)
    return _Bcast.apply(src, root, group)
