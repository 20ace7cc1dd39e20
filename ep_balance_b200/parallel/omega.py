"""Collecting the load matrix: one row per expert-parallel rank.

The library path (:func:`all_gather_omega`) is a plain ``all_gather_into_tensor`` and works on
NCCL and gloo (reference: eplb/distributed.py:17-61).  The fused MoE layer does not use it: there
each rank's row is stored straight into every peer's symmetric buffer by
``ops/csrc/route.cu::publish_counts_kernel`` and consumed by the solver kernel.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..core.loads import Loads


def is_distributed() -> bool:
    return dist.is_available() and dist.is_initialized()


def all_gather_omega(local_row: torch.Tensor, group: Optional["dist.ProcessGroup"] = None) -> Loads:
    row = local_row.to(torch.int64).contiguous()
    if not is_distributed():
        return Loads(row[None])
    world = dist.get_world_size(group)
    out = row.new_empty(world * row.numel())  # flat: the layout every backend accepts
    dist.all_gather_into_tensor(out, row, group=group)
    return Loads(out.view(world, row.numel()))


def local_counts_from_routing(expert_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Histogram of routed expert ids with a fixed output size (no data-dependent shape)."""
    out = torch.zeros(int(num_experts), dtype=torch.int64, device=expert_ids.device)
    flat = expert_ids.reshape(-1).to(torch.int64)
    return out.scatter_add_(0, flat, torch.ones_like(flat))
