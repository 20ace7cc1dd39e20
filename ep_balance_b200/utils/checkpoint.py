"""Checkpoint / resume for expert-parallel training.

Layout of one checkpoint (a directory ``<root>/iter_<step>``):

    replicated.pt        state that is identical on every rank (dense parameters, their optimizer
                         state, step counter, RNG/skew state) -- written by rank 0 only
    experts_rank<r>.pt   state owned by rank r: its own experts' parameters (the ``main(e)`` copies)
                         and their optimizer state
    <root>/latest        text file naming the newest complete step

Replica weights are transient and carry no optimizer state, so they are never saved: a checkpoint
holds exactly the owners' copies (as in the reference, where Megatron saves ``main(e)`` weights only;
eval/plot_gin_replica_transport.py:213-230).  Every file is written to a temporary name and moved
into place with ``os.replace``; ``latest`` is updated last, after a barrier, so a crash in the middle
of a save leaves the previous checkpoint as the newest complete one.
"""

from __future__ import annotations

import os
from typing import Any, Dict, Optional, Tuple

import torch
import torch.distributed as dist


def _atomic_save(obj: Any, path: str) -> None:
    tmp = f"{path}.tmp.{os.getpid()}"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def _barrier(group=None) -> None:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.barrier(group=group)


def step_dir(root: str, step: int) -> str:
    return os.path.join(root, f"iter_{int(step):07d}")


def save_checkpoint(root: str, step: int, *, replicated: Dict[str, Any], sharded: Dict[str, Any], rank: int = 0,
                    world: int = 1, group=None) -> str:
    """Write one checkpoint; returns its directory.  Collective over ``group``."""
    d = step_dir(root, step)
    os.makedirs(d, exist_ok=True)
    if rank == 0:
        _atomic_save({"step": int(step), "world": int(world), "state": replicated}, os.path.join(d, "replicated.pt"))
    _atomic_save({"step": int(step), "rank": int(rank), "world": int(world), "state": sharded},
                 os.path.join(d, f"experts_rank{int(rank)}.pt"))
    _barrier(group)
    if rank == 0:
        tmp = os.path.join(root, f"latest.tmp.{os.getpid()}")
        with open(tmp, "w") as f:
            f.write(str(int(step)))
        os.replace(tmp, os.path.join(root, "latest"))
    _barrier(group)
    return d


def latest_step(root: str) -> Optional[int]:
    try:
        with open(os.path.join(root, "latest")) as f:
            return int(f.read().strip())
    except (OSError, ValueError):
        return None


def load_checkpoint(root: str, *, step: Optional[int] = None, rank: int = 0, world: int = 1,
                    map_location="cpu") -> Tuple[int, Dict[str, Any], Dict[str, Any]]:
    """Returns ``(step, replicated, sharded)`` of the requested (default: newest complete) checkpoint.

    The expert-parallel world size must match the one that wrote the checkpoint: expert ownership
    ``main(e)`` is immutable, so the shards cannot be re-split here.
    """
    if step is None:
        step = latest_step(root)
        if step is None:
            raise FileNotFoundError(f"no complete checkpoint under {root!r}")
    d = step_dir(root, step)
    rep = torch.load(os.path.join(d, "replicated.pt"), map_location=map_location, weights_only=False)
    shard = torch.load(os.path.join(d, f"experts_rank{int(rank)}.pt"), map_location=map_location, weights_only=False)
    if int(rep["world"]) != int(world) or int(shard["world"]) != int(world):
        raise ValueError(f"checkpoint was written by {rep['world']} ranks, this run has {world}")
    if int(shard["rank"]) != int(rank):
        raise ValueError("expert shard belongs to another rank")
    return int(step), rep["state"], shard["state"]
