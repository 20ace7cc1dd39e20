"""Symmetric heap: the same buffers at known addresses on every expert-parallel rank.

Each rank owns one device allocation carved into named, 256-byte aligned regions; every peer's
allocation is mapped into this process, so a kernel can store into or load from region ``name``
of rank ``p`` through ``heap.peer_ptrs(name)[p]``.  This is what the reference obtains from NCCL
symmetric windows (nccl_gin/csrc/nccl_gin.cu:941-968, ``ncclMemAlloc`` +
``ncclCommWindowRegister``); on one NVSwitch box every peer is load/store reachable, so plain CUDA
IPC mappings are enough and no proxy or RDMA path exists.

Backends
  ``ipc``    one ``cudaMalloc`` per rank, handles exchanged through the process group, peers
             mapped with ``cudaIpcOpenMemHandle`` (multi-process, one rank per GPU).
  ``local``  single process: ``num_ranks`` heaps in one address space.  With ``num_ranks > 1`` this
             emulates a cluster on one GPU for tests: kernels of different logical ranks are
             ordered by the stream instead of by cross-rank barriers.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

ALIGN = 256
GUARD = 256          # bytes of canary after every region
GUARD_BYTE = 0xA5


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class HeapLayout:
    """Named regions inside one flat allocation; identical on every rank by construction."""

    def __init__(self) -> None:
        self.regions: Dict[str, Tuple[int, Tuple[int, ...], torch.dtype]] = {}
        self.guards: Dict[str, int] = {}
        self.nbytes = 0

    def add(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> None:
        if name in self.regions:
            raise KeyError(f"region {name!r} defined twice")
        numel = 1
        for s in shape:
            numel *= int(s)
        self.regions[name] = (self.nbytes, tuple(int(s) for s in shape), dtype)
        end = _round_up(self.nbytes + numel * torch.empty((), dtype=dtype).element_size(), ALIGN)
        self.guards[name] = end          # a canary of GUARD bytes sits between this region and the next
        self.nbytes = end + GUARD


class SymmetricHeap:
    def __init__(self, layout: HeapLayout, device: torch.device, *, group=None, backend: Optional[str] = None,
                 num_local_ranks: int = 1) -> None:
        from ..ops.extension import load

        self.ext = load()
        self.layout = layout
        self.device = torch.device(device)
        self.group = group
        distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.backend = backend or ("ipc" if distributed else "local")
        self._owned: List[int] = []
        self._opened: List[int] = []
        nbytes = max(layout.nbytes, ALIGN)
        dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        with torch.cuda.device(dev_index):
            if self.backend == "local":
                self.world, self.rank = int(num_local_ranks), 0
                self.bases = []
                for _ in range(self.world):
                    ptr, _h = self.ext.ipc_alloc(nbytes)
                    self._owned.append(ptr)
                    self.bases.append(ptr)
            elif self.backend == "ipc":
                self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
                ptr, handle = self.ext.ipc_alloc(nbytes)
                self._owned.append(ptr)
                handles: List[Optional[bytes]] = [None] * self.world
                dist.all_gather_object(handles, handle, group=group)
                self.bases = []
                for r, h in enumerate(handles):
                    if r == self.rank:
                        self.bases.append(ptr)
                    else:
                        p = self.ext.ipc_open(h)
                        self._opened.append(p)
                        self.bases.append(p)
                dist.barrier(group=group)
            else:
                raise ValueError(f"unknown symmetric heap backend {self.backend!r}")
        self._flat = [self.ext.tensor_from_ptr(b, nbytes, dev_index) for b in self.bases]
        self._ptr_tables: Dict[str, torch.Tensor] = {}
        for r in ([self.rank] if self.backend == "ipc" else range(self.world)):   # every rank paints its own heap
            for off in layout.guards.values():
                self._flat[r][off:off + GUARD].fill_(GUARD_BYTE)
        if self.backend == "ipc":
            torch.cuda.synchronize(dev_index)
            dist.barrier(group=group)

    # ---- views ---------------------------------------------------------------
    def tensor(self, name: str, rank: Optional[int] = None) -> torch.Tensor:
        """View of region ``name`` on ``rank`` (default: this rank)."""
        off, shape, dtype = self.layout.regions[name]
        r = self.rank if rank is None else int(rank)
        numel = 1
        for s in shape:
            numel *= s
        nb = numel * torch.empty((), dtype=dtype).element_size()
        return self._flat[r][off:off + nb].view(dtype).view(shape)

    def address(self, name: str, rank: Optional[int] = None) -> int:
        r = self.rank if rank is None else int(rank)
        return self.bases[r] + self.layout.regions[name][0]

    def peer_ptrs(self, name: str, *, as_seen_by: Optional[int] = None) -> torch.Tensor:
        """Device int64 array with region ``name``'s address on every rank."""
        key = name
        t = self._ptr_tables.get(key)
        if t is None:
            t = torch.tensor([self.address(name, r) for r in range(self.world)], dtype=torch.int64,
                             device=self.device)
            self._ptr_tables[key] = t
        return t

    def damaged_guards(self, rank: Optional[int] = None) -> List[str]:
        """Names of the regions whose trailing canary was overwritten on ``rank`` (default: this rank): a kernel
        wrote past the end of that region.  One device-to-host read; for tests and debugging."""
        r = self.rank if rank is None else int(rank)
        bad = []
        for name, off in self.layout.guards.items():
            if not bool((self._flat[r][off:off + GUARD] == GUARD_BYTE).all()):
                bad.append(name)
        return bad

    def close(self) -> None:
        self._flat = []
        self._ptr_tables = {}
        for p in self._opened:
            try:
                self.ext.ipc_close(p)
            except Exception:
                pass
        for p in self._owned:
            try:
                self.ext.ipc_free(p)
            except Exception:
                pass
        self._opened, self._owned = [], []

    def __del__(self) -> None:  # best effort; explicit close() is preferred
        try:
            self.close()
        except Exception:
            pass
