"""One-sided communication over the symmetric heap: symmetric tensors, get/put, signals, fences.

This is the counterpart of the reference's ``nccl_gin`` package (nccl_gin/__init__.py:
``init``, ``create_tensor``, ``is_symmetric_tensor``, ``get``/``put``, ``get_batched``/
``put_batched``, ``signal``/``wait_signal``/``test_signal``/``put_signal``, ``world_fence``,
``destroy``; kernels in nccl_gin/csrc/nccl_gin.cu:149-827).  The reference registers NCCL
symmetric windows and reaches non-NVLink peers through a network proxy; on one NVSwitch box every
peer's window is mapped into this process with CUDA IPC, so every transfer is a kernel of this
package that loads from or stores to the peer's memory directly.

A :class:`SymmetricWorld` owns one arena per rank.  ``create_tensor`` is a collective bump
allocation: every rank must call it in the same order with the same shapes, which is what makes
offset ``o`` of rank ``a``'s arena the same tensor as offset ``o`` of rank ``b``'s.

All calls enqueue on the current CUDA stream and return; nothing here synchronises the host.
Waits on the device are bounded (1.5 s); a wait that runs out writes a status triple that
:meth:`SymmetricWorld.check_status` turns into an exception.

Single-process emulation: ``SymmetricWorld.local(n)`` returns ``n`` worlds that share one address
space on one GPU.  Kernels of different logical ranks are then ordered by the stream, so
``world_fence`` and ``wait_signal`` never spin on a peer there (waiting on another kernel of the
same GPU is not allowed to depend on concurrency); they only check that the awaited value is
already present.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .symm import HeapLayout, SymmetricHeap

NUM_SIGNALS = 64      # nccl_gin: ginSignalCount=64 (nccl_gin/csrc/nccl_gin.cu:109-126)
NUM_FENCES = 16       # nccl_gin: barrierCount=16
WAIT_BUDGET_NS = 1_500_000_000
_ALIGN = 256


def _nbytes(shape: Sequence[int], dtype: torch.dtype) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n * torch.empty((), dtype=dtype).element_size()


class SymmetricWorld:
    """One rank's handle on the symmetric arena of an expert-parallel group."""

    def __init__(self, arena_bytes: int, device, *, group=None, heap: Optional[SymmetricHeap] = None,
                 rank: Optional[int] = None) -> None:
        self.device = torch.device(device)
        if heap is None:
            layout = HeapLayout()
            layout.add("arena", (int(arena_bytes),), torch.uint8)
            layout.add("signals", (NUM_SIGNALS,), torch.int32)
            layout.add("fences", (NUM_FENCES,), torch.int32)
            heap = SymmetricHeap(layout, self.device, group=group)
        self.heap = heap
        self.ext = heap.ext
        self.rank = heap.rank if rank is None else int(rank)
        self.world = heap.world
        self.emulated = heap.backend == "local" and heap.world > 1
        self.group = group
        self.arena_bytes = heap.layout.regions["arena"][1][0]
        self._arena = heap.tensor("arena", self.rank)
        self._arena_base = heap.address("arena", self.rank)
        self._cursor = 0
        self._tensors: Dict[int, Tuple[int, int]] = {}     # data_ptr -> (offset, nbytes)
        self.window_ptrs = heap.peer_ptrs("arena")
        self.signal_ptrs = heap.peer_ptrs("signals")
        self.fence_ptrs = heap.peer_ptrs("fences")
        self._signals = heap.tensor("signals", self.rank)
        self._fence_epochs = torch.zeros(NUM_FENCES, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.use_bulk = True
        # CTAs per descriptor.  None: spread about two waves of CTAs over the descriptors of a call, so a
        # short schedule (one or two replica slots) still keeps enough bytes in flight to fill NVLink.
        # The reference uses a fixed EPLB_GIN_GRID=8 (eplb/integration/gin_weights.py:106).
        self.blocks_per_desc: Optional[int] = None
        self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count

    # ------------------------------------------------------------------ construction
    @classmethod
    def local(cls, num_ranks: int, arena_bytes: int, device) -> List["SymmetricWorld"]:
        """``num_ranks`` logical ranks in this process on one GPU (tests, single-GPU bring-up)."""
        layout = HeapLayout()
        layout.add("arena", (int(arena_bytes),), torch.uint8)
        layout.add("signals", (NUM_SIGNALS,), torch.int32)
        layout.add("fences", (NUM_FENCES,), torch.int32)
        heap = SymmetricHeap(layout, torch.device(device), backend="local", num_local_ranks=num_ranks)
        return [cls(arena_bytes, device, heap=heap, rank=r) for r in range(num_ranks)]

    # ------------------------------------------------------------------ symmetric tensors
    def create_tensor(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """Collective: the next ``shape``/``dtype`` tensor of the arena (zero-initialised)."""
        nb = _nbytes(shape, dtype)
        off = (self._cursor + _ALIGN - 1) // _ALIGN * _ALIGN
        if off + nb > self.arena_bytes:
            raise MemoryError(f"symmetric arena exhausted: need {off + nb} of {self.arena_bytes} bytes")
        self._cursor = off + nb
        t = self._arena[off:off + nb].view(dtype).view(tuple(int(s) for s in shape))
        self._tensors[t.data_ptr()] = (off, nb)
        return t

    def is_symmetric_tensor(self, t: torch.Tensor) -> bool:
        p = t.data_ptr() if t.is_cuda else -1
        return self._arena_base <= p < self._arena_base + self.arena_bytes

    def offset_of(self, t: torch.Tensor) -> int:
        """Byte offset of ``t`` (a symmetric tensor or a view into one) inside the arena."""
        if not self.is_symmetric_tensor(t):
            raise ValueError("tensor does not live in the symmetric arena")
        return t.data_ptr() - self._arena_base

    def peer_view(self, t: torch.Tensor, peer: int) -> torch.Tensor:
        """The same symmetric tensor as it exists on ``peer`` (mapped memory; for tests and debugging)."""
        off = self.offset_of(t)
        nb = t.numel() * t.element_size()
        return self.heap.tensor("arena", peer)[off:off + nb].view(t.dtype).view(t.shape)

    # ------------------------------------------------------------------ transfers
    def _descs(self, rows: Sequence[Tuple[int, int, int, int]]) -> torch.Tensor:
        return torch.tensor(list(rows), dtype=torch.int64, device=self.device).view(-1, 4)

    def get_batched(self, local: torch.Tensor, desc: torch.Tensor, *, blocks: Optional[int] = None) -> None:
        """For every descriptor row ``(peer, remote_off, local_off, nbytes)``: copy ``nbytes`` from byte
        ``remote_off`` of ``peer``'s arena to byte ``local_off`` of ``local``.  ``peer < 0`` skips the row.
        ``desc`` is an int64 ``[K, 4]`` device tensor, so a schedule computed on the GPU is consumed
        without a host read (reference: nccl_gin.get_batched, nccl_gin/csrc/nccl_gin.cu:1143-1193)."""
        self._check_local(local)
        self.ext.get_batched(desc.contiguous(), self.window_ptrs, local.data_ptr(), bool(self.use_bulk),
                             self._blocks(blocks, desc), self.status)

    def put_batched(self, local: torch.Tensor, desc: torch.Tensor, *, blocks: Optional[int] = None) -> None:
        """Mirror of :meth:`get_batched`: ``local[local_off:+nbytes]`` is stored into ``peer``'s arena at
        ``remote_off``; the kernel ends with a system-scope fence, so a following :meth:`signal`
        orders after the data (reference: nccl_gin.put_batched, nccl_gin/csrc/nccl_gin.cu:1195-1230)."""
        self._check_local(local)
        self.ext.put_batched(desc.contiguous(), self.window_ptrs, local.data_ptr(), bool(self.use_bulk),
                             self._blocks(blocks, desc), self.status)

    def _blocks(self, blocks: Optional[int], desc: torch.Tensor) -> int:
        if blocks:
            return int(blocks)
        if self.blocks_per_desc:
            return int(self.blocks_per_desc)
        return max(8, min(128, 2 * self._sm_count // max(int(desc.shape[0]), 1)))

    def get(self, dst: torch.Tensor, src: torch.Tensor, peer: int, *, blocks: Optional[int] = None) -> None:
        """``dst[...] = src`` as it exists on ``peer``; ``src`` is a (view of a) symmetric tensor."""
        nb = min(dst.numel() * dst.element_size(), src.numel() * src.element_size())
        self.get_batched(dst, self._descs([(int(peer), self.offset_of(src), 0, nb)]), blocks=blocks)

    def put(self, dst: torch.Tensor, src: torch.Tensor, peer: int, *, blocks: Optional[int] = None) -> None:
        """Store local ``src`` into symmetric ``dst`` as it exists on ``peer``."""
        nb = min(dst.numel() * dst.element_size(), src.numel() * src.element_size())
        self.put_batched(src, self._descs([(int(peer), self.offset_of(dst), 0, nb)]), blocks=blocks)

    def put_signal(self, dst: torch.Tensor, src: torch.Tensor, peer: int, idx: int, value: int = 1) -> None:
        """:meth:`put` followed by a signal increment on ``peer`` that orders after the data."""
        self.put(dst, src, peer)
        self.signal(peer, idx, value)

    @staticmethod
    def _check_local(local: torch.Tensor) -> None:
        if not local.is_cuda or not local.is_contiguous():
            raise ValueError("the local side of a one-sided transfer must be a contiguous CUDA tensor")

    # ------------------------------------------------------------------ signals and fences
    def signal(self, peer: int, idx: int, value: int = 1) -> None:
        """Add ``value`` to signal ``idx`` of ``peer`` (``peer=-1``: of every rank), release at system scope."""
        self._check_idx(idx, NUM_SIGNALS)
        self.ext.signal_peers(self.signal_ptrs, int(peer), int(idx), int(value))

    def wait_signal(self, idx: int, expected: int) -> None:
        """Hold the stream until this rank's signal ``idx`` has reached ``expected`` (bounded)."""
        self._check_idx(idx, NUM_SIGNALS)
        budget = 0 if self.emulated else WAIT_BUDGET_NS
        self.ext.wait_signal(self._signals.data_ptr() + 4 * int(idx), int(expected), int(idx), budget, self.status)

    def test_signal(self, idx: int) -> int:
        """Current value of this rank's signal ``idx`` (a host read of one word; never blocks on a peer)."""
        self._check_idx(idx, NUM_SIGNALS)
        return int(self._signals[int(idx)].item()) & 0xFFFFFFFF

    def reset_signal(self, idx: int) -> None:
        self._check_idx(idx, NUM_SIGNALS)
        self._signals[int(idx)].zero_()

    def world_fence(self, idx: int = 0) -> None:
        """Device-side barrier over all ranks on the current stream: work enqueued before it on any
        rank is visible to work enqueued after it on every rank (reference: nccl_gin.world_fence,
        nccl_gin/csrc/nccl_gin.cu:823-827, 1266-1279).  In single-process emulation the stream already
        orders the logical ranks, so the fence is a no-op there."""
        self._check_idx(idx, NUM_FENCES)
        if self.emulated or self.world == 1:
            return
        self.ext.symm_barrier(self.fence_ptrs, int(idx), self.rank, self._fence_epochs[int(idx):int(idx) + 1],
                              self.status)

    @staticmethod
    def _check_idx(idx: int, limit: int) -> None:
        if not 0 <= int(idx) < limit:
            raise IndexError(f"index {idx} outside [0, {limit})")

    # ------------------------------------------------------------------ status / teardown
    def check_status(self) -> None:
        """Raise if a bounded wait ran out or a descriptor was rejected (one host read)."""
        code, site, detail, _ = self.status.tolist()
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"one-sided transfer failed on rank {self.rank}: code={code} site={site} detail={detail}")

    def destroy(self) -> None:
        self._tensors.clear()
        self._arena = None
        self._signals = None
        if self.rank == self.heap.rank or not self.emulated:
            self.heap.close()


# ---------------------------------------------------------------------- module-level facade
_WORLD: Optional[SymmetricWorld] = None


def init(arena_bytes: int, device=None, group=None) -> SymmetricWorld:
    """Create the process-wide world (collective over ``group``); mirrors ``nccl_gin.init``."""
    global _WORLD
    if _WORLD is None:
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        _WORLD = SymmetricWorld(arena_bytes, dev, group=group)
    return _WORLD


def world() -> SymmetricWorld:
    if _WORLD is None:
        raise RuntimeError("onesided.init() has not been called")
    return _WORLD


def destroy() -> None:
    global _WORLD
    if _WORLD is not None:
        if dist.is_available() and dist.is_initialized() and _WORLD.world > 1:
            dist.barrier(group=_WORLD.group)
        _WORLD.destroy()
        _WORLD = None


def get_rank() -> int:
    return world().rank


def get_world_size() -> int:
    return world().world


def create_tensor(shape, dtype) -> torch.Tensor:
    return world().create_tensor(shape, dtype)


def is_symmetric_tensor(t: torch.Tensor) -> bool:
    return _WORLD is not None and _WORLD.is_symmetric_tensor(t)
