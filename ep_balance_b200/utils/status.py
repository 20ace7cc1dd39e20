"""Device status words, read by the host without stalling the step.

Every wait inside the native kernels is bounded, and capacity guards drop rows instead of writing out of
bounds; both record ``{code, site, detail}`` in a 4-int status word and carry on.  A step that ran with a
non-zero status is damaged (rows were dropped, or a peer's data did not arrive in time) and must not reach
the weights.  Two pieces make that a detected, contained failure:

* :class:`StatusBoard` -- one ``[n, 4]`` int32 device tensor; row ``i`` is the status word of layer ``i``.
  ``FusedAdamW(..., guard=board.words)`` makes the optimizer kernel skip its update while any row is
  non-zero, so the damaged step leaves the parameters bit-unchanged.
* :class:`StatusMonitor` -- every step it enqueues an asynchronous copy of the board into pinned memory
  and looks at the copies of earlier steps that have landed (no synchronisation: a copy is read at the
  earliest one step late, like a loss that is logged late).  A non-zero word raises
  :class:`MoEStatusError` naming layer, code, site and detail.

The reference never drops tokens (scripts/README.md:494-497) and guards its row budget with a device-side
assert (eplb/integration/grouped_mlp.py:180-205); here the guard is a status that the host turns into an
exception while the CUDA context stays usable.
"""

from __future__ import annotations

from collections import deque
from typing import Deque, List, Optional, Tuple

import torch

STATUS_NAMES = {0: "ok", 1: "barrier timeout", 2: "signal timeout", 3: "pipeline timeout", 4: "row overflow",
                5: "bad argument"}


class MoEStatusError(RuntimeError):
    def __init__(self, layer: int, code: int, site: int, detail: int, step: Optional[int] = None) -> None:
        self.layer, self.code, self.site, self.detail, self.step = layer, code, site, detail, step
        when = f" (seen in the copy taken at step {step})" if step is not None else ""
        super().__init__(f"MoE runtime status on layer {layer}: {STATUS_NAMES.get(code, code)} "
                         f"(code {code}, site {site}, detail {detail}){when}")


def raise_if_set(words, step: Optional[int] = None) -> None:
    """``words``: nested list / CPU tensor ``[n, 4]``.  Raises for the first non-zero row."""
    rows = words.tolist() if isinstance(words, torch.Tensor) else words
    for layer, (code, site, detail, _) in enumerate(rows):
        if code != 0:
            raise MoEStatusError(layer, int(code), int(site), int(detail), step)


class StatusBoard:
    """The status words of ``n`` layers in one tensor (so that one copy, and one optimizer guard, covers all)."""

    def __init__(self, n: int, device) -> None:
        self.words = torch.zeros((max(int(n), 1), 4), dtype=torch.int32, device=device)

    def row(self, i: int) -> torch.Tensor:
        return self.words[i]

    def clear(self) -> None:
        self.words.zero_()

    def check_now(self) -> None:
        """Synchronous read (tests, end of a run, before writing a checkpoint)."""
        raise_if_set(self.words.cpu())


class StatusMonitor:
    def __init__(self, words: torch.Tensor, depth: int = 4) -> None:
        if words.dim() != 2 or words.shape[1] != 4 or words.dtype != torch.int32:
            raise ValueError("status words must be an int32 tensor [n, 4]")
        self.words = words
        self._slots: List[torch.Tensor] = [torch.zeros(words.shape, dtype=torch.int32).pin_memory() if words.is_cuda
                                           else torch.zeros(words.shape, dtype=torch.int32) for _ in range(depth)]
        self._pending: Deque[Tuple[int, int, Optional["torch.cuda.Event"]]] = deque()  # (step, slot, event)
        self._step = 0

    def poll(self) -> None:
        """Call once per step, after the step's kernels are enqueued.  Never blocks unless every staging slot is
        still in flight (the host is ``depth`` steps ahead of the device)."""
        self._inspect(block=len(self._pending) == len(self._slots))
        slot = self._step % len(self._slots)
        self._slots[slot].copy_(self.words, non_blocking=True)
        event = None
        if self.words.is_cuda:
            event = torch.cuda.Event()
            event.record()
        self._pending.append((self._step, slot, event))
        self._step += 1

    def _inspect(self, block: bool) -> None:
        while self._pending:
            step, slot, event = self._pending[0]
            if event is not None and not event.query():
                if not block:
                    return
                event.synchronize()
            self._pending.popleft()
            block = False
            raise_if_set(self._slots[slot], step)

    def drain(self) -> None:
        """Wait for every copy in flight and check it (end of training, before a checkpoint)."""
        while self._pending:
            self._inspect(block=True)
