"""Host-side failure detection for an expert-parallel group.

The reference has no failure detection: its device waits are unbounded and a lost rank hangs the
job (nccl_gin/csrc/nccl_gin.cu:520-533, 300, 825-826).  Here every device wait is bounded and reports
through a status word; this module is the host half: ranks publish a heartbeat to a c10d store after
every step, look at their peers' heartbeats *before* enqueuing the next step (whose kernels would wait
on those peers), and publish their own device-side failures so that the others stop launching too.

Nothing here touches a GPU, so the whole module is exercised with CPU processes (tests/test_health_cpu.py):
a rank that raises between steps, a rank that never joins, a heartbeat that is dropped, a corrupted
omega row.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional

import torch


class PeerFailure(RuntimeError):
    """One or more ranks are missing, stale, or reported a failure."""

    def __init__(self, message: str, ranks: Iterable[int]) -> None:
        super().__init__(message)
        self.ranks = sorted(int(r) for r in ranks)


@dataclass
class PeerState:
    step: int
    wall_time: float
    failed: Optional[str] = None


class Heartbeat:
    """Per-rank ``(step, wall time)`` records in a ``torch.distributed`` store.

    ``store`` is any c10d store (``TCPStore``, ``FileStore``, ``HashStore``, or the store of the default
    process group).  Keys: ``<prefix>/hb/<rank>`` and ``<prefix>/fail/<rank>``.
    """

    def __init__(self, store, rank: int, world: int, *, prefix: str = "epb", stale_after_s: float = 30.0,
                 clock=time.time) -> None:
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.prefix, self.stale_after_s, self.clock = prefix, float(stale_after_s), clock

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{int(rank)}"

    # ---- writers
    def beat(self, step: int) -> None:
        self.store.set(self._key("hb", self.rank), f"{int(step)}:{self.clock():.6f}")

    def report_failure(self, reason: str) -> None:
        """Tell the group that this rank cannot continue (device status word set, exception, ...)."""
        self.store.set(self._key("fail", self.rank), str(reason)[:512])

    # ---- readers
    def _get(self, key: str) -> Optional[str]:
        if self.store.num_keys() == 0 or not self.store.check([key]):
            return None
        return self.store.get(key).decode()

    def peers(self) -> Dict[int, Optional[PeerState]]:
        out: Dict[int, Optional[PeerState]] = {}
        for r in range(self.world):
            raw = self._get(self._key("hb", r))
            fail = self._get(self._key("fail", r))
            if raw is None:
                out[r] = PeerState(-1, 0.0, fail) if fail is not None else None
                continue
            step, wall = raw.split(":")
            out[r] = PeerState(int(step), float(wall), fail)
        return out

    def wait_for_all(self, timeout_s: float, poll_s: float = 0.05) -> None:
        """Block until every rank has published a first heartbeat; raise ``PeerFailure`` with the
        missing ranks when ``timeout_s`` passes."""
        deadline = self.clock() + timeout_s
        while True:
            state = self.peers()
            missing = [r for r, s in state.items() if s is None]
            failed = [r for r, s in state.items() if s is not None and s.failed]
            if failed:
                raise PeerFailure(f"ranks {failed} reported a failure before joining", failed)
            if not missing:
                return
            if self.clock() >= deadline:
                raise PeerFailure(f"ranks {missing} never joined within {timeout_s:.1f} s", missing)
            time.sleep(poll_s)

    def check_peers(self, min_step: Optional[int] = None) -> None:
        """Raise ``PeerFailure`` when a peer reported a failure, has no heartbeat, is older than
        ``stale_after_s``, or (with ``min_step``) has not reached that step."""
        now = self.clock()
        bad: Dict[int, str] = {}
        for r, s in self.peers().items():
            if r == self.rank:
                continue
            if s is None:
                bad[r] = "no heartbeat"
            elif s.failed:
                bad[r] = f"reported: {s.failed}"
            elif now - s.wall_time > self.stale_after_s:
                bad[r] = f"last heartbeat {now - s.wall_time:.1f} s ago (step {s.step})"
            elif min_step is not None and s.step < min_step:
                bad[r] = f"at step {s.step}, expected >= {min_step}"
        if bad:
            raise PeerFailure("; ".join(f"rank {r}: {why}" for r, why in sorted(bad.items())), bad.keys())


class StepGuard:
    """Glue for a training loop: ``before_step`` refuses to launch when a peer is gone, ``after_step``
    turns a device status word into a published failure and a heartbeat otherwise.

    ``status_checks`` are callables that raise when a device-side bounded wait ran out
    (``FusedMoE.check_status``, ``SymmetricWorld.check_status``, ``GPTMoE.check_status``); each costs one
    small device-to-host read, so pass ``check_every`` > 1 to amortise it.
    """

    def __init__(self, heartbeat: Heartbeat, status_checks=(), *, check_every: int = 1) -> None:
        self.hb, self.status_checks, self.check_every = heartbeat, list(status_checks), max(1, int(check_every))

    def before_step(self, step: int) -> None:
        self.hb.check_peers()

    def after_step(self, step: int) -> None:
        if step % self.check_every == 0:
            for check in self.status_checks:
                try:
                    check()
                except Exception as exc:  # publish, then let the caller see it
                    self.hb.report_failure(f"step {step}: {exc}")
                    raise
        self.hb.beat(step)


def check_omega(omega: torch.Tensor, expected_row_sums: Optional[torch.Tensor] = None) -> List[int]:
    """Ranks whose row of the gathered load matrix cannot be right: negative counts, or a row sum that
    differs from the number of routing units that rank reported (tokens x top-k).  An empty list means
    the matrix is plausible.  One host read; meant for debugging and for the failure tests."""
    om = omega.detach().to("cpu", torch.int64)
    bad = set((om < 0).any(dim=1).nonzero().flatten().tolist())
    if expected_row_sums is not None:
        want = torch.as_tensor(expected_row_sums).to("cpu", torch.int64).flatten()
        bad |= set((om.sum(dim=1) != want).nonzero().flatten().tolist())
    return sorted(bad)
