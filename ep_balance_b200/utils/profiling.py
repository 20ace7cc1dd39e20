"""Region timing for the balancer and the MoE layer.

A :class:`Profiler` keeps a ledger of named regions.  GPU regions are bracketed by CUDA events taken from
a per-device pool and left *in flight*: nothing waits for them when the region closes.  They are settled
in one batch -- by waiting on the newest event of each stream, not on the whole device -- when a report
is asked for or the in-flight list is full, so profiling adds no per-region host synchronisation.  A
ledger can be reduced over the ranks of a process group (mean and max per region: the max is the
straggler that a device-side wait on the other ranks would see).

The module-level functions drive one process-wide profiler configured from the environment:

``EPLB_PROFILE=1``       aggregate table every ``EPLB_PROFILE_EVERY`` MoE invocations,
``EPLB_DEBUG_TIMING=1``  one ``[EPLB-debug rN] ...`` line per MoE invocation,
``EPLB_PROFILE_ALL_RANKS``, ``EPLB_PROFILE_MAX_PENDING``, ``EPLB_PROFILE_RESET_AT`` as named.

Region names, the ``name=1.234ms(x2)/64.00MiB/31.86GB/s`` field format, the ``[EPLB-profile rN]`` table and
the ``[EPLB-debug rN]`` lines are those of the reference (eplb/integration/profiling.py:15-338;
scripts/README.md:313-329), so its log extractors read these logs unchanged.  Every region is also a
``torch.profiler.record_function("eplb/<name>")`` range.
"""

from __future__ import annotations

import atexit
import contextlib
import os
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Iterable, List, Mapping, Optional, Tuple

import torch

MIB = float(1 << 20)

# bucket label -> the region names that feed it (apply-mode and native-Megatron regions share buckets)
FORWARD_PHASES: Tuple[Tuple[str, Tuple[str, ...]], ...] = (
    ("solver", ("solve",)),
    ("omega_gather", ("all_gather_omega",)),
    ("router", ("apply/route", "native/route")),
    ("shared_expert", ("apply/shared_expert", "native/shared_expert")),
    ("expert_transfer", ("apply/weight_move",)),
    ("dispatch", ("apply/dispatch", "native/dispatch")),
    ("expert_gemm", ("apply/expert_gemm", "native/expert_gemm")),
    ("combine", ("apply/combine", "native/combine")),
)
BACKWARD_PHASES: Tuple[Tuple[str, Tuple[str, ...]], ...] = (
    ("expert_repull", ("apply/weight_repull",)),
    ("expert_grad_reduce", ("apply/grad_move",)),
)


def _env_on(env: Mapping[str, str], key: str) -> bool:
    return env.get(key, "0").strip().lower() not in ("", "0", "false", "no", "off")


@dataclass
class RegionStat:
    """Running totals of one region."""

    count: int = 0
    total_ms: float = 0.0
    min_ms: float = float("inf")
    max_ms: float = 0.0
    last_ms: float = 0.0
    total_bytes: int = 0
    last_bytes: int = 0

    def add(self, ms: float, nbytes: int = 0) -> None:
        self.count += 1
        self.total_ms += ms
        self.last_ms = ms
        if ms < self.min_ms:
            self.min_ms = ms
        if ms > self.max_ms:
            self.max_ms = ms
        self.total_bytes += nbytes
        self.last_bytes = nbytes

    @property
    def mean_ms(self) -> float:
        return self.total_ms / self.count if self.count else 0.0


def _payload(value) -> int:
    """Bytes moved by a region: an int, or a one-element tensor that is only read when settled."""
    if value is None:
        return 0
    if isinstance(value, torch.Tensor):
        if value.numel() != 1:
            raise ValueError("profiling payload_bytes tensor must contain exactly one value")
        value = value.item()
    value = int(value)
    if value < 0:
        raise ValueError("profiling payload_bytes must be non-negative")
    return value


class _EventPool:
    """Timing events are reused: a hot loop with profiling on creates no CUDA objects after warm-up."""

    def __init__(self) -> None:
        self._free: List["torch.cuda.Event"] = []

    def take(self) -> "torch.cuda.Event":
        return self._free.pop() if self._free else torch.cuda.Event(enable_timing=True)

    def give(self, *events) -> None:
        self._free.extend(events)


@dataclass
class _InFlight:
    name: str
    begin: "torch.cuda.Event"
    end: "torch.cuda.Event"
    stream_key: int
    payload: object


@dataclass
class Profiler:
    profile: bool = False          # aggregate table mode
    debug: bool = False            # one line per MoE invocation
    every: int = 20
    all_ranks: bool = False
    max_in_flight: int = 1024
    reset_peak_at: int = 0
    rank: str = ""
    ledger: Dict[str, RegionStat] = field(default_factory=dict)      # since the last reset
    window: Dict[str, RegionStat] = field(default_factory=dict)      # since the last begin_window (debug mode)
    calls: int = 0
    logger: Optional[Callable[[str], None]] = None                    # where deferred backward lines go

    def __post_init__(self) -> None:
        self._in_flight: Deque[_InFlight] = deque()
        self._pool = _EventPool()

    # ------------------------------------------------------------------ configuration
    @classmethod
    def from_env(cls, env: Mapping[str, str] = os.environ) -> "Profiler":
        return cls(profile=_env_on(env, "EPLB_PROFILE"), debug=_env_on(env, "EPLB_DEBUG_TIMING"),
                   every=int(env.get("EPLB_PROFILE_EVERY", "20")), all_ranks=_env_on(env, "EPLB_PROFILE_ALL_RANKS"),
                   max_in_flight=int(env.get("EPLB_PROFILE_MAX_PENDING", "1024")),
                   reset_peak_at=int(env.get("EPLB_PROFILE_RESET_AT", "0")), rank=env.get("RANK", ""))

    @property
    def active(self) -> bool:
        return self.profile or self.debug

    def tag(self, kind: str) -> str:
        return f"[EPLB-{kind} r{self.rank}]" if self.rank else f"[EPLB-{kind}]"

    # ------------------------------------------------------------------ recording
    def _book(self, name: str, ms: float, payload) -> None:
        nbytes = _payload(payload)
        self.ledger.setdefault(name, RegionStat()).add(ms, nbytes)
        if self.debug:
            self.window.setdefault(name, RegionStat()).add(ms, nbytes)

    @contextlib.contextmanager
    def region(self, name: str, *, time_it: bool = False, device=None, stream=None, payload_bytes=0):
        with torch.profiler.record_function(f"eplb/{name}"):
            if not (self.active and time_it):
                yield
                return
            gpu = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
            if not gpu:
                t0 = time.perf_counter()
                try:
                    yield
                finally:
                    self._book(name, (time.perf_counter() - t0) * 1e3, payload_bytes)
                return
            begin, end = self._pool.take(), self._pool.take()
            begin.record(stream)
            try:
                yield
            finally:
                end.record(stream)
                key = stream.cuda_stream if stream is not None else torch.cuda.current_stream().cuda_stream
                self._in_flight.append(_InFlight(name, begin, end, key, payload_bytes))
                if len(self._in_flight) >= self.max_in_flight:
                    self.settle()

    def settle(self) -> None:
        """Book every region still in flight.  Waits once per stream, on that stream's newest event."""
        if not self._in_flight:
            return
        newest: Dict[int, "torch.cuda.Event"] = {}
        for item in self._in_flight:
            newest[item.stream_key] = item.end
        for ev in newest.values():
            ev.synchronize()
        while self._in_flight:
            item = self._in_flight.popleft()
            self._book(item.name, item.begin.elapsed_time(item.end), item.payload)
            self._pool.give(item.begin, item.end)

    def reset(self) -> None:
        self.settle()
        self.ledger.clear()
        self.window.clear()
        self.calls = 0

    # ------------------------------------------------------------------ reports
    def _bucket_fields(self, buckets: Iterable[Tuple[str, Tuple[str, ...]]], missing: Optional[Mapping[str, str]] = None
                       ) -> List[str]:
        missing = missing or {}
        fields = []
        for label, names in buckets:
            n, ms, nb = 0, 0.0, 0
            for name in names:
                st = self.window.get(name)
                if st is not None:
                    n, ms, nb = n + st.count, ms + st.total_ms, nb + st.total_bytes
            if n == 0:
                if label in missing:
                    fields.append(f"{label}={missing[label]}")
                continue
            text = f"{label}={ms:.3f}ms"
            if n > 1:
                text += f"(x{n})"
            if nb:
                text += f"/{nb / MIB:.2f}MiB/{nb / (max(ms, 1e-12) * 1e6):.2f}GB/s"
            fields.append(text)
        return fields

    def begin_window(self) -> None:
        """Start the timing window of one MoE invocation.  Backward regions of the previous invocation
        finish after its forward line was printed, so they are reported here, one window late."""
        if not self.debug:
            return
        self.settle()
        self._flush_backward()
        self.window.clear()

    def _flush_backward(self) -> None:
        fields = self._bucket_fields(BACKWARD_PHASES)
        if fields and self.logger is not None:
            self.logger(f"{self.tag('debug')} mode=apply direction=backward " + " ".join(fields))

    def window_line(self, context: str = "", missing: Optional[Mapping[str, str]] = None) -> str:
        self.settle()
        fields = self._bucket_fields(FORWARD_PHASES, missing)
        self.window.clear()
        head = self.tag("debug") + (f" {context}" if context else "")
        return head + " " + (" ".join(fields) if fields else "no timing samples")

    def memory_line(self) -> str:
        tag = self.tag("profile")
        if not torch.cuda.is_available():
            return f"{tag} peak memory: n/a (no CUDA)"
        return (f"{tag} peak memory  allocated={torch.cuda.max_memory_allocated() / MIB:9.1f} MiB"
                f"   reserved={torch.cuda.max_memory_reserved() / MIB:9.1f} MiB")

    def table(self) -> str:
        self.settle()
        tag = self.tag("profile")
        if not self.ledger:
            return f"{tag} no samples (set EPLB_PROFILE=1)"
        rows = [f"{tag} region                 count    mean(ms)   min(ms)   max(ms)  mean(MiB)  payload(GB/s)"]
        for name, st in self.ledger.items():
            n = max(st.count, 1)
            rows.append(f"{tag} {name:<22} {st.count:>6}   {st.total_ms / n:>8.3f}  {st.min_ms:>8.3f}  {st.max_ms:>8.3f}"
                        f"  {st.total_bytes / n / MIB:>9.2f}  {st.total_bytes / (max(st.total_ms, 1e-12) * 1e6):>12.2f}")
        rows.append(self.memory_line())
        return "\n".join(rows)

    def after_invocation(self, logger: Optional[Callable[[str], None]], context: str = "",
                         missing: Optional[Mapping[str, str]] = None) -> None:
        if not self.active:
            return
        if self.debug:
            self.logger = logger
            line = self.window_line(context, missing)
            if logger is not None:
                logger(line)
        if not self.profile or logger is None:
            return
        self.calls += 1
        if self.every > 0 and self.calls % self.every == 0:
            logger(self.table())
        if self.reset_peak_at and self.calls == self.reset_peak_at and torch.cuda.is_available():
            torch.cuda.reset_peak_memory_stats()

    def reduce_over_ranks(self, group=None) -> Dict[str, Tuple[float, float]]:
        """{region: (mean over ranks, max over ranks)} of the per-rank mean time, in ms.  Every rank of
        ``group`` must call it with the same set of regions recorded."""
        import torch.distributed as dist

        self.settle()
        names = sorted(self.ledger)
        mine = torch.tensor([self.ledger[n].mean_ms for n in names], dtype=torch.float64)
        if not (dist.is_available() and dist.is_initialized()) or not names:
            return {n: (float(v), float(v)) for n, v in zip(names, mine)}
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
        total, worst = mine.to(dev), mine.to(dev).clone()
        dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX, group=group)
        world = dist.get_world_size(group)
        return {n: (float(t) / world, float(w)) for n, t, w in zip(names, total.cpu(), worst.cpu())}


# ---------------------------------------------------------------------- process-wide profiler
_P = Profiler.from_env()


def configure(**overrides) -> Profiler:
    """Replace the process-wide profiler (``configure()`` re-reads the environment; keyword arguments such as
    ``debug=True`` override single fields).  Returns it."""
    global _P
    _P = Profiler.from_env()
    for key, value in overrides.items():
        if not hasattr(_P, key):
            raise TypeError(f"unknown profiler field {key!r}")
        setattr(_P, key, value)
    return _P


def current() -> Profiler:
    return _P


def enabled() -> bool:
    return _P.active


def regions_requested() -> bool:
    return _P.active or _env_on(os.environ, "PROFILE_TRACE")


def debug_enabled() -> bool:
    return _P.debug


def all_ranks() -> bool:
    """Every rank reports (needed to see max-vs-mean over ranks, i.e. the straggler)."""
    return _P.all_ranks


def record(name: str, *, time_it: bool = False, device=None, stream=None, payload_bytes=0):
    """Profiler range ``eplb/<name>``; timed when a timing mode is on and ``time_it`` is set.
    ``payload_bytes``: int or one-element device tensor (read when settled).  ``stream``: the stream the
    region's work is enqueued on, when it is not the current one."""
    return _P.region(name, time_it=time_it, device=device, stream=stream, payload_bytes=payload_bytes)


def begin_debug_window() -> None:
    _P.begin_window()


def last_ms(name: str) -> float:
    _P.settle()
    st = _P.ledger.get(name)
    return st.last_ms if st is not None else 0.0


def stats() -> Dict[str, RegionStat]:
    _P.settle()
    return _P.ledger


def reset() -> None:
    _P.reset()


def reset_peak_memory() -> None:
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()


def memory_str() -> str:
    return _P.memory_line()


def summary_str() -> str:
    return _P.table()


def debug_str(context: str = "", *, missing: Optional[Mapping[str, str]] = None) -> str:
    """One invocation's compact breakdown; clears the window."""
    return _P.window_line(context, missing)


def maybe_summary(logger: Optional[Callable[[str], None]], *, context: str = "",
                  missing: Optional[Mapping[str, str]] = None) -> None:
    _P.after_invocation(logger, context, missing)


def reduce_over_ranks(group=None) -> Dict[str, Tuple[float, float]]:
    return _P.reduce_over_ranks(group)


@atexit.register
def _report_trailing_backward() -> None:
    if not _P.debug:
        return
    try:  # CUDA may already be gone at interpreter exit
        _P.settle()
        _P._flush_backward()
        _P.window.clear()
    except Exception:
        pass
