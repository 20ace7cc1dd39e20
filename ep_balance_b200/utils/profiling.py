"""Region timing for the balancer and the MoE layer.

Two env-gated modes (names and line formats follow the reference so its log extractors keep
working; reference: eplb/integration/profiling.py:15-338):

``EPLB_PROFILE=1``       aggregate table every ``EPLB_PROFILE_EVERY`` invocations,
``EPLB_DEBUG_TIMING=1``  one ``[EPLB-debug rN] ...`` line per MoE invocation.

GPU regions are bracketed with CUDA events that are only *queued*; they are resolved in
one batch (a single device sync) when a summary is read or the queue is full, so turning
profiling on adds no per-region host sync.  Every region is also a
``torch.profiler.record_function("eplb/<name>")`` range.
"""

from __future__ import annotations

import atexit
import contextlib
import os
import time
from collections import OrderedDict
from typing import Callable, List, Mapping, Optional, Sequence, Tuple

import torch

MIB = 1024.0 * 1024.0

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


def _flag(name: str) -> bool:
    return os.environ.get(name, "0").strip().lower() not in ("0", "", "false", "no")


class RegionStat:
    __slots__ = ("count", "total_ms", "min_ms", "max_ms", "last_ms", "total_bytes", "last_bytes")

    def __init__(self) -> None:
        self.count, self.total_ms, self.min_ms, self.max_ms = 0, 0.0, float("inf"), 0.0
        self.last_ms, self.total_bytes, self.last_bytes = 0.0, 0, 0

    def add(self, ms: float, nbytes: int = 0) -> None:
        self.count += 1
        self.total_ms += ms
        self.last_ms = ms
        self.min_ms = min(self.min_ms, ms)
        self.max_ms = max(self.max_ms, ms)
        self.total_bytes += nbytes
        self.last_bytes = nbytes


def _bytes_of(value) -> int:
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


# Module-level state (tests monkeypatch these names).
_PROFILE_ENABLED = _flag("EPLB_PROFILE")
_DEBUG_ENABLED = _flag("EPLB_DEBUG_TIMING")
_ENABLED = _PROFILE_ENABLED or _DEBUG_ENABLED
_PERIOD = int(os.environ.get("EPLB_PROFILE_EVERY", "20"))
_ALL_RANKS = _flag("EPLB_PROFILE_ALL_RANKS")
_MAX_PENDING = int(os.environ.get("EPLB_PROFILE_MAX_PENDING", "1024"))
_RESET_AT = int(os.environ.get("EPLB_PROFILE_RESET_AT", "0"))
_RANK = os.environ.get("RANK", "")
_PREFIX = f"[EPLB-profile r{_RANK}]" if _RANK else "[EPLB-profile]"
_DEBUG_PREFIX = f"[EPLB-debug r{_RANK}]" if _RANK else "[EPLB-debug]"

_STATS: "OrderedDict[str, RegionStat]" = OrderedDict()
_WINDOW_STATS: "OrderedDict[str, RegionStat]" = OrderedDict()
_PENDING: List[tuple] = []
_calls = 0
_debug_logger: Optional[Callable[[str], None]] = None


def enabled() -> bool:
    return _ENABLED


def regions_requested() -> bool:
    return _ENABLED or _flag("PROFILE_TRACE")


def debug_enabled() -> bool:
    return _DEBUG_ENABLED


def all_ranks() -> bool:
    """Every rank reports (needed to see max-vs-mean over ranks, i.e. the straggler)."""
    return _ALL_RANKS


def _add_sample(name: str, ms: float, payload_bytes=0) -> None:
    nbytes = _bytes_of(payload_bytes)
    _STATS.setdefault(name, RegionStat()).add(ms, nbytes)
    if _DEBUG_ENABLED:
        _WINDOW_STATS.setdefault(name, RegionStat()).add(ms, nbytes)


def _drain() -> None:
    """Resolve all queued event pairs with one device synchronisation."""
    global _PENDING
    if not _PENDING:
        return
    queued, _PENDING = _PENDING, []
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        for name, start, end, payload in queued:
            _add_sample(name, start.elapsed_time(end), payload)


def _fields(phases: Sequence[Tuple[str, Tuple[str, ...]]], missing: Optional[Mapping[str, str]] = None) -> List[str]:
    out = []
    missing = missing or {}
    for label, names in phases:
        stats = [_WINDOW_STATS[n] for n in names if n in _WINDOW_STATS]
        if not stats:
            if label in missing:
                out.append(f"{label}={missing[label]}")
            continue
        n = sum(s.count for s in stats)
        ms = sum(s.total_ms for s in stats)
        nb = sum(s.total_bytes for s in stats)
        text = f"{label}={ms:.3f}ms" + (f"(x{n})" if n > 1 else "")
        if nb:
            text += f"/{nb / MIB:.2f}MiB/{nb / (max(ms, 1e-12) * 1e6):.2f}GB/s"
        out.append(text)
    return out


def _emit_backward() -> None:
    f = _fields(BACKWARD_PHASES)
    if f and _debug_logger is not None:
        _debug_logger(f"{_DEBUG_PREFIX} mode=apply direction=backward " + " ".join(f))


def begin_debug_window() -> None:
    """Open the timing window of one MoE invocation (debug mode syncs here, by design)."""
    if not _DEBUG_ENABLED:
        return
    _drain()
    _emit_backward()
    _WINDOW_STATS.clear()


@contextlib.contextmanager
def record(name: str, *, time_it: bool = False, device=None, stream=None, payload_bytes=0):
    """Profiler range ``eplb/<name>``; timed when a timing mode is on and ``time_it`` is set.

    ``payload_bytes`` may be an int or a one-element device tensor (read only when drained).
    ``stream`` places the events on a side stream for hand-scheduled transfers.
    """
    with torch.profiler.record_function(f"eplb/{name}"):
        if not (_ENABLED and time_it):
            yield
            return
        on_gpu = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        if on_gpu:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            try:
                yield
            finally:
                end.record(stream)
                _PENDING.append((name, start, end, payload_bytes))
                if len(_PENDING) >= _MAX_PENDING:
                    _drain()
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                _add_sample(name, (time.perf_counter() - t0) * 1e3, payload_bytes)


def last_ms(name: str) -> float:
    _drain()
    s = _STATS.get(name)
    return s.last_ms if s is not None else 0.0


def stats() -> "OrderedDict[str, RegionStat]":
    _drain()
    return _STATS


def reset() -> None:
    global _PENDING, _calls
    _STATS.clear()
    _WINDOW_STATS.clear()
    _PENDING = []
    _calls = 0


def reset_peak_memory() -> None:
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()


def memory_str() -> str:
    if not torch.cuda.is_available():
        return f"{_PREFIX} peak memory: n/a (no CUDA)"
    return (f"{_PREFIX} peak memory  allocated={torch.cuda.max_memory_allocated() / MIB:9.1f} MiB"
            f"   reserved={torch.cuda.max_memory_reserved() / MIB:9.1f} MiB")


def summary_str() -> str:
    _drain()
    if not _STATS:
        return f"{_PREFIX} no samples (set EPLB_PROFILE=1)"
    lines = [f"{_PREFIX} region                 count    mean(ms)   min(ms)   max(ms)  mean(MiB)  payload(GB/s)"]
    for name, s in _STATS.items():
        n = max(s.count, 1)
        lines.append(f"{_PREFIX} {name:<22} {s.count:>6}   {s.total_ms / n:>8.3f}  {s.min_ms:>8.3f}"
                     f"  {s.max_ms:>8.3f}  {s.total_bytes / n / MIB:>9.2f}"
                     f"  {s.total_bytes / (max(s.total_ms, 1e-12) * 1e6):>12.2f}")
    lines.append(memory_str())
    return "\n".join(lines)


def debug_str(context: str = "", *, missing: Optional[Mapping[str, str]] = None) -> str:
    """One invocation's compact breakdown; clears the window."""
    _drain()
    f = _fields(FORWARD_PHASES, missing)
    _WINDOW_STATS.clear()
    where = f" {context}" if context else ""
    return f"{_DEBUG_PREFIX}{where} " + (" ".join(f) if f else "no timing samples")


def maybe_summary(logger: Optional[Callable[[str], None]], *, context: str = "",
                  missing: Optional[Mapping[str, str]] = None) -> None:
    global _calls, _debug_logger
    if not _ENABLED:
        return
    if _DEBUG_ENABLED:
        _debug_logger = logger
        line = debug_str(context, missing=missing)
        if logger is not None:
            logger(line)
    if not _PROFILE_ENABLED or logger is None:
        return
    _calls += 1
    if _PERIOD > 0 and _calls % _PERIOD == 0:
        logger(summary_str())
    if _RESET_AT and _calls == _RESET_AT:
        reset_peak_memory()


def _at_exit() -> None:
    if not _DEBUG_ENABLED:
        return
    try:
        _drain()
        _emit_backward()
        _WINDOW_STATS.clear()
    except Exception:  # CUDA may already be gone at interpreter exit
        pass


atexit.register(_at_exit)
