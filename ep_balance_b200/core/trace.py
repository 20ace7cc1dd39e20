"""Routing-trace files: the one persisted artefact of the balancer.

A trace is ``torch.save({"meta": {...}, "samples": [...]})`` with
``meta.format_version == 3`` (reference writer: eplb/integration/megatron.py:161-214,
reader: eplb/trace_analysis.py:12-228).  ``meta.n_slot`` is the TOTAL slot count
per rank.  Older files that call the matrix ``lam`` are accepted.
"""

from __future__ import annotations

import os
import tempfile
from collections import defaultdict
from pathlib import Path
from typing import Dict, Iterable, List, Tuple, Union

import torch

OMEGA_SEMANTICS = "source_ep_rank_by_logical_expert_token_assignments"
TRACE_FORMAT_VERSION = 3


# ---------------------------------------------------------------- writing

def build_trace_meta(topo, spec, *, counts_reduced_over_tp_cp: bool = False) -> dict:
    """Header from which a replay can rebuild the exact Topology and ProblemSpec."""
    return {
        "format_version": TRACE_FORMAT_VERSION,
        "num_ranks": topo.num_ranks,
        "num_experts": int(spec.num_experts),
        "omega_semantics": OMEGA_SEMANTICS,
        "counts_reduced_over_tp_cp": bool(counts_reduced_over_tp_cp),
        "s_tok": int(spec.s_tok),
        "n_slot": int(spec.n_slot),
        "num_domains": topo.num_domains,
        "main_rank": spec.main_rank.detach().cpu().clone(),
        "weight_bytes": spec.weight_bytes.detach().cpu().clone(),
        "domain_of_rank": topo.domain_of_rank.detach().cpu().clone(),
        "cost": topo.cost.detach().cpu().clone(),
    }


def save_trace(path: Union[str, Path], meta: dict, samples: List[dict]) -> None:
    """Write to a temporary file in the target directory, then rename (atomic on POSIX)."""
    path = os.fspath(path)
    out_dir = os.path.dirname(path) or "."
    os.makedirs(out_dir, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=out_dir, suffix=".tmp")
    os.close(fd)
    try:
        torch.save({"meta": meta, "samples": samples}, tmp)
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.unlink(tmp)


class TraceWriter:
    """Accumulates ``omega`` samples and flushes every ``every`` additions."""

    def __init__(self, path: str, meta: dict, *, max_samples: int = 0, every: int = 25) -> None:
        self.path = path
        self.meta = meta
        self.max_samples = int(max_samples)
        self.every = max(1, int(every))
        self.samples: List[dict] = []
        self._dirty = 0
        self._ordinal = 0

    def add(self, layer: int, mb: int, omega: torch.Tensor) -> bool:
        if self.max_samples and len(self.samples) >= self.max_samples:
            return False
        self.samples.append({
            "layer": int(layer), "mb": int(mb), "ordinal": self._ordinal,
            "omega": omega.detach().to("cpu", torch.int64).clone(),
        })
        self._ordinal += 1
        self._dirty += 1
        if self._dirty >= self.every:
            self.flush()
        return True

    def flush(self) -> None:
        if self.samples:
            save_trace(self.path, self.meta, self.samples)
            self._dirty = 0


# ---------------------------------------------------------------- reading

def load_routing_trace(path: Union[str, Path]) -> dict:
    trace = torch.load(Path(path), map_location="cpu", weights_only=False)
    if not isinstance(trace, dict) or not isinstance(trace.get("meta"), dict):
        raise ValueError(f"{path}: expected a trace dict with a 'meta' mapping")
    samples = trace.get("samples")
    if not isinstance(samples, list) or not samples:
        raise ValueError(f"{path}: trace has no samples")
    shape = (int(trace["meta"]["num_ranks"]), int(trace["meta"]["num_experts"]))
    for i, s in enumerate(samples):
        if not isinstance(s, dict) or "layer" not in s or ("omega" not in s and "lam" not in s):
            raise ValueError(f"{path}: malformed sample {i}")
        if "omega" not in s:
            s["omega"] = s["lam"]
        om = torch.as_tensor(s["omega"])
        if tuple(om.shape) != shape:
            raise ValueError(f"{path}: sample {i} Ω shape {tuple(om.shape)} != {shape}")
        if bool((om < 0).any()):
            raise ValueError(f"{path}: sample {i} contains negative token counts")
    return trace


def spec_and_topology_from_meta(meta: dict):
    """Rebuild ``(Topology, ProblemSpec)`` from a trace header."""
    from .problem import ProblemSpec
    from .topology import Topology

    R, E = int(meta["num_ranks"]), int(meta["num_experts"])
    main_rank = resolve_main_rank(meta)
    if "domain_of_rank" in meta:
        dom = torch.as_tensor(meta["domain_of_rank"], dtype=torch.int64)
        cost = torch.as_tensor(meta["cost"], dtype=torch.int64)
        topo = Topology(dom, cost, num_domains_hint=int(meta.get("num_domains", int(dom.max()) + 1)))
    else:
        nd = int(meta.get("num_domains", 1))
        topo = Topology.from_nvlink_rdma(nd, R // nd)
    wb = meta.get("weight_bytes")
    wb = torch.as_tensor(wb, dtype=torch.int64) if wb is not None else torch.ones(E, dtype=torch.int64)
    spec = ProblemSpec(E, main_rank, wb, int(meta.get("s_tok", 1)), int(meta["n_slot"]))
    return topo, spec


def expert_counts_by_layer(trace: dict) -> Dict[int, List[torch.Tensor]]:
    """``{layer: [counts[E] in capture order]}``."""
    bucket: Dict[int, List[Tuple[int, torch.Tensor]]] = defaultdict(list)
    for pos, s in enumerate(trace["samples"]):
        counts = torch.as_tensor(s["omega"], dtype=torch.int64).sum(0)
        bucket[int(s["layer"])].append((int(s.get("ordinal", pos)), counts))
    return {layer: [c for _, c in sorted(items, key=lambda it: it[0])] for layer, items in bucket.items()}


def _common_occurrences(grouped: Dict[int, List[torch.Tensor]], max_occurrences: int) -> int:
    if max_occurrences < 0:
        raise ValueError("max_occurrences must be non-negative")
    n = min(len(v) for v in grouped.values())
    return min(n, max_occurrences) if max_occurrences else n


def expert_count_cube(trace: dict, *, max_occurrences: int = 0) -> Tuple[List[int], torch.Tensor]:
    """Counts as ``[layer, occurrence, expert]`` over the occurrences every layer has."""
    if max_occurrences < 0:
        raise ValueError("max_occurrences must be non-negative")
    grouped = expert_counts_by_layer(trace)
    layers = sorted(grouped)
    n = _common_occurrences(grouped, max_occurrences)
    if n <= 0:
        raise ValueError("trace has no complete layer occurrences")
    return layers, torch.stack([torch.stack(grouped[l][:n]) for l in layers])


def _ratio(mx: torch.Tensor, mean: torch.Tensor) -> torch.Tensor:
    return torch.where(mean > 0, mx / mean, torch.zeros_like(mean))


def expert_max_mean_by_layer(trace: dict, *, max_occurrences: int = 0):
    """``(layers, per-occurrence max/mean [L, O], aggregate max/mean [L])``."""
    layers, cube = expert_count_cube(trace, max_occurrences=max_occurrences)
    cube = cube.to(torch.float64)
    per = _ratio(cube.max(-1).values, cube.mean(-1))
    agg = cube.sum(1)
    return layers, per, _ratio(agg.max(-1).values, agg.mean(-1))


def select_expert_count_matrix(trace: dict, *, view: str, occurrence: int = 0,
                               max_occurrences: int = 0) -> Tuple[List[int], torch.Tensor]:
    """``[layer, expert]`` counts of one occurrence (``snapshot``) or summed (``aggregate``)."""
    if view not in ("snapshot", "aggregate"):
        raise ValueError("view must be 'snapshot' or 'aggregate'")
    grouped = expert_counts_by_layer(trace)
    layers = sorted(grouped)
    n = _common_occurrences(grouped, max_occurrences)
    rows = []
    for layer in layers:
        vals = grouped[layer]
        if view == "snapshot":
            if not -len(vals) <= occurrence < len(vals):
                raise ValueError(f"layer {layer} has {len(vals)} occurrences, cannot select {occurrence}")
            rows.append(vals[occurrence])
        else:
            if not vals[:n]:
                raise ValueError(f"layer {layer} has no selected occurrences")
            rows.append(torch.stack(vals[:n]).sum(0))
    return layers, torch.stack(rows)


def normalize_expert_counts(counts: torch.Tensor, mode: str) -> torch.Tensor:
    v = counts.to(torch.float64)
    if mode == "share":
        return v / v.sum(1, keepdim=True).clamp_min(1)
    if mode == "relative":
        return v / v.mean(1, keepdim=True).clamp_min(1)
    if mode == "count":
        return v
    raise ValueError("normalization mode must be share, relative, or count")


def resolve_main_rank(meta: dict) -> torch.Tensor:
    R, E = int(meta["num_ranks"]), int(meta["num_experts"])
    if "main_rank" in meta:
        mr = torch.as_tensor(meta["main_rank"], dtype=torch.int64)
    else:
        if E % R:
            raise ValueError("trace lacks main_rank and experts are not evenly divisible by ranks")
        mr = torch.arange(E, dtype=torch.int64) // (E // R)
    if tuple(mr.shape) != (E,):
        raise ValueError(f"main_rank shape {tuple(mr.shape)} != ({E},)")
    if bool((mr < 0).any()) or bool((mr >= R).any()):
        raise ValueError("main_rank contains a rank outside the trace topology")
    return mr


def rank_loads_from_expert_counts(counts: torch.Tensor, meta: dict) -> torch.Tensor:
    """Receiving-rank load per row of ``counts`` if every expert is served only by its owner."""
    mr = resolve_main_rank(meta).to(counts.device)
    out = counts.new_zeros((counts.shape[0], int(meta["num_ranks"])))
    out.index_add_(1, mr, counts)
    return out


def _max_over_mean(v: torch.Tensor) -> float:
    m = v.to(torch.float64).mean()
    return float(v.max().to(torch.float64) / m) if m > 0 else 0.0


def metric_rows(*, label: str, view: str, layers: Iterable[int], expert_counts: torch.Tensor,
                meta: dict) -> List[dict]:
    ranks = rank_loads_from_expert_counts(expert_counts, meta)
    rows = []
    for i, layer in enumerate(layers):
        ex, rk = expert_counts[i], ranks[i]
        total = int(ex.sum())
        he = int(ex.argmax()) if total else -1
        rows.append({
            "label": label, "view": view, "layer": int(layer), "total_assignments": total,
            "expert_max_mean": _max_over_mean(ex), "rank_max_mean": _max_over_mean(rk),
            "hot_expert": he,
            "hot_expert_share": float(ex[he].to(torch.float64) / total) if total else 0.0,
            "hot_rank": int(rk.argmax()) if total else -1,
        })
    return rows
