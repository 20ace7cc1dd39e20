"""Raw routing imbalance per (layer, micro-batch) from a routing trace, joined with what the
balancer left over (``[EPLB] layer= mb= theta= imbalance= ...`` log lines).

``absorbed = (rank_max_mean - residual) / (rank_max_mean - 1)``: the share of the excess over a
perfectly flat load that replication removed.  Reference: eval/extract_routing_imbalance.py:51-341.
"""

from __future__ import annotations

import argparse
import csv
import json
import re
import statistics as st
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..core.trace import load_routing_trace, resolve_main_rank

EPLB_LINE = re.compile(r"\[EPLB\] layer=(?P<layer>\d+) mb=(?P<mb>\d+) theta=(?P<theta>\d+) "
                       r"imbalance=(?P<imbalance>[\d.]+) replicas=(?P<replicas>\d+) phi_token=(?P<phi_token>\d+)")


def _mm(v: torch.Tensor) -> float:
    m = v.double().mean()
    return float(v.double().max() / m) if m > 0 else 0.0


def raw_rows(trace: dict) -> List[Dict[str, Any]]:
    main_rank = resolve_main_rank(trace["meta"])
    R = int(trace["meta"]["num_ranks"])
    rows = []
    for s in trace["samples"]:
        om = torch.as_tensor(s["omega"], dtype=torch.int64)
        per_e = om.sum(0)
        rank_load = torch.zeros(R, dtype=torch.int64).index_add_(0, main_rank, per_e)
        rows.append({"layer": int(s["layer"]), "mb": int(s.get("mb", 0)), "tokens": int(om.sum()),
                     "expert_max_mean": _mm(per_e), "rank_max_mean": _mm(rank_load), "source_max_mean": _mm(om.sum(1)),
                     "hot_expert": int(per_e.argmax()), "hot_rank": int(rank_load.argmax())})
    return rows


def residuals(log_paths: List[Path]) -> Dict[Tuple[int, int], Dict[str, float]]:
    out: Dict[Tuple[int, int], Dict[str, float]] = {}
    for p in log_paths:
        for m in EPLB_LINE.finditer(Path(p).read_text(errors="replace")):
            out[(int(m["layer"]), int(m["mb"]))] = {"theta": int(m["theta"]), "residual": float(m["imbalance"]),
                                                    "replicas": int(m["replicas"]), "phi_token": int(m["phi_token"])}
    return out


def join(rows: List[Dict[str, Any]], res: Dict[Tuple[int, int], Dict[str, float]]) -> List[Dict[str, Any]]:
    for r in rows:
        hit = res.get((r["layer"], r["mb"]))
        if hit:
            r.update(hit)
            excess = r["rank_max_mean"] - 1.0
            r["absorbed"] = (r["rank_max_mean"] - hit["residual"]) / excess if excess > 1e-9 else 1.0
    return rows


def summarize(rows: List[Dict[str, Any]]) -> Dict[str, Any]:
    def agg(key):
        v = [r[key] for r in rows if key in r]
        return {"mean": st.fmean(v), "p50": st.median(v), "max": max(v), "n": len(v)} if v else None

    return {k: agg(k) for k in ("expert_max_mean", "rank_max_mean", "source_max_mean", "residual", "absorbed")}


def main(argv=None) -> Dict[str, Any]:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--trace", required=True, type=Path)
    p.add_argument("--log", type=Path, nargs="*", default=[])
    p.add_argument("--out-dir", type=Path, default=None)
    a = p.parse_args(argv)
    rows = join(raw_rows(load_routing_trace(a.trace)), residuals(a.log))
    summary = summarize(rows)
    if a.out_dir:
        a.out_dir.mkdir(parents=True, exist_ok=True)
        cols: List[str] = []
        for r in rows:
            cols += [c for c in r if c not in cols]
        with open(a.out_dir / "routing_imbalance.csv", "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=cols)
            w.writeheader()
            w.writerows(rows)
        (a.out_dir / "summary.json").write_text(json.dumps(summary, indent=1))
    return {"rows": rows, "summary": summary}


if __name__ == "__main__":
    print(json.dumps(main()["summary"], indent=1))
