"""Turn ``[EPLB-debug rN] ...`` log lines into per-phase time budgets.

Ranks interleave their prints, so records are split on the tag, not on newlines.  Each forward
record is ``mode=<m> layer=<l> mb=<k> name=1.234ms(x2)/64.00MiB/31.86GB/s ...``; backward transfer
phases arrive as ``mode=apply direction=backward ...`` at the next invocation boundary and are
attached to the previous forward record of the same rank.  Writes ``rows.csv``, ``by_bucket.csv``,
``by_rank.csv`` and ``summary.json`` under ``--out-dir``.  Reference: eval/extract_eplb_debug.py:45-346.
"""

from __future__ import annotations

import argparse
import csv
import json
import re
import statistics as st
from pathlib import Path
from typing import Any, Dict, List, Tuple

RECORD_SPLIT = re.compile(r"\[EPLB-debug r(\d+)\]\s*")
FORWARD_RE = re.compile(r"mode=(\w+) layer=(\d+) mb=(\d+)")
BACKWARD_RE = re.compile(r"mode=(\w+) direction=backward")
FIELD_RE = re.compile(r"(?P<name>\w+)=(?P<ms>[\d.]+)ms(?:\(x(?P<count>\d+)\))?(?:/(?P<mib>[\d.]+)MiB/(?P<gbps>[\d.]+)GB/s)?")
FORWARD_PHASES = ("solver", "omega_gather", "router", "shared_expert", "expert_transfer", "dispatch", "expert_gemm", "combine")
BACKWARD_PHASES = ("expert_repull", "expert_grad_reduce")
EPLB_ONLY = ("solver", "omega_gather", "expert_transfer", "expert_repull", "expert_grad_reduce")


def parse(paths: List[Path]) -> List[Dict[str, Any]]:
    rows: List[Dict[str, Any]] = []
    last_by_rank: Dict[int, Dict[str, Any]] = {}
    for path in paths:
        text = Path(path).read_text(errors="replace")
        parts = RECORD_SPLIT.split(text)
        for i in range(1, len(parts) - 1, 2):
            rank, body = int(parts[i]), parts[i + 1]
            fields = {m["name"]: m for m in FIELD_RE.finditer(body)}
            fwd = FORWARD_RE.search(body)
            if fwd:
                row = {"rank": rank, "mode": fwd[1], "layer": int(fwd[2]), "mb": int(fwd[3])}
                for name, m in fields.items():
                    row[f"{name}_ms"] = float(m["ms"])
                    if m["mib"]:
                        row[f"{name}_mib"], row[f"{name}_gbps"] = float(m["mib"]), float(m["gbps"])
                rows.append(row)
                last_by_rank[rank] = row
            elif BACKWARD_RE.search(body) and rank in last_by_rank:
                for name, m in fields.items():
                    last_by_rank[rank][f"{name}_ms"] = float(m["ms"])
                    if m["mib"]:
                        last_by_rank[rank][f"{name}_mib"], last_by_rank[rank][f"{name}_gbps"] = float(m["mib"]), float(m["gbps"])
    return rows


def steady(rows: List[Dict[str, Any]], warmup: int) -> List[Dict[str, Any]]:
    return [r for r in rows if r["mb"] >= warmup]


def summarize(rows: List[Dict[str, Any]], warmup: int = 0) -> Dict[str, Any]:
    rows = steady(rows, warmup)
    out: Dict[str, Any] = {"records": len(rows), "phases": {}}
    for ph in FORWARD_PHASES + BACKWARD_PHASES:
        vals = [r[f"{ph}_ms"] for r in rows if f"{ph}_ms" in r]
        if vals:
            bw = [r[f"{ph}_gbps"] for r in rows if f"{ph}_gbps" in r]
            out["phases"][ph] = {"mean_ms": st.fmean(vals), "p50_ms": st.median(vals), "max_ms": max(vals), "n": len(vals),
                                 **({"mean_gbps": st.fmean(bw)} if bw else {})}
    tot = sum(p["mean_ms"] for p in out["phases"].values())
    out["mean_total_ms"] = tot
    out["eplb_only_ms"] = sum(out["phases"][p]["mean_ms"] for p in EPLB_ONLY if p in out["phases"])
    return out


def by_key(rows, key_fn) -> List[Dict[str, Any]]:
    groups: Dict[Any, List[Dict[str, Any]]] = {}
    for r in rows:
        groups.setdefault(key_fn(r), []).append(r)
    table = []
    for k in sorted(groups):
        entry = {"key": k, "records": len(groups[k])}
        for ph in FORWARD_PHASES + BACKWARD_PHASES:
            vals = [r[f"{ph}_ms"] for r in groups[k] if f"{ph}_ms" in r]
            if vals:
                entry[f"{ph}_ms"] = st.fmean(vals)
        table.append(entry)
    return table


def write_csv(rows: List[Dict[str, Any]], path: Path) -> None:
    cols: List[str] = []
    for r in rows:
        cols += [c for c in r if c not in cols]
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=cols)
        w.writeheader()
        w.writerows(rows)


def main(argv=None) -> Dict[str, Any]:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--log", required=True, type=Path, nargs="+")
    p.add_argument("--out-dir", required=True, type=Path)
    p.add_argument("--warmup", type=int, default=0, help="drop records whose micro-batch index is below this")
    p.add_argument("--bucket", type=int, default=250)
    a = p.parse_args(argv)
    rows = parse(a.log)
    a.out_dir.mkdir(parents=True, exist_ok=True)
    write_csv(rows, a.out_dir / "rows.csv")
    write_csv(by_key(steady(rows, a.warmup), lambda r: r["mb"] // a.bucket * a.bucket), a.out_dir / "by_bucket.csv")
    write_csv(by_key(steady(rows, a.warmup), lambda r: r["rank"]), a.out_dir / "by_rank.csv")
    summary = summarize(rows, a.warmup)
    (a.out_dir / "summary.json").write_text(json.dumps(summary, indent=1))
    return summary


if __name__ == "__main__":
    print(json.dumps(main(), indent=1))
