"""Figures for routing traces, slot sweeps and solver scaling (headless matplotlib ``Agg``).

    python -m ep_balance_b200.eval.plots hotspots        --trace t.pt --out fig.png
    python -m ep_balance_b200.eval.plots max-mean        --trace a.pt b.pt --out fig.png
    python -m ep_balance_b200.eval.plots max-mean-layer  --trace t.pt --out fig.png
    python -m ep_balance_b200.eval.plots hotspots-mm     --trace t.pt --out fig.png
    python -m ep_balance_b200.eval.plots slot-sweep      --json sweep.json --out fig.png
    python -m ep_balance_b200.eval.plots solver-scaling  --json scaling.json --out fig.png
    python -m ep_balance_b200.eval.plots transport       --out fig.png

Every command first computes the plotted numbers and writes them next to the figure as
``<out>.json``; the image itself needs matplotlib and is skipped with a note when it is missing.
Reference: eval/plot_*.py (seven separate CLIs there).
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Any, Dict, List, Optional

import torch

from ..core.trace import (expert_max_mean_by_layer, load_routing_trace, normalize_expert_counts,
                          rank_loads_from_expert_counts, select_expert_count_matrix)


def _plt():
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt

        return plt
    except Exception:
        return None


def _save(data: Dict[str, Any], out: Path, draw) -> Dict[str, Any]:
    out = Path(out)
    out.parent.mkdir(parents=True, exist_ok=True)
    Path(str(out) + ".json").write_text(json.dumps(data))
    plt = _plt()
    if plt is None:
        data["figure"] = "skipped: matplotlib is not installed"
        return data
    fig = draw(plt)
    fig.savefig(out, dpi=150, bbox_inches="tight")
    plt.close(fig)
    data["figure"] = str(out)
    return data


def hotspots(trace_path, out, view="aggregate", occurrence=0, normalize="share") -> Dict[str, Any]:
    trace = load_routing_trace(trace_path)
    layers, counts = select_expert_count_matrix(trace, view=view, occurrence=occurrence)
    grid = normalize_expert_counts(counts, normalize)
    data = {"layers": layers, "normalize": normalize, "grid": grid.tolist()}

    def draw(plt):
        fig, ax = plt.subplots(figsize=(10, 4))
        im = ax.imshow(grid.numpy(), aspect="auto", cmap="magma")
        ax.set_xlabel("logical expert")
        ax.set_ylabel("MoE layer")
        ax.set_yticks(range(len(layers)), [str(l) for l in layers])
        fig.colorbar(im, ax=ax, label=normalize)
        return fig

    return _save(data, out, draw)


def max_mean(trace_paths: List[str], out, labels: Optional[List[str]] = None) -> Dict[str, Any]:
    series = []
    for i, tp in enumerate(trace_paths):
        layers, per, agg = expert_max_mean_by_layer(load_routing_trace(tp))
        series.append({"label": (labels or [Path(p).stem for p in trace_paths])[i], "layers": layers,
                       "mean": per.mean(1).tolist(), "aggregate": agg.tolist()})
    data = {"series": series}

    def draw(plt):
        fig, ax = plt.subplots(figsize=(8, 4))
        for s in series:
            ax.plot(s["layers"], s["mean"], marker="o", label=s["label"])
        ax.set_xlabel("MoE layer")
        ax.set_ylabel("expert max / mean")
        ax.legend()
        return fig

    return _save(data, out, draw)


def max_mean_by_layer(trace_path, out) -> Dict[str, Any]:
    layers, per, agg = expert_max_mean_by_layer(load_routing_trace(trace_path))
    q = torch.quantile(per, torch.tensor([0.1, 0.5, 0.9], dtype=per.dtype), dim=1)
    data = {"layers": layers, "p10": q[0].tolist(), "median": q[1].tolist(), "p90": q[2].tolist(),
            "mean": per.mean(1).tolist(), "aggregate": agg.tolist()}

    def draw(plt):
        fig, ax = plt.subplots(figsize=(8, 4))
        ax.fill_between(layers, data["p10"], data["p90"], alpha=0.3, label="P10-P90")
        ax.plot(layers, data["mean"], marker="o", label="mean over occurrences")
        ax.set_xlabel("MoE layer")
        ax.set_ylabel("expert max / mean")
        ax.legend()
        return fig

    return _save(data, out, draw)


def hotspots_with_max_mean(trace_path, out) -> Dict[str, Any]:
    trace = load_routing_trace(trace_path)
    layers, counts = select_expert_count_matrix(trace, view="aggregate")
    share = normalize_expert_counts(counts, "share")
    ranks = rank_loads_from_expert_counts(counts, trace["meta"]).double()
    data = {"layers": layers, "share": share.tolist(),
            "expert_max_mean": (counts.double().max(1).values / counts.double().mean(1)).tolist(),
            "rank_max_mean": (ranks.max(1).values / ranks.mean(1)).tolist()}

    def draw(plt):
        fig, (a, b) = plt.subplots(1, 2, figsize=(12, 4), gridspec_kw={"width_ratios": [3, 1]})
        a.imshow(share.numpy(), aspect="auto", cmap="magma")
        a.set_xlabel("logical expert")
        a.set_ylabel("MoE layer")
        b.plot(data["expert_max_mean"], range(len(layers)), label="expert")
        b.plot(data["rank_max_mean"], range(len(layers)), label="rank")
        b.invert_yaxis()
        b.legend()
        return fig

    return _save(data, out, draw)


def slot_sweep(json_path, out) -> Dict[str, Any]:
    """Input: ``[{"n_slot": k, "rows": [<benchmark rows>]}...]`` as written by ``launch/slot_sweep.py``."""
    sweep = json.loads(Path(json_path).read_text())
    by: Dict[str, List] = {}
    for point in sweep:
        for r in point["rows"]:
            if "quality_imbalance" in r:
                by.setdefault(r["strategy"], []).append((point["n_slot"], r["quality_imbalance"]))
    data = {"series": {k: sorted(v) for k, v in by.items()}}

    def draw(plt):
        fig, ax = plt.subplots(figsize=(6, 4))
        for k, v in data["series"].items():
            ax.plot([p[0] for p in v], [p[1] for p in v], marker="o", label=k)
        ax.set_xlabel("additional replica slots per rank")
        ax.set_ylabel("rank load max / mean")
        ax.legend()
        return fig

    return _save(data, out, draw)


def solver_scaling(json_path, out) -> Dict[str, Any]:
    """Input: ``[{"sweep": "ranks"|"experts", "x": value, "min_us": t}...]`` from ``launch/solver_scaling.py``."""
    pts = json.loads(Path(json_path).read_text())
    data = {"ranks": sorted((p["x"], p["min_us"]) for p in pts if p["sweep"] == "ranks"),
            "experts": sorted((p["x"], p["min_us"]) for p in pts if p["sweep"] == "experts")}

    def draw(plt):
        fig, (a, b) = plt.subplots(1, 2, figsize=(10, 4))
        for ax, key in ((a, "ranks"), (b, "experts")):
            ax.plot([p[0] for p in data[key]], [p[1] for p in data[key]], marker="o")
            ax.set_xlabel(key)
            ax.set_ylabel("solver min (us)")
            ax.set_xscale("log", base=2)
        return fig

    return _save(data, out, draw)


def transport_schematic(out) -> Dict[str, Any]:
    """Replica weight channel of this framework: owners' home slots, replica slots, gradient slots."""
    data = {"regions": ["home slots [0, E/R): the parameters", "replica slots [E/R, w_slots): pulled by peer loads",
                        "gradient slots: Wgrad target; owner adds replicas' slots with peer loads"],
            "barriers": ["after dispatch + pull", "after GEMM2 scatter", "after gradient dispatch", "after Dgrad1 scatter"]}

    def draw(plt):
        fig, ax = plt.subplots(figsize=(8, 3))
        ax.axis("off")
        for i, text in enumerate(data["regions"]):
            ax.text(0.02, 0.85 - 0.3 * i, text, fontsize=10, bbox=dict(boxstyle="round", fc="#dde"))
        return fig

    return _save(data, out, draw)


def main(argv=None) -> Dict[str, Any]:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = p.add_subparsers(dest="cmd", required=True)
    for name in ("hotspots", "max-mean-layer", "hotspots-mm"):
        s = sub.add_parser(name)
        s.add_argument("--trace", required=True)
        s.add_argument("--out", required=True)
        if name == "hotspots":
            s.add_argument("--view", default="aggregate", choices=["aggregate", "snapshot"])
            s.add_argument("--occurrence", type=int, default=0)
            s.add_argument("--normalize", default="share", choices=["share", "relative", "count"])
    s = sub.add_parser("max-mean")
    s.add_argument("--trace", required=True, nargs="+")
    s.add_argument("--label", nargs="*")
    s.add_argument("--out", required=True)
    for name in ("slot-sweep", "solver-scaling"):
        s = sub.add_parser(name)
        s.add_argument("--json", required=True)
        s.add_argument("--out", required=True)
    sub.add_parser("transport").add_argument("--out", required=True)
    a = p.parse_args(argv)
    if a.cmd == "hotspots":
        return hotspots(a.trace, a.out, a.view, a.occurrence, a.normalize)
    if a.cmd == "max-mean":
        return max_mean(a.trace, a.out, a.label)
    if a.cmd == "max-mean-layer":
        return max_mean_by_layer(a.trace, a.out)
    if a.cmd == "hotspots-mm":
        return hotspots_with_max_mean(a.trace, a.out)
    if a.cmd == "slot-sweep":
        return slot_sweep(a.json, a.out)
    if a.cmd == "solver-scaling":
        return solver_scaling(a.json, a.out)
    return transport_schematic(a.out)


if __name__ == "__main__":
    print(main().get("figure"))
