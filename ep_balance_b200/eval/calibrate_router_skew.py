"""Which synthetic router skew gives which imbalance?

Offline model of a biased router: ``logits[t, e] = N(0, 1) + b[e]`` with ``b ~ N(0, |std|)`` drawn
per expert (``iid``) or per owner rank (``block``); top-k counts give the expert max/mean and,
under the contiguous owner placement ``main(e) = e // (E/R)``, the rank max/mean over ``draws``
independent bias draws.  ``--target`` bisects ``|std|`` for a wanted median rank imbalance.
Reference: eval/calibrate_router_skew.py:44-212.

    python -m ep_balance_b200.eval.calibrate_router_skew --experts 128 --topk 8 --ranks 32 --target 2.5
"""

from __future__ import annotations

import argparse
import json
from typing import Any, Dict, List, Optional, Sequence

import torch

DEFAULT_STDS = (0.0, 0.1, 0.2, 0.3, 0.5, 0.75, 1.0, 1.5, 2.0, 3.0)


def draw_bias(std: float, num_experts: int, main_rank: torch.Tensor, mode: str) -> torch.Tensor:
    if mode == "iid":
        return torch.empty(num_experts).normal_(std=abs(std)) if std else torch.zeros(num_experts)
    if mode == "block":
        per_rank = torch.empty(int(main_rank.max()) + 1).normal_(std=abs(std)) if std else torch.zeros(int(main_rank.max()) + 1)
        return per_rank[main_rank]
    raise ValueError("bias mode must be 'iid' or 'block'")


def realise(std: float, *, num_experts: int, topk: int, main_rank: torch.Tensor, num_ranks: int, tokens: int,
            draws: int, mode: str) -> Dict[str, torch.Tensor]:
    ex, rk = torch.empty(draws), torch.empty(draws)
    for i in range(draws):
        bias = draw_bias(std, num_experts, main_rank, mode)
        chosen = (torch.randn(tokens, num_experts) + bias).topk(topk, dim=-1).indices
        counts = torch.bincount(chosen.reshape(-1), minlength=num_experts).double()
        load = torch.zeros(num_ranks, dtype=torch.float64).index_add_(0, main_rank, counts)
        ex[i], rk[i] = counts.max() / counts.mean(), load.max() / load.mean()
    return {"expert_max_mean": ex, "rank_max_mean": rk}


def quantiles(v: torch.Tensor) -> Dict[str, float]:
    v = v.double()
    p10, p50, p90 = torch.quantile(v, torch.tensor([0.1, 0.5, 0.9], dtype=v.dtype)).tolist()
    return {"p10": round(p10, 4), "median": round(p50, 4), "p90": round(p90, 4), "max": round(float(v.max()), 4)}


def sweep(stds: Sequence[float], **kw: Any) -> List[Dict[str, Any]]:
    rows = []
    for std in stds:
        got = realise(std, **kw)
        rows.append({"std": std, "router_skew_stationary": -abs(std) if std else 0.0,
                     "expert_max_mean": quantiles(got["expert_max_mean"]), "rank_max_mean": quantiles(got["rank_max_mean"])})
    return rows


def solve_for_target(target: float, tolerance: float, **kw: Any) -> Optional[Dict[str, Any]]:
    lo, hi = 0.0, 4.0
    if float(torch.quantile(realise(hi, **kw)["rank_max_mean"], 0.5)) < target:
        return None
    best = None
    for _ in range(18):
        mid = 0.5 * (lo + hi)
        got = realise(mid, **kw)
        med = float(torch.quantile(got["rank_max_mean"], 0.5))
        best = {"router_skew": round(-mid, 4), "rank_max_mean": quantiles(got["rank_max_mean"]),
                "expert_max_mean": quantiles(got["expert_max_mean"])}
        if abs(med - target) <= tolerance:
            break
        lo, hi = (mid, hi) if med < target else (lo, mid)
    return best


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--experts", type=int, default=128)
    p.add_argument("--topk", type=int, default=8)
    p.add_argument("--ranks", type=int, default=32)
    p.add_argument("--tokens", type=int, default=8192)
    p.add_argument("--draws", type=int, default=16)
    p.add_argument("--bias-mode", default="iid", choices=["iid", "block"])
    p.add_argument("--stds", type=float, nargs="*", default=list(DEFAULT_STDS))
    p.add_argument("--target", type=float, default=None, help="median rank max/mean to solve for")
    p.add_argument("--tolerance", type=float, default=0.05)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--json", action="store_true")
    a = p.parse_args(argv)
    if a.experts % a.ranks:
        raise SystemExit("--experts must be divisible by --ranks")
    torch.manual_seed(a.seed)
    main_rank = torch.arange(a.experts) // (a.experts // a.ranks)
    kw = dict(num_experts=a.experts, topk=a.topk, main_rank=main_rank, num_ranks=a.ranks, tokens=a.tokens,
              draws=a.draws, mode=a.bias_mode)
    out: Dict[str, Any] = {"sweep": sweep(a.stds, **kw)}
    if a.target is not None:
        out["target"] = {"wanted": a.target, "solution": solve_for_target(a.target, a.tolerance, **kw)}
    if a.json:
        print(json.dumps(out))
    else:
        print(f"{'std':>6}  {'ROUTER_SKEW':>11}  {'rank max/mean (p10/med/p90)':^30}  {'expert max/mean (med)':^22}")
        for r in out["sweep"]:
            rk, ex = r["rank_max_mean"], r["expert_max_mean"]
            print(f"{r['std']:>6.2f}  {r['router_skew_stationary']:>11.2f}  {rk['p10']:>8.2f} {rk['median']:>8.2f} {rk['p90']:>8.2f}      {ex['median']:>10.2f}")
        if a.target is not None:
            print("target:", json.dumps(out["target"]))
    return out


if __name__ == "__main__":
    main()
