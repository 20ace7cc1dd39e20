"""Imbalance vs additional replica slots per rank, for every strategy (input of the slot-sweep figure).

    python -m ep_balance_b200.launch.slot_sweep --slots 0 1 2 3 4 --json sweep.json

Reference: scripts/run_slot_sweep.sh:1-85.
"""

from __future__ import annotations

import argparse
import json

from ..baselines import benchmark as bm


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--slots", type=int, nargs="+", default=[1, 2, 3, 4])
    p.add_argument("--strategies", default="scale,eplb,fastermoe,flexmoe")
    p.add_argument("--json", default=None)
    a, rest = p.parse_known_args(argv)
    out = []
    for k in a.slots:
        rows = bm.main(["--n-slot", str(k), "--strategies", a.strategies, "--include-no-balance", *rest])
        out.append({"n_slot": k, "rows": rows})
    if a.json:
        with open(a.json, "w") as f:
            json.dump(out, f)
    return out


if __name__ == "__main__":
    main()
