"""Print what this machine offers and whether the native path can run on it.

    python -m ep_balance_b200.launch.env_check [--json]

Counterpart of the reference's bootstrap scripts, minus the downloads: versions of torch / CUDA / NCCL (built
against and actually loaded), the GPUs, their peer-access matrix, and whether the in-tree extension builds.
"""

from __future__ import annotations

import argparse
import json


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--build", action="store_true", help="also compile the extension if it is stale")
    a = ap.parse_args(argv)
    from ..utils.env import describe_environment, problems

    info = describe_environment()
    info["problems"] = problems(info)
    if a.build:
        try:
            from ..ops.extension import build

            build()
            info["extension"] = "built"
        except Exception as exc:  # report, do not raise: this is a diagnostic tool
            info["extension"] = f"build failed: {exc}"
    if a.json:
        print(json.dumps(info, indent=1))
    else:
        for k in ("torch", "cuda_build", "nccl_compiled", "nccl_loaded", "extension"):
            if k in info:
                print(f"{k:>14}: {info[k]}")
        for g in info["gpus"]:
            print(f"{'gpu ' + str(g['index']):>14}: {g['name']}, sm_{g['sm'].replace('.', '')}, {g['sms']} SMs, {g['memory_gib']} GiB")
        print(f"{'verdict':>14}: " + ("ok" if not info["problems"] else "; ".join(info["problems"])))
    return 0 if not info["problems"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
