"""What this machine offers: library versions, GPUs, peer access.

The reference pins its environment with shell scripts that download and build NCCL, Megatron and DeepEP
(scripts/env_nccl_2307.sh, install_*.sh, bootstrap_new_machine.sh) and probes the loaded NCCL through
``/proc/self/maps`` (eplb/integration/eplb_manager.py:39-62).  Nothing is downloaded here; this module only
reports what is present, so that a failed launch can be told apart from a missing capability.
"""

from __future__ import annotations

import ctypes
import os
import re
from typing import Any, Dict, List, Optional


def nccl_runtime_version() -> Optional[str]:
    """Version of the NCCL shared library actually mapped into this process (not the one torch was built
    against): found through ``/proc/self/maps`` and asked with ``ncclGetVersion``.  None when no NCCL is loaded."""
    try:
        with open("/proc/self/maps") as f:
            paths = {line.split()[-1] for line in f if "libnccl" in line and ".so" in line}
    except OSError:
        return None
    for path in sorted(paths):
        try:
            lib = ctypes.CDLL(path)
            v = ctypes.c_int(0)
            if lib.ncclGetVersion(ctypes.byref(v)) == 0 and v.value > 0:
                major, rest = divmod(v.value, 10000)
                minor, patch = divmod(rest, 100)
                return f"{major}.{minor}.{patch}"
        except (OSError, AttributeError):
            continue
    return None


def describe_environment() -> Dict[str, Any]:
    import torch

    info: Dict[str, Any] = {
        "torch": torch.__version__, "cuda_build": torch.version.cuda, "cuda_available": torch.cuda.is_available(),
        "nccl_compiled": ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None,
        "nccl_loaded": nccl_runtime_version(), "gpus": [], "peer_access": None,
    }
    if not torch.cuda.is_available():
        return info
    n = torch.cuda.device_count()
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        info["gpus"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                             "memory_gib": round(p.total_memory / 2 ** 30, 1)})
    info["peer_access"] = [[i == j or bool(torch.cuda.can_device_access_peer(i, j)) for j in range(n)] for i in range(n)]
    info["blackwell"] = all(g["sm"].startswith("10.") for g in info["gpus"])
    return info


def problems(info: Dict[str, Any]) -> List[str]:
    """Reasons why the native path cannot run here (empty list: it can)."""
    out = []
    if not info["cuda_available"]:
        out.append("no CUDA device is visible")
        return out
    if not info.get("blackwell"):
        out.append("the kernels are built for sm_100a only; a visible GPU is not compute capability 10.x")
    pa = info["peer_access"]
    if pa and not all(all(row) for row in pa):
        out.append("not every pair of GPUs has peer access: the symmetric heap needs load/store reachability")
    return out
