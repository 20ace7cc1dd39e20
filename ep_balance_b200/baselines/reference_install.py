"""Locating an installed copy of the upstream package (``pip install --target baseline/_ref``).

The upstream CUDA solver is a JIT extension; when it was pre-built into ``baseline/_ref/_torch_ext`` its
``build.ninja`` records the absolute source path used at build time.  If the tree is later reached
through a different path (a copy, a symlink), importing through the *recorded* path lets ninja see an
up-to-date build instead of recompiling for minutes.
"""

from __future__ import annotations

import os
import sys
from typing import Optional


def locate_reference(repo_root: str) -> Optional[str]:
    """Directory that contains the upstream ``eplb`` package, or None when it is not installed."""
    root = os.path.join(repo_root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(root, "eplb")):
        return None
    ninja = os.path.join(root, "_torch_ext", "_scale_eplb_fast_cuda", "build.ninja")
    try:
        with open(ninja) as f:
            for line in f:
                if "fast_solver.cu" in line and "cuda_compile" in line:
                    src = line.split("cuda_compile", 1)[1].strip()
                    built_root = src.split("/eplb/csrc/")[0]
                    if os.path.isdir(os.path.join(built_root, "eplb")) and os.path.samefile(built_root, root):
                        return built_root
    except OSError:
        pass
    return root


def use_reference(repo_root: str) -> Optional[str]:
    """Put the upstream package on ``sys.path`` and point its extension cache at the pre-built copy."""
    root = locate_reference(repo_root)
    if root is None:
        return None
    os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(root, "_torch_ext"))
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0+PTX")
    if root not in sys.path:
        sys.path.insert(0, root)
    return root
