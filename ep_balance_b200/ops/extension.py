"""In-tree build of the native extension for sm_100a.

The shared object is written to ``ep_balance_b200/ops/_build`` so that it travels with the source
tree.  ``load()`` imports an existing build whose source stamp matches and only invokes the
compiler otherwise; there is no silent Python fallback -- on a CUDA machine a missing or broken
extension is an error.
"""

from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
from pathlib import Path
from types import ModuleType
from typing import Optional

NAME = "_epb_C"
HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD_DIR = HERE / "_build"
SOURCES = ["binding.cpp", "solver.cu", "route.cu", "grouped_gemm.cu", "runtime.cu", "optim.cu"]
CUDA_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "--expt-relaxed-constexpr"]

_module: Optional[ModuleType] = None


def _optional_sources() -> list:
    return [p.name for p in sorted(CSRC.glob("*.cu")) if p.name not in SOURCES]


def source_stamp() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.iterdir()):
        if p.suffix in (".cu", ".cuh", ".h", ".cpp"):
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join(CUDA_FLAGS).encode())
    return h.hexdigest()


def _so_path() -> Path:
    return BUILD_DIR / f"{NAME}.so"


def _import_built() -> ModuleType:
    spec = importlib.util.spec_from_file_location(NAME, _so_path())
    mod = importlib.util.module_from_spec(spec)
    sys.modules[NAME] = mod
    spec.loader.exec_module(mod)
    return mod


def build(verbose: bool = bool(int(os.environ.get("EPLB_CUDA_BUILD_VERBOSE", "0") or 0))) -> ModuleType:
    """Compile every source for sm_100a (no GPU needed) and import the result."""
    import torch  # noqa: F401  (must be imported before the extension)
    from torch.utils.cpp_extension import load

    BUILD_DIR.mkdir(exist_ok=True)
    # the arch comes from -gencode above; keep torch from adding its own list
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    sources = [str(CSRC / s) for s in SOURCES + _optional_sources()]
    mod = load(name=NAME, sources=sources, build_directory=str(BUILD_DIR), extra_cuda_cflags=CUDA_FLAGS,
               extra_cflags=["-O3", "-std=c++17"], extra_include_paths=[str(CSRC)], verbose=verbose)
    (BUILD_DIR / "stamp").write_text(source_stamp())
    return mod


def load() -> ModuleType:
    """Import the extension, building it when the in-tree binary is absent or stale."""
    global _module
    if _module is not None:
        return _module
    import torch  # noqa: F401

    stamp = BUILD_DIR / "stamp"
    if _so_path().exists() and stamp.exists() and stamp.read_text() == source_stamp():
        _module = _import_built()
    else:
        _module = build()
    return _module
