#!/usr/bin/env bash
# Bring a machine to the point where this framework runs (counterpart of the reference's
# scripts/bootstrap_new_machine.sh, install_megatron.sh and env_nccl_2307.sh, for a stack that needs no clones):
#   1. report torch / CUDA / NCCL (compiled and loaded) / GPUs / peer access and what is wrong with them,
#   2. compile the native extension in-tree for sm_100a (nvcc cross-compiles without a GPU),
#   3. with REFERENCE_SRC=<path to an EP_balance checkout>: install the unmodified reference arm of bench.py into
#      baseline/_ref from a local wheelhouse (WHEELHOUSE, default /opt/wheelhouse), offline,
#   4. with a GPU present: one tiny forward + backward of the fused layer, then the CPU test-suite's smoke subset.
# Nothing is downloaded.  Usage:  bash ep_balance_b200/launch/bootstrap.sh [--no-tests]
set -euo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")/../.."
export MASTER_ADDR="${MASTER_ADDR:-127.0.0.1}"       # single node: the container hostname may not resolve
echo "== environment"
python -m ep_balance_b200.launch.env_check || echo "(problems listed above; continuing)"
echo "== native extension (sm_100a, in-tree)"
python -c "import __graft_entry__ as g; g.build(); print('extension built and importable')"
if [ -n "${REFERENCE_SRC:-}" ]; then
  echo "== reference arm -> baseline/_ref"
  src="$REFERENCE_SRC"
  if [ ! -w "$src" ]; then                             # a read-only checkout: build from a copy
    src="$(mktemp -d)/reference"; cp -r "$REFERENCE_SRC" "$src"
  fi
  python -m pip install --no-index --no-build-isolation --no-deps --find-links "${WHEELHOUSE:-/opt/wheelhouse}" \
      --target baseline/_ref "$src"
fi
if python -c "import torch, sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then
  echo "== GPU smoke"
  python -c "import __graft_entry__ as g; g.smoke()"
else
  echo "== no GPU visible: skipping the GPU smoke (the build above is the cross-compile check)"
fi
if [ "${1:-}" != "--no-tests" ]; then
  echo "== CPU tests (core, solver, status)"
  python -m pytest tests/test_core_cpu.py tests/test_solver_cpu.py tests/test_status_cpu.py -q -p no:warnings
fi
echo "== next: bash ep_balance_b200/launch/run_train.sh   |   python bench.py   |   python -m pytest tests -m gpu"
