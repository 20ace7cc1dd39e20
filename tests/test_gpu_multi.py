"""Fused layer across real GPUs (one process per GPU); skipped when fewer than two are visible."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_fused_layer_on_multiple_gpus():
    n = torch.cuda.device_count()
    n = n if n in (2, 4, 8) else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29517", "-m", "ep_balance_b200.launch.check_multi",
           "--steps", "2"]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "CHECK_MULTI PASS" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_library_path_weight_channels_on_multiple_gpus():
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29519", "-m",
           "ep_balance_b200.launch.check_library_multi", "--bandwidth-mb", "64"]
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "CHECK_LIBRARY_MULTI PASS" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
