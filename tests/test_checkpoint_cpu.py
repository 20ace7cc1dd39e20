"""Checkpoint files: atomic layout, newest-complete pointer, world-size guard."""

import os

import pytest
import torch

from ep_balance_b200.utils.checkpoint import latest_step, load_checkpoint, save_checkpoint, step_dir


def test_round_trip_and_latest_pointer(tmp_path):
    root = str(tmp_path)
    assert latest_step(root) is None
    for step in (2, 4):
        for rank in (1, 0):
            save_checkpoint(root, step, rank=rank, world=2, replicated={"w": torch.full((3,), float(step))},
                            sharded={"e": torch.full((2,), float(10 * step + rank))})
    assert latest_step(root) == 4
    step, rep, shard = load_checkpoint(root, rank=1, world=2)
    assert step == 4 and rep["w"].tolist() == [4.0] * 3 and shard["e"].tolist() == [41.0, 41.0]
    step, rep, shard = load_checkpoint(root, step=2, rank=0, world=2)
    assert step == 2 and shard["e"].tolist() == [20.0, 20.0]
    assert sorted(os.listdir(step_dir(root, 4))) == ["experts_rank0.pt", "experts_rank1.pt", "replicated.pt"]
    assert not [f for f in os.listdir(root) if ".tmp." in f]


def test_world_size_mismatch_is_rejected(tmp_path):
    root = str(tmp_path)
    save_checkpoint(root, 1, rank=0, world=1, replicated={}, sharded={})
    with pytest.raises(ValueError):
        load_checkpoint(root, rank=0, world=2)
    with pytest.raises(FileNotFoundError):
        load_checkpoint(str(tmp_path / "missing"), rank=0, world=1)
