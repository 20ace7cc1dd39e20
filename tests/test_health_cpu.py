"""Failure detection on the host: CPU processes share a FileStore; no GPU is involved.
A rank raises between steps, a rank never joins, a heartbeat goes missing, an omega row is corrupted."""

import os
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ep_balance_b200.parallel.health import Heartbeat, PeerFailure, StepGuard, check_omega


def _store(path, world):
    return dist.FileStore(path, world)


def _rank_that_dies(rank, path, world, result_dir):
    hb = Heartbeat(_store(path, world), rank, world, stale_after_s=0.6)
    hb.beat(0)
    hb.wait_for_all(10.0)
    outcome = "finished"
    try:
        for step in range(1, 200):
            if rank == 1 and step == 3:
                raise RuntimeError("rank 1 stops between steps")   # no kernel or collective is in flight
            StepGuard(hb).before_step(step)
            time.sleep(0.05)                                       # the "step"
            hb.beat(step)
    except PeerFailure as exc:
        outcome = f"peer_failure:{exc.ranks}"
    except RuntimeError:
        outcome = "died"
    with open(os.path.join(result_dir, f"r{rank}"), "w") as f:
        f.write(outcome)


def test_survivors_learn_of_a_rank_that_stopped(tmp_path):
    world = 3
    path = str(tmp_path / "store")
    mp.spawn(_rank_that_dies, args=(path, world, str(tmp_path)), nprocs=world, join=True)
    got = {r: open(tmp_path / f"r{r}").read() for r in range(world)}
    assert got[1] == "died"
    assert got[0] == "peer_failure:[1]" and got[2] == "peer_failure:[1]"


def test_a_rank_that_never_joins_is_named(tmp_path):
    store = _store(str(tmp_path / "s"), 1)
    hb0 = Heartbeat(store, 0, 3, stale_after_s=5)
    hb2 = Heartbeat(store, 2, 3, stale_after_s=5)
    hb0.beat(0)
    hb2.beat(0)
    with pytest.raises(PeerFailure) as e:
        hb0.wait_for_all(0.3)
    assert e.value.ranks == [1]


def test_dropped_heartbeat_and_reported_failure(tmp_path):
    store = _store(str(tmp_path / "s"), 1)
    now = [100.0]
    hbs = [Heartbeat(store, r, 2, stale_after_s=1.0, clock=lambda: now[0]) for r in range(2)]
    hbs[0].beat(1)
    hbs[1].beat(1)
    hbs[0].check_peers()                         # both fresh
    now[0] += 0.8
    hbs[0].beat(2)                               # rank 1's beat for step 2 is dropped
    hbs[0].check_peers()                         # still inside the window
    with pytest.raises(PeerFailure) as e:
        hbs[0].check_peers(min_step=2)           # but it has not reached step 2
    assert e.value.ranks == [1]
    now[0] += 0.8
    with pytest.raises(PeerFailure, match="last heartbeat"):
        hbs[0].check_peers()                     # and now it is stale
    hbs[1].beat(3)
    hbs[0].check_peers()

    def bad_status():
        raise RuntimeError("MoE runtime status: signal timeout (site 20, detail 1)")

    guard = StepGuard(hbs[1], [bad_status])
    with pytest.raises(RuntimeError):
        guard.after_step(4)                      # device status word was set: published, not beaten
    with pytest.raises(PeerFailure, match="signal timeout"):
        hbs[0].check_peers()


def test_corrupted_omega_row_is_found():
    omega = torch.tensor([[3, 1, 0, 4], [2, 2, 2, 2], [0, 8, 0, 0]])
    assert check_omega(omega, torch.tensor([8, 8, 8])) == []
    omega[1, 2] = 7                              # a flipped count: row sum no longer matches the units sent
    assert check_omega(omega, torch.tensor([8, 8, 8])) == [1]
    omega[2, 0] = -1
    assert check_omega(omega) == [2]
