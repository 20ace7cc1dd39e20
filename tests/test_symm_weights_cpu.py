"""Schedule of the device-initiated replica weight channel (pure tensor code, runs on CPU)."""

import torch

from ep_balance_b200.parallel.symm_weights import local_slot_table, replica_schedule, symm_weights_enabled


def test_local_slot_table_counts_owners_in_id_order():
    main = torch.tensor([1, 0, 1, 1, 0, 2])
    ls, cap = local_slot_table(main, 3)
    assert ls.tolist() == [0, 0, 1, 2, 1, 0] and cap == 3


def test_schedule_lists_hosted_experts_by_slot():
    main = torch.tensor([0, 0, 1, 1, 2, 2, 3, 3])
    ls, _ = local_slot_table(main, 4)
    x = torch.zeros((8, 4), dtype=torch.int8)
    x[torch.arange(8), main] = 1
    x[0, 2] = 1
    x[7, 2] = 1
    s = replica_schedule(x, main, ls, me=2, n_slot=5, world=4)
    assert s["slot_to_e"].tolist() == [0, 4, 5, 7, -1]
    assert s["owner"].tolist() == [0, 2, 2, 3, -1]
    assert s["home_row"].tolist()[:4] == [0, 0, 1, 1]
    assert s["inbox_row"].tolist()[:4] == [0 * 4 + 2, 0 * 4 + 2, 1 * 4 + 2, 1 * 4 + 2]
    assert s["remote"].tolist() == [True, False, False, True, False]


def test_schedule_ignores_hosts_beyond_the_slot_budget():
    main = torch.tensor([0, 0, 0, 1])
    ls, _ = local_slot_table(main, 2)
    x = torch.tensor([[1, 0], [1, 0], [1, 0], [1, 1]], dtype=torch.int8)
    s = replica_schedule(x, main, ls, me=0, n_slot=3, world=2)
    assert s["slot_to_e"].tolist() == [0, 1, 2]


def test_env_switch_accepts_reference_spellings(monkeypatch):
    for name in ("symm", "gin", "nccl_gin", "devnccl", "GIN"):
        monkeypatch.setenv("EPLB_WEIGHT_COMM", name)
        assert symm_weights_enabled()
    monkeypatch.setenv("EPLB_WEIGHT_COMM", "broadcast")
    assert not symm_weights_enabled()
