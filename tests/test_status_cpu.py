"""Status words: the host learns of a damaged step late, without synchronising, and raises a typed error."""

import pytest
import torch

from ep_balance_b200.utils.status import MoEStatusError, StatusBoard, StatusMonitor, raise_if_set


def test_board_rows_are_views_and_check_now_raises():
    board = StatusBoard(3, "cpu")
    board.check_now()
    row = board.row(1)
    row[0], row[1], row[2] = 4, 30, 12345          # what a kernel writes: code, site, detail
    with pytest.raises(MoEStatusError) as err:
        board.check_now()
    assert (err.value.layer, err.value.code, err.value.site, err.value.detail) == (1, 4, 30, 12345)
    assert "row overflow" in str(err.value)
    board.clear()
    board.check_now()


def test_monitor_reports_at_the_next_poll_and_on_drain():
    board = StatusBoard(2, "cpu")
    mon = StatusMonitor(board.words, depth=3)
    mon.poll()                                      # step 0: clean copy taken
    board.row(0)[:3] = torch.tensor([2, 10, 0], dtype=torch.int32)
    mon.poll()                                      # step 1: the copy holds the error; step 0's copy is inspected (clean)
    with pytest.raises(MoEStatusError) as err:
        mon.poll()                                  # step 2: step 1's copy is inspected
    assert err.value.code == 2 and err.value.step == 1 and "signal timeout" in str(err.value)
    board.clear()
    mon2 = StatusMonitor(board.words)
    mon2.poll()
    board.row(1)[0] = 3
    mon2.poll()
    with pytest.raises(MoEStatusError):
        mon2.drain()


def test_monitor_rejects_wrong_shapes():
    with pytest.raises(ValueError):
        StatusMonitor(torch.zeros(4, dtype=torch.int32))
    raise_if_set([[0, 0, 0, 0], [0, 9, 9, 9]])      # only the code column decides


def test_row_budget_overflow_is_a_status_not_a_trap():
    """Rows beyond EPLB_MAX_RECV_ROWS are dropped, recorded, and raised by the host-side check."""
    from ep_balance_b200.parallel.grouped_mlp import (check_row_budget, grouped_expert_mlp, make_batched_gated_mlp,
                                                       make_grouped_gated_mlp, row_budget_status)
    torch.manual_seed(0)
    S, H, F, T = 2, 8, 16, 10
    w = (torch.randn(S, F, H), torch.randn(S, H, F))
    x = torch.randn(T, H)
    slot = torch.tensor([0, 1, 0, 1, 0, 1, 0, 1, 0, 0])
    sizes = torch.bincount(slot, minlength=S)
    act = torch.nn.functional.gelu
    kw = dict(w_stacked=w, batched_mlp_fn=make_batched_gated_mlp(False, act), grouped_mlp_fn=make_grouped_gated_mlp(False, act))
    check_row_budget()                       # clean to start with
    full = grouped_expert_mlp(x, slot, sizes, max_recv_rows=T, **kw)
    check_row_budget()                       # the budget held: nothing recorded
    assert int(row_budget_status("cpu")[0, 0]) == 0
    cut = grouped_expert_mlp(x, slot, sizes, max_recv_rows=T - 3, **kw)
    words = row_budget_status("cpu")[0].tolist()
    assert words == [4, 20, T, T - 3]
    # the rows that fitted are unchanged, the dropped ones come back as zeros
    order = torch.argsort(slot, stable=True)
    kept, dropped = order[: T - 3], order[T - 3:]
    assert torch.allclose(cut[kept], full[kept], atol=1e-5)
    assert torch.count_nonzero(cut[dropped]) == 0
    with pytest.raises(MoEStatusError) as err:
        check_row_budget()
    assert err.value.code == 4 and err.value.detail == T and "EPLB_MAX_RECV_ROWS" in str(err.value)
    check_row_budget()                       # reading it cleared it
    # the same word feeds the late monitor
    grouped_expert_mlp(x, slot, sizes, max_recv_rows=T - 1, **kw)
    mon = StatusMonitor(row_budget_status("cpu"))
    mon.poll()
    with pytest.raises(MoEStatusError):
        mon.drain()
    row_budget_status("cpu").zero_()
