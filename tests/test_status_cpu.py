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
