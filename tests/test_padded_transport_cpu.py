"""Contract of the zero-sync padded token transport (single process: the all-to-all is the identity)."""

import pytest
import torch

from ep_balance_b200.parallel.grouped_mlp import check_row_budget, row_budget_status
from ep_balance_b200.parallel.library_path import PaddedAllToAllAdapter
from ep_balance_b200.utils.status import MoEStatusError


def test_blocks_are_aligned_and_masked():
    ad = PaddedAllToAllAdapter(rows_per_pair=5)
    assert ad.uses_padded_layout() and ad.cap == 8                      # rounded up to the alignment
    sent = torch.tensor([3])                                            # one rank: everything goes to rank 0
    payload = torch.arange(12.0).view(3, 4)
    rows = ad.dispatch_chunk(payload, sent, sent, None, tag=7)
    assert rows.shape == (8, 4)
    assert torch.equal(rows[:3], payload) and torch.count_nonzero(rows[3:]) == 0
    assert ad.valid_mask(7).tolist() == [True] * 3 + [False] * 5
    ids = ad.dispatch_ids(torch.tensor([4, 5, 6]), None, tag=7)
    assert ids.tolist() == [4, 5, 6, 0, 0, 0, 0, 0]
    back = ad.combine_chunk(rows * 2, sent, sent, None, tag=7)          # un-pads to the rows that were sent
    assert torch.equal(back, payload * 2)
    assert ad.chunk_state(7) is not None and ad.chunk_state(7) is None  # state is per chunk and released


def test_rows_beyond_the_block_are_dropped_and_recorded():
    row_budget_status("cpu").zero_()
    ad = PaddedAllToAllAdapter(rows_per_pair=8)
    sent = torch.tensor([11])
    payload = torch.randn(11, 2, requires_grad=True)
    rows = ad.dispatch_chunk(payload, sent, sent, None, tag=0)
    assert rows.shape == (8, 2) and torch.equal(rows.detach(), payload.detach()[:8])
    assert ad.valid_mask(0).all()
    back = ad.combine_chunk(rows, sent, sent, None, tag=0)
    assert torch.equal(back[:8].detach(), payload.detach()[:8]) and torch.count_nonzero(back[8:]) == 0
    back.sum().backward()                                               # dropped rows get no gradient
    assert payload.grad[:8].eq(1).all() and payload.grad[8:].eq(0).all()
    assert row_budget_status("cpu")[0].tolist() == [4, 21, 11, 8]
    with pytest.raises(MoEStatusError, match="rows per rank pair"):
        check_row_budget()
    check_row_budget()


def test_megatron_factory_builds_it_from_the_environment(monkeypatch):
    from ep_balance_b200.integration.megatron_moe import _make_adapter

    monkeypatch.setenv("EPLB_ADAPTER", "padded")
    monkeypatch.delenv("EPLB_PAIR_ROWS", raising=False)
    with pytest.raises(ValueError, match="EPLB_PAIR_ROWS"):
        _make_adapter()
    monkeypatch.setenv("EPLB_PAIR_ROWS", "100")
    ad = _make_adapter()
    assert isinstance(ad, PaddedAllToAllAdapter) and ad.cap == 104
