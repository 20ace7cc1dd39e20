"""Invariants of the fused layer's token transport, checked on its host model for rank counts up to 16."""

import pytest
import torch

from ep_balance_b200 import EPLBConfig, ProblemSpec, Topology, solve
from ep_balance_b200.parallel.transport_model import block_rows_for, buffer_layout, simulate
from ep_balance_b200.utils.workload import make_loads


@pytest.mark.parametrize("nodes,gpus,E,extra,tile", [(1, 2, 8, 1, 128), (2, 2, 16, 2, 256), (2, 4, 64, 2, 256),
                                                      (1, 8, 32, 2, 256), (4, 4, 64, 1, 128)])
def test_every_row_is_written_once_and_every_tile_hears_from_everyone(nodes, gpus, E, extra, tile):
    R = nodes * gpus
    loads = make_loads(R, E, 512, 4, 1.2, 0.25, 7)
    topo = Topology.from_nvlink_rdma(nodes, gpus)
    spec = ProblemSpec.contiguous_main_placement(E, R, weight_bytes_each=1000, s_tok=64, n_slot=E // R + extra)
    plan = solve(loads, topo, spec, EPLBConfig())
    x, q = plan.x.to(torch.int64), plan.q.to(torch.int64)
    assert int(x.sum()) > E, "the case needs at least one replica"
    writer, arrivals = simulate(x, q, spec.main_rank, tile)
    expected_signals = (tile // block_rows_for(R, tile)) * R
    positions = [set() for _ in range(R)]
    for d in range(R):
        lay = buffer_layout(x, q, spec.main_rank, d, tile)
        owned = [e for e, _, _ in lay.groups if int(spec.main_rank[e]) == d]
        assert [e for e, _, _ in lay.groups][: len(owned)] == sorted(owned)            # owned groups first, by id
        rows_expected = set()
        for e, off, rows in lay.groups:
            assert off % tile == 0 and rows == int(q[:, e, d].sum())
            rows_expected.update(range(off, off + rows))
            # inside a group the rows are ordered by source, each source's rows by its position
            got = [writer[d][r] for r in range(off, off + rows)]
            assert [g[0] for g in got] == sorted(g[0] for g in got)
            assert all(g[2] == e for g in got)
            for s in range(R):
                mine = [g[1] for g in got if g[0] == s]
                assert len(mine) == int(q[s, e, d]) and mine == list(range(mine[0], mine[0] + len(mine))) if mine else True
        assert set(writer[d]) == rows_expected                                          # nothing lands in the padding
        tiles = lay.padded_rows // tile
        assert arrivals[d] == {t: expected_signals for t in range(tiles)}               # every tile: one signal per block and rank
        for src, pos, _ in writer[d].values():
            assert pos not in positions[src], "a unit was sent twice"
            positions[src].add(pos)
    for s in range(R):                                                                  # every unit of every rank went out
        assert positions[s] == set(range(int(q[s].sum())))
