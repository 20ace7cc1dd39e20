"""Host model of the fused layer's token transport: who writes which row of whose buffer, and when a tile is complete.

The device code (``ops/csrc/solver.cu`` ``build_tables``, ``ops/csrc/comm.cuh`` ``comm_dispatch``) derives
everything below from the plan ``(x, q)`` without any exchange between ranks: every rank computes the layout
of EVERY rank's receive buffer, so a sender knows where its rows go and a receiver knows how many arrivals
make a tile complete.  This module restates those rules in plain Python.  It is the specification that
``tests/test_transport_model_cpu.py`` checks for ranks counts the GPU tests cannot reach, and a reading aid
for the kernels; nothing on the hot path imports it.

Layout of rank ``h``'s receive buffer (rows): the experts it hosts form groups, owned experts first, then
replicas, each by ascending id; a group starts on a multiple of ``tile_rows`` and holds the rows of its
expert ordered by source rank (source 0's rows, then source 1's, ...), each source's rows in the order of the
units in that source's expert-sorted list.  Senders walk a receiver's buffer in blocks of ``block_rows``
(``tile_rows`` is a multiple): item ``(block b, destination d)`` moves the rows of this sender that fall into
rows ``[b * block_rows, (b + 1) * block_rows)`` of ``d``'s buffer and then adds 1 to the arrival counter of
the tile the block lies in -- also when it had no row there -- so a tile is complete after
``(tile_rows / block_rows) * R`` arrivals.  A row carries ``(source, position)``, the position of its unit in
the source's expert-sorted list; the host returns the expert's output (and gradients) to that position.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


@dataclass
class BufferLayout:
    """Receive buffer of one rank: ``groups`` = [(expert, first row, rows)], in buffer order."""

    groups: List[Tuple[int, int, int]]
    padded_rows: int

    def offset_of(self, expert: int) -> int:
        for e, off, _ in self.groups:
            if e == expert:
                return off
        return -1


def buffer_layout(x: torch.Tensor, q: torch.Tensor, main_rank: torch.Tensor, h: int, tile_rows: int) -> BufferLayout:
    """``x`` int [E, R] placement, ``q`` int [R, E, R] quotas (source, expert, destination)."""
    E = x.shape[0]
    hosted = [e for e in range(E) if int(x[e, h]) != 0]
    order = [e for e in hosted if int(main_rank[e]) == h] + [e for e in hosted if int(main_rank[e]) != h]
    groups, off = [], 0
    for e in order:
        rows = int(q[:, e, h].sum())
        groups.append((e, off, rows))
        off += _round_up(rows, tile_rows)
    return BufferLayout(groups, off)


def sender_tables(x, q, main_rank, me: int, tile_rows: int) -> Dict[str, torch.Tensor]:
    """What rank ``me`` needs to send: ``row_base[e, d]`` (first row of its rows for expert e in d's buffer, -1 if
    d does not host e), ``send_off[e, d]`` (how many of its units of expert e go to destinations before d),
    ``tiles_of[d]`` (tiles of d's buffer)."""
    E, R = x.shape
    row_base = torch.full((E, R), -1, dtype=torch.int64)
    send_off = torch.zeros((E, R), dtype=torch.int64)
    tiles_of = torch.zeros(R, dtype=torch.int64)
    for d in range(R):
        lay = buffer_layout(x, q, main_rank, d, tile_rows)
        tiles_of[d] = lay.padded_rows // tile_rows
        for e, off, _ in lay.groups:
            row_base[e, d] = off + int(q[:me, e, d].sum())
    for e in range(E):
        send_off[e] = torch.cumsum(q[me, e], 0) - q[me, e]
    return {"row_base": row_base, "send_off": send_off, "tiles_of": tiles_of}


def block_rows_for(R: int, tile_rows: int) -> int:
    """Largest power of two that is at most ``min(tile_rows, 32 * R)`` (the runtime's choice)."""
    b = 1
    while b * 2 <= min(tile_rows, 32 * R):
        b *= 2
    return b


def transport_items(q: torch.Tensor, tables: Dict[str, torch.Tensor], me: int, tile_rows: int, block_rows: int):
    """Items in ticket order.  Yields ``(dst, block, pieces)`` with ``pieces`` = [(expert, first position in the
    sender's expert-sorted list, first row in dst's buffer, rows)]; an item with no piece still signals."""
    _, E, R = q.shape
    exp_prefix = torch.cumsum(q[me].sum(1), 0) - q[me].sum(1)          # first position of each expert at the sender
    bpt = tile_rows // block_rows
    n_items = int(tables["tiles_of"].max()) * bpt * R
    for it in range(n_items):
        b, k = divmod(it, R)
        dst = (me + k) % R
        if b >= int(tables["tiles_of"][dst]) * bpt:
            continue
        r0, r1 = b * block_rows, (b + 1) * block_rows
        pieces = []
        for e in range(E):
            base, cnt = int(tables["row_base"][e, dst]), int(q[me, e, dst])
            lo, hi = max(base, r0), min(base + cnt, r1)
            if base >= 0 and lo < hi:
                pieces.append((e, int(exp_prefix[e]) + int(tables["send_off"][e, dst]) + (lo - base), lo, hi - lo))
        yield dst, b, pieces


def simulate(x: torch.Tensor, q: torch.Tensor, main_rank: torch.Tensor, tile_rows: int):
    """Run every rank's items.  Returns ``(writer, arrivals)``: ``writer[d]`` maps a row of d's buffer to
    ``(source, position at the source, expert)``; ``arrivals[d][tile]`` counts the signals d received."""
    R = q.shape[0]
    block_rows = block_rows_for(R, tile_rows)
    writer: List[Dict[int, Tuple[int, int, int]]] = [dict() for _ in range(R)]
    arrivals: List[Dict[int, int]] = [dict() for _ in range(R)]
    for me in range(R):
        tables = sender_tables(x, q, main_rank, me, tile_rows)
        for dst, b, pieces in transport_items(q, tables, me, tile_rows, block_rows):
            for e, pos, row, n in pieces:
                for j in range(n):
                    if row + j in writer[dst]:
                        raise AssertionError(f"row {row + j} of rank {dst} written twice")
                    writer[dst][row + j] = (me, pos + j, e)
            tile = b * block_rows // tile_rows
            arrivals[dst][tile] = arrivals[dst].get(tile, 0) + 1
    return writer, arrivals
