"""Expert MLP over slot-grouped rows with library GEMMs (``torch._grouped_mm`` / ``torch.bmm``).

This is the portable compute stage of :mod:`ep_balance_b200.parallel.library_path` -- the CPU
oracle and the NCCL baseline.  The fused layer does not use it (it runs
``ops/csrc/grouped_gemm.cu``).  Reference: eplb/integration/grouped_mlp.py:31-349.

Weights follow the ``[out, in]`` convention and are stacked per local slot:
``w[0]`` is ``[S, F or 2F, H]``, ``w[1]`` is ``[S, H, F]``.
"""

from __future__ import annotations

import os
from typing import Callable, Optional, Sequence, Tuple

import torch

from ..utils import profiling


# ---------------------------------------------------------------- capability probes
def grouped_mm_usable(x: torch.Tensor) -> bool:
    """``torch._grouped_mm`` exists and the tensor qualifies (CUDA, cc >= 9, 16-bit float)."""
    if not hasattr(torch, "_grouped_mm") or not x.is_cuda:
        return False
    if x.dtype not in (torch.bfloat16, torch.float16):
        return False
    return torch.cuda.get_device_capability(x.device)[0] >= 9


def ragged_enabled(x: torch.Tensor) -> bool:
    if os.environ.get("EPLB_GROUPED_GEMM", "1").strip().lower() in ("0", "false", "no", ""):
        return False
    return grouped_mm_usable(x)


def widths_aligned(element_size: int, *widths: int) -> bool:
    """Grouped GEMM needs every row stride to be a multiple of 16 bytes."""
    return all((int(w) * int(element_size)) % 16 == 0 for w in widths)


def ragged_expert_ok(hidden: int, element_size: int, w1_eff: torch.Tensor, w2_eff: torch.Tensor, gated: bool) -> bool:
    widths = [hidden, *w1_eff.shape[1:], *w2_eff.shape[1:]]
    if gated:
        widths.append(w1_eff.shape[-1] // 2)
    return widths_aligned(element_size, *widths)


# ---------------------------------------------------------------- MLP factories
def _activate(h: torch.Tensor, gated: bool, act: Callable) -> torch.Tensor:
    if gated:
        gate, up = torch.chunk(h, 2, dim=-1)
        return act(gate) * up
    return act(h)


def make_batched_gated_mlp(gated: bool, act: Callable) -> Callable:
    """``fn(x[S, N, H], (W1[S, *, H], W2[S, H, *])) -> y[S, N, H]`` with ``x @ W.t()`` per slot."""

    def fn(x: torch.Tensor, w: Tuple[torch.Tensor, ...]) -> torch.Tensor:
        h = _activate(torch.bmm(x, w[0].transpose(1, 2)), gated, act)
        return torch.bmm(h, w[1].transpose(1, 2))

    return fn


def make_grouped_gated_mlp(gated: bool, act: Callable) -> Callable:
    """Ragged twin: ``fn(x[T, H], (W1, W2), offs[S]) -> y[T, H]``; ``offs`` = int32 exclusive row ends."""

    def fn(x: torch.Tensor, w: Tuple[torch.Tensor, ...], offs: torch.Tensor) -> torch.Tensor:
        h = _activate(ragged_mm(x, w[0].transpose(1, 2), offs), gated, act)
        return ragged_mm(h, w[1].transpose(1, 2), offs)

    def supports(x: torch.Tensor, w: Tuple[torch.Tensor, ...]) -> bool:
        return ragged_expert_ok(x.shape[-1], x.element_size(), w[0].transpose(1, 2), w[1].transpose(1, 2), gated)

    fn.supports = supports
    return fn


# ---------------------------------------------------------------- row bookkeeping (no host reads)
def slot_offsets(group_sizes: torch.Tensor, max_rows: Optional[int] = None) -> torch.Tensor:
    """int32 exclusive end offset of each slot, clamped to ``max_rows`` when given."""
    offs = group_sizes.to(torch.int64).cumsum(0)
    if max_rows is not None:
        offs = offs.clamp(max=int(max_rows))
    return offs.to(torch.int32)


def slot_sort(recv_slot: torch.Tensor, valid: Optional[torch.Tensor], n_slot: int) -> torch.Tensor:
    """Stable permutation putting rows in slot-major order; invalid rows go last."""
    key = recv_slot.to(torch.int64)
    if valid is not None:
        key = torch.where(valid, key, torch.full_like(key, int(n_slot)))
    return torch.argsort(key, stable=True)


def compact_rows(x: torch.Tensor, order: torch.Tensor, total_rows: torch.Tensor, max_rows: Optional[int]) -> torch.Tensor:
    """Rows in slot-major order, truncated to a host-static budget.

    When more rows arrive than the budget holds, the extra rows are dropped (they come back as zeros from
    :func:`scatter_rows`) and the overflow is recorded in this device's row-budget status word -- code 4
    (row overflow), site 20, detail = the number of rows that arrived.  Nothing traps and nothing
    synchronises: the host learns of it from :func:`check_row_budget` or from a
    :class:`~ep_balance_b200.utils.status.StatusMonitor` on :func:`row_budget_status`, and an optimizer
    guarded by that word skips the damaged step.  The reference guards the same budget with a device-side
    assert (eplb/integration/grouped_mlp.py:180-205), which ends the CUDA context.
    """
    if max_rows is None:
        return x.index_select(0, order)
    _record_overflow(total_rows, int(max_rows))
    return x.index_select(0, order[: int(max_rows)])


_ROW_BUDGET_SITE = 20
_row_budget_words: dict = {}


def row_budget_status(device) -> torch.Tensor:
    """The ``[1, 4]`` int32 status word of the portable path's row budget on ``device`` (created on first use)."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    words = _row_budget_words.get(device)
    if words is None:
        words = _row_budget_words[device] = torch.zeros((1, 4), dtype=torch.int32, device=device)
    return words


def _record_overflow(total_rows: torch.Tensor, max_rows: int, site: int = _ROW_BUDGET_SITE) -> None:
    words = row_budget_status(total_rows.device)
    total = total_rows.reshape(()).to(torch.int64)
    over = (total > max_rows) & (words[0, 0] == 0)          # the first overflow stays on record
    hit = torch.stack([torch.full_like(total, 4), torch.full_like(total, site),
                       total.clamp(max=2 ** 31 - 1), torch.full_like(total, max_rows)]).to(torch.int32)
    words[0].copy_(torch.where(over, hit, words[0]))


def check_row_budget(device=None, clear: bool = True) -> None:
    """Synchronous read of the row-budget status; raises :class:`MoEStatusError` if a step overflowed."""
    from ..utils.status import MoEStatusError
    for dev, words in list(_row_budget_words.items()):
        if device is not None and torch.device(device) != dev:
            continue
        code, site, detail, budget = (int(v) for v in words[0].tolist())
        if code:
            if clear:
                words.zero_()
            err = MoEStatusError(0, code, site, detail)
            what = "EPLB_MAX_RECV_ROWS" if site == _ROW_BUDGET_SITE else "the padded transport's rows per rank pair"
            err.args = (f"{err.args[0]}: {detail} rows arrived, {what} holds {budget}",)
            raise err


def scatter_rows(y: torch.Tensor, order: torch.Tensor, num_rows: int) -> torch.Tensor:
    """Inverse of the slot-major gather (rows that were truncated away come back as zeros)."""
    out = y.new_zeros((int(num_rows),) + tuple(y.shape[1:]))
    return out.index_copy(0, order[: y.shape[0]], y)


def ragged_mm(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
    """``y[rows of slot s] = x[rows of slot s] @ w[s]`` with ``w`` ``[S, in, out]``."""
    if grouped_mm_usable(x):
        return torch._grouped_mm(x, w, offs=offs)
    out = x.new_zeros((x.shape[0], w.shape[-1]))
    lo = 0
    for s, hi in enumerate(offs.tolist()):  # host loop: CPU / unsupported-GPU fallback only
        if hi > lo:
            out[lo:hi] = x[lo:hi] @ w[s]
        lo = hi
    return out


def ragged_mm_tn(a: torch.Tensor, b: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
    """Per-slot ``a_s^T b_s`` (weight gradient): returns ``[S, a_cols, b_cols]``."""
    if grouped_mm_usable(a):
        return torch._grouped_mm(a.t(), b, offs=offs)
    S = offs.numel()
    out = a.new_zeros((S, a.shape[1], b.shape[1]))
    lo = 0
    for s, hi in enumerate(offs.tolist()):
        if hi > lo:
            out[s] = a[lo:hi].t() @ b[lo:hi]
        lo = hi
    return out


def mask_rows(x: torch.Tensor, keep: torch.Tensor) -> torch.Tensor:
    """Zero rows with ``where`` (a multiply would let NaN/Inf garbage in padding through)."""
    return torch.where(keep.view(-1, *([1] * (x.dim() - 1))), x, torch.zeros_like(x))


# ---------------------------------------------------------------- dispatcher
def grouped_expert_mlp(recv_tokens: torch.Tensor, recv_slot: torch.Tensor, group_sizes: torch.Tensor,
                       w_stacked: Sequence[torch.Tensor], batched_mlp_fn: Callable, cap: Optional[int] = None,
                       valid_mask: Optional[torch.Tensor] = None, grouped_mlp_fn: Optional[Callable] = None,
                       max_recv_rows: Optional[int] = None) -> torch.Tensor:
    """Run every received row through the expert in its slot; returns rows in the received order.

    Ragged path (``grouped_mlp_fn`` given and supported): rows are gathered slot-major and the slot
    boundaries come from ``group_sizes`` on the device -- no padding, no ``cap``.  Padded path: a
    dense ``[S, cap, H]`` batch; ``cap`` must bound every slot's row count.
    """
    n_slot = int(group_sizes.shape[0])
    T, H = recv_tokens.shape
    w = tuple(w_stacked)
    use_ragged = (grouped_mlp_fn is not None and ragged_enabled(recv_tokens)
                  and getattr(grouped_mlp_fn, "supports", lambda *_: True)(recv_tokens, w))
    if grouped_mlp_fn is not None and not recv_tokens.is_cuda:
        use_ragged = True  # host fallback of ragged_mm keeps CPU tests on the same code path
    if use_ragged:
        order = slot_sort(recv_slot, valid_mask, n_slot)
        x = compact_rows(recv_tokens, order, group_sizes.sum(), max_recv_rows)
        offs = slot_offsets(group_sizes, max_recv_rows)
        with profiling.record("apply/expert_gemm", time_it=True, device=recv_tokens.device):
            y = grouped_mlp_fn(x, w, offs)
        keep = torch.arange(y.shape[0], device=y.device) < offs[-1]
        return scatter_rows(mask_rows(y, keep), order, T)

    if cap is None:
        raise ValueError("padded expert path needs a per-slot capacity `cap`")
    cap = int(cap)
    slot = recv_slot.to(torch.int64)
    if valid_mask is not None:
        # padding rows are ranked in a slot of their own so that they do not take positions of slot 0's real rows
        pos = _position_in_slot(torch.where(valid_mask, slot, torch.full_like(slot, n_slot)), n_slot + 1)
        slot = torch.where(valid_mask, slot, torch.zeros_like(slot))
        inside = (pos < cap) & valid_mask
    else:
        pos = _position_in_slot(slot, n_slot)
        inside = pos < cap
    flat = torch.where(inside, slot * cap + pos, torch.full_like(slot, n_slot * cap))  # overflow row
    x_pad = recv_tokens.new_zeros((n_slot * cap + 1, H)).index_copy(0, flat, recv_tokens)
    with profiling.record("apply/expert_gemm", time_it=True, device=recv_tokens.device):
        y_pad = batched_mlp_fn(x_pad[:-1].view(n_slot, cap, H), w).reshape(n_slot * cap, -1)
    y_pad = torch.cat([y_pad, y_pad.new_zeros((1, y_pad.shape[1]))])
    return mask_rows(y_pad.index_select(0, flat), inside)


def _position_in_slot(slot: torch.Tensor, n_slot: int) -> torch.Tensor:
    order = torch.argsort(slot, stable=True)
    counts = torch.zeros(n_slot, dtype=torch.int64, device=slot.device).scatter_add_(0, slot, torch.ones_like(slot))
    starts = counts.cumsum(0) - counts
    pos_sorted = torch.arange(slot.numel(), device=slot.device) - starts[slot[order]]
    return torch.empty_like(pos_sorted).index_copy_(0, order, pos_sorted)
