"""Per-step page parameters and exact top-b page selection (host wrappers).

``derive_page_params`` and ``topb_select`` keep the reference signatures
(``selection/select.py:51-58`` and ``:183-222``); each is one kernel launch,
fixed-shape, allocation-free and sync-free.
"""
from __future__ import annotations

import torch

from .. import _cabi

COMBINE_NONE, COMBINE_NRM, COMBINE_MAX = 0, 1, 2


# A batch with more (request, kv-head) rows than this many resident CTAs gets
# its rows launched longest first (``locks_row_order``): the selector holds two
# CTAs per SM, the decode one.
ROW_ORDER_MIN_ROWS = 148


def _row_order(st, n_req: int) -> None:
    """Longest-first launch order of the step's rows for the selector and the
    decode (device-side rank sort of the page parameters just derived); small
    batches keep grid order."""
    if n_req * st.n_kv <= ROW_ORDER_MIN_ROWS or n_req > 2048:    # (rank sort: O(n^2))
        st.row_order_n = 0
        return
    if getattr(st, "order_sel", None) is None:
        st.order_sel = torch.zeros(st.max_reqs, device=st.n_pages.device,
                                   dtype=torch.int32)
        st.order_dec = torch.zeros_like(st.order_sel)
    _cabi.call("locks_row_order", _cabi.ptr(st.n_pages), _cabi.ptr(st.n_sel_hi),
               _cabi.ptr(st.b_fix), int(n_req), int(st.sink_pages),
               _cabi.ptr(st.order_sel), _cabi.ptr(st.order_dec), _cabi.stream())
    st.row_order_n = int(n_req)


def derive_page_params(st, seq_lens, n_req: int) -> None:
    """Refresh ``st.n_pages / n_sel_hi / b_fix`` for this decode step."""
    assert n_req <= st.max_reqs
    if getattr(st, "budget_req", None) is not None:
        _cabi.call("locks_derive_page_params_req", _cabi.ptr(seq_lens), int(n_req),
                   int(st.page), int(st.window_pages), int(st.sink_pages),
                   _cabi.ptr(st.budget_req), float(st.budget),
                   _cabi.ptr(st.n_pages), _cabi.ptr(st.n_sel_hi),
                   _cabi.ptr(st.b_fix), _cabi.stream())
    else:
        _cabi.call("locks_derive_page_params", _cabi.ptr(seq_lens), int(n_req),
                   int(st.page), int(st.window_pages), int(st.sink_pages),
                   int(getattr(st, "budget_abs", 0)), float(st.budget),
                   _cabi.ptr(st.n_pages), _cabi.ptr(st.n_sel_hi),
                   _cabi.ptr(st.b_fix), _cabi.stream())
    _row_order(st, n_req)


def append_advance(st, seq_lens, block_table, n_req: int, slot, slot_prev,
                   positions) -> None:
    """One decode step's bookkeeping on the device: ``positions`` <- lengths,
    ``slot_prev`` <- ``slot``, ``slot`` <- the appended token's cache slot,
    lengths grow by one, then :func:`derive_page_params` for the new lengths."""
    assert n_req <= st.max_reqs
    assert seq_lens.dtype == torch.int32 and block_table.dtype == torch.int32
    assert slot.dtype == slot_prev.dtype == positions.dtype == torch.int64
    assert block_table.stride(1) == 1
    if getattr(st, "budget_req", None) is not None:
        _cabi.call("locks_append_advance_req", _cabi.ptr(seq_lens),
                   _cabi.ptr(block_table), block_table.stride(0),
                   int(block_table.shape[1]), int(n_req), int(st.page),
                   int(st.window_pages), int(st.sink_pages),
                   _cabi.ptr(st.budget_req), float(st.budget), _cabi.ptr(slot),
                   _cabi.ptr(slot_prev), _cabi.ptr(positions),
                   _cabi.ptr(st.n_pages), _cabi.ptr(st.n_sel_hi),
                   _cabi.ptr(st.b_fix), _cabi.stream())
        return
    _cabi.call("locks_append_advance", _cabi.ptr(seq_lens), _cabi.ptr(block_table),
               block_table.stride(0), int(block_table.shape[1]), int(n_req),
               int(st.page), int(st.window_pages), int(st.sink_pages),
               int(getattr(st, "budget_abs", 0)), float(st.budget),
               _cabi.ptr(slot), _cabi.ptr(slot_prev), _cabi.ptr(positions),
               _cabi.ptr(st.n_pages), _cabi.ptr(st.n_sel_hi), _cabi.ptr(st.b_fix),
               _cabi.stream())


def _select(st, n_req: int, combine: int, use_hmax: bool, append=None) -> None:
    args = (int(combine), _cabi.ptr(st.score_h), _cabi.ptr(st.score),
            _cabi.ptr(st.hmax if (use_hmax and st.hmax is not None) else None),
            _cabi.ptr(st.n_pages), _cabi.ptr(st.n_sel_hi),
            _cabi.ptr(st.b_fix), _cabi.ptr(st.page_table),
            _cabi.ptr(st.page_cnt), int(n_req), int(st.n_kv), int(st.G),
            int(st.max_pages), int(st.sink_pages))
    if append is None and getattr(st, "row_order_n", 0) == n_req:
        _cabi.call("locks_topb_select_rows", *args, _cabi.ptr(st.order_sel),
                   _cabi.stream())
    elif append is None:
        _cabi.call("locks_topb_select", *args, _cabi.stream())
    else:       # a KvAppendDesc (attention.kv_append_desc): the layer's KV write
        import ctypes
        _cabi.call("locks_topb_select_append", *args,
                   ctypes.cast(ctypes.pointer(append), ctypes.c_void_p),
                   _cabi.stream())


def topb_select(st, n_req: int) -> None:
    """Top-b on an already combined ``st.score`` -> ``st.page_table`` /
    ``st.page_cnt`` (static budget ``st.b_fix``)."""
    _select(st, n_req, COMBINE_NONE, False)


def nrmtopb_select(st, n_req: int, has_hmax: bool = False, append=None) -> None:
    """Fused GQA combine + top-b from ``st.score_h`` using the state's combine
    mode (reference ``selection/select_cuda.py:3614-3731``).  ``append``: the
    layer's KV write, stored by the same launch."""
    _select(st, n_req, COMBINE_NRM if st.combine == "nrm" else COMBINE_MAX,
            has_hmax and st.combine == "nrm", append)
