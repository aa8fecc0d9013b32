"""Page scorer entry points (host wrappers around ``locks_rki4_score_bt``).

Names and argument meaning follow the reference's
``selection/rki4_score_cuda.py``: ``rki4_score_only`` (:3263-3448),
``rki4_select_only`` (:3450-3497) and ``rki4_score_state`` (:3500-3504).
"""
from __future__ import annotations

import torch

from .. import _cabi
from .select import nrmtopb_select


def rki4_score_only(st, lidx: int, q, block_table, seq_lens, n_req: int,
                    scale: float, publish_hmax: bool = True) -> None:
    """Fill ``st.score_h[r, kh, g, p]`` for p < n_sel_hi[r] from layer
    ``lidx``'s summaries.  q: bf16 (>= n_req, n_kv*G, d)."""
    assert q.dtype == torch.bfloat16 and q.stride(-1) == 1
    assert q.stride(1) == st.d, "q heads must be contiguous"
    assert block_table.dtype == torch.int32 and block_table.stride(1) == 1
    rec = st.pp_rec[lidx]
    hmax = st.hmax if (publish_hmax and st.hmax is not None) else None
    if getattr(st, "row_order_n", 0) == n_req:      # large batch: longest row first
        _cabi.call("locks_rki4_score_bt_rows", _cabi.ptr(q), q.stride(0),
                   _cabi.ptr(rec), _cabi.ptr(block_table), block_table.stride(0),
                   _cabi.ptr(st.n_sel_hi), _cabi.ptr(st.score_h), _cabi.ptr(hmax),
                   int(n_req), int(st.n_kv), int(st.G), int(st.d), int(st.page),
                   int(st.max_pages), int(block_table.shape[1]), int(st.NB),
                   float(scale), int(st.zsplit or 0), _cabi.ptr(st.order_sel),
                   _cabi.ptr(st.status), _cabi.stream())
        return
    _cabi.call("locks_rki4_score_bt", _cabi.ptr(q), q.stride(0),
               _cabi.ptr(rec), _cabi.ptr(block_table), block_table.stride(0),
               _cabi.ptr(st.n_sel_hi), _cabi.ptr(st.score_h), _cabi.ptr(hmax),
               int(n_req), int(st.n_kv), int(st.G), int(st.d), int(st.page),
               int(st.max_pages), int(block_table.shape[1]), int(st.NB),
               float(scale), int(st.zsplit or 0), _cabi.ptr(st.status),
               _cabi.stream())


def rki4_select_only(st, n_req: int, has_hmax: bool = True, append=None) -> None:
    """GQA combine (``st.combine``) + exact top-b from ``st.score_h``.
    ``append`` (``attention.kv_append_desc``): the layer's KV write rides in the
    same launch."""
    nrmtopb_select(st, n_req, has_hmax=has_hmax, append=append)


def rki4_score_state(st, lidx: int, q, block_table, seq_lens, n_req: int,
                     scale: float, append=None) -> None:
    """Score then select: the whole Stage A of one layer (2 launches)."""
    rki4_score_only(st, lidx, q, block_table, seq_lens, n_req, scale)
    rki4_select_only(st, n_req, append=append)
