"""Split-K merge (host wrapper of ``locks_merge_splits``).

out[r, h] = sum_s w_s acc_s / sum_s w_s l_s with w_s = exp(m_s - max_s m_s)
over the ACTIVE splits (recomputed from ``page_cnt`` with the split kernel's
own rule); rows without attended pages become 0, never NaN.  Reference:
``attention/merge.py:105-152``.
"""
from __future__ import annotations

from .. import _cabi


def merge_splits(st, out, n_req: int, pps_min: int) -> None:
    _cabi.call("locks_merge_splits", _cabi.ptr(st.m_part), _cabi.ptr(st.l_part),
               _cabi.ptr(st.acc_part), _cabi.ptr(st.page_cnt), _cabi.ptr(out),
               out.stride(0), int(n_req), int(st.n_kv), int(st.G), int(st.d),
               int(st.split), int(pps_min), _cabi.stream())
