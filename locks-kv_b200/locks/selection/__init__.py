"""Stage A -- decode-time page selection.

  rki4_build_*(st, K_layers, block_table, settled_lens, ...)   page finalize
  derive_page_params(st, seq_lens, n_req)                      once per step
  rki4_score_state(st, layer, q, block_table, seq_lens, n_req, scale)
        -> st.score_h -> st.score -> st.page_table / st.page_cnt

All persistent state lives in :class:`Rki4State`.  Same surface as the
reference's ``selection/__init__.py``.
"""
from __future__ import annotations

from .rki4_build import (rki4_build_bulk, rki4_build_delta,
                         rki4_build_refresh, rki4_build_slots,
                         rki4_build_tail)
from .rki4_score import rki4_score_only, rki4_score_state, rki4_select_only
from .rki4_state import TAGW, Rki4State
from .select import (append_advance, derive_page_params, nrmtopb_select,
                     topb_select)
from .mla_select import (MlaState, build_page_factors, build_prompt_factors,
                         mla_decode, mla_derive, mla_forward, mla_page_score,
                         mla_refresh_rows, mla_select_pages)

__all__ = [
    "Rki4State", "TAGW", "rki4_build_refresh", "rki4_build_slots",
    "rki4_build_tail",
    "rki4_build_bulk", "rki4_build_delta", "append_advance", "derive_page_params", "topb_select",
    "nrmtopb_select", "rki4_score_only", "rki4_select_only", "rki4_score_state",
    "MlaState", "build_page_factors", "build_prompt_factors", "mla_derive",
    "mla_page_score", "mla_select_pages", "mla_decode", "mla_forward",
    "mla_refresh_rows",
]
