"""Process-wide glue between the plugin classes and the kernels.

Mirrors the part of the reference's ``backend/_runtime.py`` that sits on the
decode hot path: the config singleton (:95-120), the kv-cache -> layer index
map (:430-450), the Stage-A adapter ``_rki4_select_adapter`` (:661-723), the
Stage-B ``decode_dispatch`` (:807-838) and ``resolve_selection`` (:841-861).
Instrumentation lanes, the DRAM tier and the query-first experiments of the
reference are outside this build.
"""
from __future__ import annotations

import sys
from typing import Optional

from ..config import LocksConfig

_CONFIG: Optional[LocksConfig] = None
_ANNOUNCED = False

# decode launcher choice: the one-launch cluster decode from this many requests up
# (1 = always; the split + merge pair stays available below it)
FUSED_MIN_REQS = 1


def set_config(cfg: Optional[LocksConfig]) -> None:
    global _CONFIG
    _CONFIG = cfg


def get_config() -> Optional[LocksConfig]:
    return _CONFIG


def _layer_index(st, kv_cache) -> int:
    """Layer of an engine kv-cache tensor (the builder fills ``st._layer_of``
    from the tensors' data pointers)."""
    try:
        return st._layer_of[int(kv_cache.data_ptr())]
    except (AttributeError, KeyError):
        raise RuntimeError(
            "locks: kv_cache tensor is not registered with the selection "
            "state (builder did not map its data_ptr to a layer)") from None


def _rki4_select_adapter(q, kv_cache, block_table, seq_lens, st, n_req, scale,
                         cfg, append=None) -> None:
    """Stage A of one layer: score every selectable page from the packed
    summaries into ``st.score_h``, combine over the GQA group and keep the
    top-b pages (``st.page_table`` / ``st.page_cnt``).  The builder already
    derived the per-step page parameters."""
    from ..selection import rki4_score_state
    global _ANNOUNCED
    if not _ANNOUNCED:
        _ANNOUNCED = True
        print(f"[locks] selection kernels: sm_100a rki4 score (zsplit="
              f"{st.zsplit or 'auto'}, combine={st.combine}) + radix top-b",
              file=sys.stderr, flush=True)
    lidx = _layer_index(st, kv_cache)
    rki4_score_state(st, lidx, q, block_table, seq_lens, n_req, scale,
                     append=append)


def decode_dispatch(q, kv_cache, block_table, seq_lens, st, out, vsource,
                    scale, cfg) -> None:
    """Stage B of one layer.  Both launchers are sm_100a kernels of this
    library; a missing library raises (there is nothing to fall back to)."""
    from ..attention import (sparse_paged_decode_batched,
                             sparse_paged_decode_fused)
    if int(seq_lens.shape[0]) >= FUSED_MIN_REQS:
        sparse_paged_decode_fused(q, kv_cache, block_table, seq_lens, st, out,
                                  vsource, scale=scale)
    else:
        sparse_paged_decode_batched(q, kv_cache, block_table, seq_lens, st,
                                    out, vsource, scale=scale)


def resolve_selection():
    """(StateClass, derive_fn, select_fn, graph_safe)."""
    from .. import selection as sel
    return (sel.Rki4State, sel.derive_page_params, _rki4_select_adapter, True)
