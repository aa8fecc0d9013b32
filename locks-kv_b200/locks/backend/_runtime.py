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


# ---- the selection state the builder latched (read by the KV-write hook) ------
_STATE = None
_K_LAYERS = None


def set_state(st, K_layers) -> None:
    global _STATE, _K_LAYERS
    _STATE, _K_LAYERS = st, K_layers


def get_state():
    return _STATE, _K_LAYERS


# ---- profiling window ------------------------------------------------------------
# vLLM measures its CUDA-graph memory with a dummy run against a THROW-AWAY
# minimal KV cache (num_gpu_blocks is set during that run, so the field cannot
# tell the phases apart).  register() brackets those runs; the builder does not
# latch its kv-cache -> layer map inside the window (reference
# backend/_runtime.py:105-121, backend/builder.py:658-672).
_in_profiling = False


def set_profiling(on: bool) -> None:
    global _in_profiling
    _in_profiling = bool(on)


def in_profiling() -> bool:
    return _in_profiling


# ---- sparse-activation accounting (reference backend/attn.py:190-226) -------------
# decode rows served by the sparse path vs handed to the stock dense attention,
# with the gate that sent them there; printed once at exit.  A fraction below 1
# means part of a run that is labelled LOCKS was in fact full-KV attention.
_ACT = {"decode_rows_sparse": 0, "decode_rows_dense": 0, "dense_reasons": {}}


def count_sparse(n: int) -> None:
    _ACT["decode_rows_sparse"] += int(n)


def count_dense(n: int, reason: str) -> None:
    if n > 0:
        _ACT["decode_rows_dense"] += int(n)
        _ACT["dense_reasons"][reason] = _ACT["dense_reasons"].get(reason, 0) + int(n)


def get_activation():
    s, d = _ACT["decode_rows_sparse"], _ACT["decode_rows_dense"]
    if s + d == 0:
        return None
    return {"sparse": s, "dense": d, "frac": s / (s + d),
            "dense_reasons": dict(_ACT["dense_reasons"])}


def _activation_report() -> None:
    a = get_activation()
    if a is None:
        return
    ok = a["frac"] >= 1.0
    print(f"[locks] SPARSE ACTIVATION {a['sparse']}/{a['sparse'] + a['dense']} "
          f"decode rows = {100 * a['frac']:.2f}%  "
          f"[{'OK' if ok else 'part of this run was full-KV attention'}]",
          flush=True)
    if a["dense_reasons"]:
        print(f"[locks]   decode rows served DENSE by gate: {a['dense_reasons']}",
              flush=True)


__import__("atexit").register(_activation_report)


# ---- one-step dump for cross-checking a run inside the engine ------------------
# LOCKS_DUMP_STEP=<n> LOCKS_DUMP_PATH=<file>: at the n-th pure-decode step
# (eager runs only: the dump synchronises) every layer's query, selection and
# output are saved together with the KV cache, block table and lengths, so that
# the step can be recomputed outside the engine (the reference's gate
# instrument LOCKS_DUMP_PTAB, backend/_runtime.py:267-332).
_DUMP = {"step": -1, "seen": 0, "layers": {}, "done": False}


def dump_step_begin() -> None:
    """Called by the builder once per pure-decode step."""
    import os
    if _DUMP["done"] or "LOCKS_DUMP_STEP" not in os.environ:
        return
    _DUMP["step"] = int(os.environ["LOCKS_DUMP_STEP"])
    _DUMP["seen"] += 1


def dump_layer(lidx, q, kv_cache, block_table, seq_lens, st, out, n_req) -> None:
    import os
    import torch
    if _DUMP["done"] or _DUMP["seen"] != _DUMP["step"] or _DUMP["step"] < 0:
        return
    if torch.cuda.is_current_stream_capturing():
        return
    torch.cuda.synchronize()
    c = lambda t: t.detach().float().cpu() if t.dtype == torch.bfloat16 \
        else t.detach().cpu()
    # only the blocks the rows use travel, renumbered 0..n-1 (the engine's cache
    # holds every block of the pool)
    page = int(st.page)
    sl = seq_lens[:n_req]
    npg = int((int(sl.max().item()) + page - 1) // page)
    bt = block_table[:n_req, :npg].long()
    used, inv = torch.unique(bt.reshape(-1), return_inverse=True)
    bt_small = inv.reshape(n_req, npg).to(torch.int32)
    from ..attention.decode import _split_kv
    k, v = _split_kv(kv_cache)
    _DUMP["layers"][int(lidx)] = {
        "q": c(q[:n_req]), "out": c(out[:n_req]),
        "k_cache": c(k[used]), "v_cache": c(v[used]),
        "records": c(st.pp_rec[lidx][used]), "score_h": c(st.score_h[:n_req]),
        "page_table": c(st.page_table[:n_req]), "page_cnt": c(st.page_cnt[:n_req]),
        "block_table": c(bt_small), "seq_lens": c(sl),
        "b_fix": c(st.b_fix[:n_req]), "n_sel_hi": c(st.n_sel_hi[:n_req])}
    if len(_DUMP["layers"]) == st.L:
        torch.save(_DUMP["layers"], os.environ.get("LOCKS_DUMP_PATH",
                                                   "locks_dump.pt"))
        _DUMP["done"] = True
        print(f"[locks] dumped decode step {_DUMP['step']}", flush=True)


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
