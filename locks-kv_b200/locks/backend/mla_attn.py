"""MLA decode hook: ``LocksMLAImpl.forward_mqa`` selects pages of the latent
cache and attends only those; prefill stays stock MLA.  Same hook and result
``(o, lse)`` as the reference's ``backend/mla_attn.py:86-210``, but the whole
call is a fixed sequence of kernel launches with no host synchronisation: which
rows need (new) page factors is decided on the device (``mla_refresh_rows``), so
the hook can sit inside a captured decode graph.
"""
from __future__ import annotations

import torch
from vllm.v1.attention.backends.mla.triton_mla import (TritonMLABackend,
                                                       TritonMLAImpl)

from ..selection.mla_select import (HEADS, LKV, PAGE, ROPE, MlaState,
                                    mla_decode, mla_derive, mla_page_score,
                                    mla_refresh_rows, mla_select_pages)
from . import _runtime

_ANNOUNCED = False


def _budget_pages(cfg, max_pages: int) -> int:
    if cfg.budget_pages is not None and cfg.budget_pages > 0:
        return int(cfg.budget_pages)
    if cfg.budget is not None:
        import math
        return max(1, math.ceil(cfg.budget * max_pages))
    raise RuntimeError(
        "LOCKS MLA path requires a fixed budget: set 'budget_pages' (pages) or "
        "'budget' (fraction) in LOCKS_CONFIG")


class LocksMLAImpl(TritonMLAImpl):

    def __init__(self, *args, **kwargs):
        kwargs.pop("topk_indices_buffer", None)      # DSA-only kwarg, unused here
        super().__init__(*args, **kwargs)
        self._locks_state = None

    def _state(self, cache, bt, cfg):
        B, MP = bt.shape
        st = self._locks_state
        if st is not None and (B > st.max_rows or MP > st.max_pages or
                               cache.shape[0] > st.NB):
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("LOCKS MLA: the decode batch outgrew the "
                                   "selection state during graph capture")
            st = self._locks_state = None
        if self._locks_state is None:
            self._locks_state = MlaState(
                cache.device, num_layers=1, num_blocks=cache.shape[0],
                max_rows=max(B, 64), max_pages=MP,
                budget_pages=_budget_pages(cfg, MP), sink_pages=cfg.sink_pages,
                window_pages=cfg.window_pages)
        return self._locks_state

    def forward_mqa(self, q, kv_c_and_k_pe_cache, attn_metadata, layer):
        cfg = _runtime.get_config()
        assert cfg is not None, "LocksMLAImpl reached with no LocksConfig"
        if isinstance(q, tuple):
            q = torch.cat(q, dim=-1)
        B, H, HS = q.shape
        cache = kv_c_and_k_pe_cache
        assert HS == LKV + ROPE and cache.shape[1] == PAGE, \
            "LOCKS MLA (B200 build) supports kv_lora_rank 512 + rope 64, page 16"
        assert H <= HEADS, f"LOCKS MLA (B200 build) supports <= {HEADS} heads per rank"
        global _ANNOUNCED
        if not _ANNOUNCED:
            _ANNOUNCED = True
            print(f"[locks] ACTIVE (MLA) budget_pages={cfg.budget_pages} "
                  f"sink={cfg.sink_pages} window={cfg.window_pages}", flush=True)
        dec = attn_metadata.decode
        bt, seq_lens = dec.block_table, dec.seq_lens
        st = self._state(cache, bt, cfg)
        if H < HEADS:                                   # pad heads with zero rows
            qp = q.new_zeros(B, HEADS, HS)
            qp[:, :H] = q
            q = qp
        q = q.contiguous()
        # factors of rows seen for the first time (or whose blocks were reused):
        # flagged and rebuilt on the device
        mla_refresh_rows(st, 0, cache, bt, seq_lens, B)
        scale = float(self.scale)
        out = torch.empty(B, HEADS, LKV, dtype=torch.bfloat16, device=q.device)
        lse = torch.empty(B, HEADS, dtype=torch.float32, device=q.device)
        mla_derive(st, seq_lens, B)
        mla_page_score(st, 0, q, cache, bt, B, scale)
        mla_select_pages(st, B)
        mla_decode(st, q, cache, bt, seq_lens, out, lse, B, scale)
        return out[:, :H].to(q.dtype), lse[:, :H].to(q.dtype)


class LocksMLABackend(TritonMLABackend):
    """Triton MLA backend with the LOCKS impl; ``get_name()`` is inherited."""

    @staticmethod
    def get_impl_cls():
        return LocksMLAImpl
