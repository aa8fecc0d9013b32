"""``LocksAttentionImpl`` -- the per-layer attention hook.

Pure single-token decode steps run page selection + sparse paged decode;
everything else (prefill, mixed steps, cascade, sliding window, ALiBi, sinks,
quantised KV, non-decoder attention, no state) is delegated to the stock
FlashAttention impl it inherits from.  Same gate list and call order as the
reference's ``backend/attn.py:232-386``.
"""
from __future__ import annotations

import torch
from vllm.v1.attention.backends.flash_attn import FlashAttentionImpl

from . import _runtime

_ANNOUNCED = False


class LocksAttentionImpl(FlashAttentionImpl):

    def _locks_eligible(self, kv_cache, attn_metadata, output) -> bool:
        cfg = _runtime.get_config()
        if cfg is None or cfg.variant != "fast":
            return False
        if attn_metadata is None or output is None:
            return False
        if getattr(attn_metadata, "locks", None) is None:
            return False
        if int(attn_metadata.max_query_len) != 1:
            return False
        if kv_cache is None or kv_cache.numel() == 0:
            return False
        if getattr(attn_metadata, "use_cascade", False):
            return False
        if not getattr(attn_metadata, "causal", True):
            return False
        if getattr(self, "attn_type", "decoder") not in ("decoder", None) and \
                str(getattr(self, "attn_type", "decoder")).lower().find("decoder") < 0:
            return False
        sw = getattr(self, "sliding_window", None)
        if sw is not None and tuple(sw) != (-1, -1):
            return False
        if getattr(self, "alibi_slopes", None) is not None:
            return False
        if getattr(self, "sinks", None) is not None:
            return False
        if getattr(attn_metadata, "max_dcp_context_kv_len", None):
            return False
        if str(getattr(self, "kv_cache_dtype", "auto")).startswith("fp8"):
            return False
        return True

    def forward(self, layer, query, key, value, kv_cache, attn_metadata,
                output=None, output_scale=None, output_block_scale=None):
        if not self._locks_eligible(kv_cache, attn_metadata, output):
            return super().forward(layer, query, key, value, kv_cache,
                                   attn_metadata, output, output_scale,
                                   output_block_scale)
        global _ANNOUNCED
        cfg = _runtime.get_config()
        st = attn_metadata.locks
        n_req = int(attn_metadata.seq_lens.shape[0])
        n_tok = int(attn_metadata.num_actual_tokens)
        if not _ANNOUNCED:
            _ANNOUNCED = True
            print(f"[locks] sparse decode ACTIVE (budget_pages={cfg.budget_pages} "
                  f"budget={cfg.budget} sink={cfg.sink_pages} "
                  f"window={cfg.window_pages})", flush=True)
        _state_cls, _derive, select_pages, _ = _runtime.resolve_selection()
        q = query[:n_tok].view(n_tok, st.n_kv * st.G, st.d)
        out3 = output[:n_tok].view(n_tok, st.n_kv * st.G, st.d)
        bt, sl = attn_metadata.block_table, attn_metadata.seq_lens
        scale = float(self.scale)
        select_pages(q, kv_cache, bt, sl, st, n_req, scale, cfg)
        from ..attention import ResidentVSource
        _runtime.decode_dispatch(q, kv_cache, bt, sl, st, out3,
                                 ResidentVSource(kv_cache), scale, cfg)
        return output
