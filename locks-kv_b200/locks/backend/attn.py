"""``LocksAttentionImpl`` -- the per-layer attention hook.

Pure single-token decode steps run page selection + sparse paged decode.  Steps
in which chunked prefill co-schedules a prompt chunk with decode rows are
SPLIT: the stock FlashAttention pass serves the whole batch (right for the
prefill rows), then the decode rows are recomputed on a compacted sub-batch
with the same derive -> select -> decode chain and written over their slots.
Everything else (cascade, sliding window, ALiBi, sinks, quantised KV,
non-decoder attention, no state) is delegated to the stock FlashAttention impl
this class inherits from.  Same gate list and call order as the reference's
``backend/attn.py:232-386`` (forward) and ``:514-624`` (batch-split);
``do_kv_cache_update`` (reference ``:389-509``) stores the step's K/V with this
library's write kernel and, in the last layer's call, builds the summaries of
the pages the step completed.
"""
from __future__ import annotations

import torch
from vllm.v1.attention.backends.flash_attn import FlashAttentionImpl

from . import _runtime

_ANNOUNCED = False
_KV_ANNOUNCED = False
_NO_STATE_WARNED = False


class LocksAttentionImpl(FlashAttentionImpl):

    # ---- gates ---------------------------------------------------------------
    def _locks_reasons(self, kv_cache, attn_metadata, output):
        """Names of the conditions that keep this call off the sparse path
        (empty = eligible)."""
        r = []
        cfg = _runtime.get_config()
        if cfg is None or cfg.variant != "fast":
            r.append("no-config")
        if attn_metadata is None or output is None:
            r.append("no-metadata")
            return r
        if getattr(attn_metadata, "locks", None) is None:
            r.append("no-state")
        if int(attn_metadata.max_query_len) != 1:
            r.append("max_query_len!=1")
        if kv_cache is None or kv_cache.numel() == 0:
            r.append("empty-cache")
        if getattr(attn_metadata, "use_cascade", False):
            r.append("cascade")
        if not getattr(attn_metadata, "causal", True):
            r.append("non-causal")
        at = str(getattr(self, "attn_type", None) or "decoder").lower()
        if "decoder" not in at or "encoder" in at:
            r.append("attn-type")
        sw = getattr(self, "sliding_window", None)
        if sw is not None and tuple(sw) != (-1, -1):
            r.append("sliding-window")
        if getattr(self, "alibi_slopes", None) is not None:
            r.append("alibi")
        if getattr(self, "sinks", None) is not None:
            r.append("sinks")
        if getattr(attn_metadata, "max_dcp_context_kv_len", None):
            r.append("dcp")
        if str(getattr(self, "kv_cache_dtype", "auto")).startswith("fp8"):
            r.append("fp8-kv")
        return r

    def _locks_eligible(self, kv_cache, attn_metadata, output) -> bool:
        return not self._locks_reasons(kv_cache, attn_metadata, output)

    # ---- forward ---------------------------------------------------------------
    def forward(self, layer, query, key, value, kv_cache, attn_metadata,
                output=None, output_scale=None, output_block_scale=None):
        global _ANNOUNCED, _NO_STATE_WARNED
        reasons = self._locks_reasons(kv_cache, attn_metadata, output)
        if reasons:
            m = attn_metadata
            if reasons == ["max_query_len!=1"] and \
                    getattr(m, "locks_qsl_cpu", None) is not None and \
                    not torch.cuda.is_current_stream_capturing():
                return self._forward_batchsplit(layer, query, key, value,
                                                kv_cache, m, output, output_scale,
                                                output_block_scale)
            # decode rows this delegation hands to the dense path (rows with one
            # query token; pure-prefill steps contribute none)
            if m is not None and _runtime.get_config() is not None and \
                    _runtime.get_config().variant == "fast" and \
                    not _runtime.in_profiling() and \
                    not torch.cuda.is_current_stream_capturing():
                n_dec = 0
                if int(getattr(m, "max_query_len", 0)) == 1:
                    n_dec = int(m.seq_lens.shape[0])
                elif getattr(m, "locks_qsl_cpu", None) is not None:
                    q = m.locks_qsl_cpu
                    n_dec = int(((q[1:] - q[:-1]) == 1).sum())
                _runtime.count_dense(n_dec, reasons[0])
                if reasons == ["no-state"] and n_dec and not _NO_STATE_WARNED:
                    _NO_STATE_WARNED = True
                    print("[locks] FALLBACK no-state: a decode step reached the "
                          "attention layers without a selection state (the "
                          "builder could not allocate or latch it); serving "
                          "full-KV attention", flush=True)
            return super().forward(layer, query, key, value, kv_cache,
                                   attn_metadata, output, output_scale,
                                   output_block_scale)
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
        if not torch.cuda.is_current_stream_capturing():
            _runtime.count_sparse(n_req)
            _runtime.dump_layer(_runtime._layer_index(st, kv_cache), q, kv_cache,
                                bt, sl, st, out3, n_req)
        return output

    def _forward_batchsplit(self, layer, query, key, value, kv_cache, m, output,
                            output_scale, output_block_scale):
        """A step that mixes prefill chunks and decode rows: dense pass for every
        row, then the decode rows again through the sparse path on a compacted
        sub-batch (same q, block-table rows and lengths as a pure decode step
        would see), overwriting their output rows.  Eager only: the engine
        captures graphs for uniform decode batches alone."""
        from ..attention import ResidentVSource
        from ..selection import derive_page_params
        super().forward(layer, query, key, value, kv_cache, m, output,
                        output_scale, output_block_scale)
        st, cfg = m.locks, _runtime.get_config()
        n_req = int(m.seq_lens.shape[0])
        bs = getattr(m, "_locks_bs_idx", None)
        if bs is None:              # step constants, shared by the step's layers
            qsl, sl_cpu = m.locks_qsl_cpu, m.locks_sl_cpu
            ql = (qsl[1:n_req + 1] - qsl[:n_req]).tolist()
            sl = sl_cpu[:n_req].tolist()
            rows = [r for r in range(n_req) if ql[r] == 1 and sl[r] > 0]
            dev = query.device
            bs = {"n": len(rows)}
            if rows:
                bs["rows"] = torch.tensor(rows, dtype=torch.long, device=dev)
                bs["tok"] = torch.tensor([int(qsl[r]) for r in rows],
                                         dtype=torch.long, device=dev)
                bs["bt"] = m.block_table.index_select(0, bs["rows"]).contiguous()
                bs["sl"] = m.seq_lens.index_select(0, bs["rows"]).contiguous()
            m._locks_bs_idx = bs
        n_dec = bs["n"]
        if n_dec == 0:
            return output
        if n_dec > st.max_reqs:
            _runtime.count_dense(n_dec, "more-decode-rows-than-state-rows")
            return output
        nt = int(m.num_actual_tokens)
        H = st.n_kv * st.G
        q3 = query[:nt].view(nt, H, st.d)
        out3 = output[:nt].view(nt, H, st.d)
        q_dec = q3.index_select(0, bs["tok"]).contiguous()
        out_dec = torch.empty_like(q_dec)
        _s, _d, select_pages, _g = _runtime.resolve_selection()
        derive_page_params(st, bs["sl"], n_dec)
        scale = float(self.scale)
        select_pages(q_dec, kv_cache, bs["bt"], bs["sl"], st, n_dec, scale, cfg)
        _runtime.decode_dispatch(q_dec, kv_cache, bs["bt"], bs["sl"], st, out_dec,
                                 ResidentVSource(kv_cache), scale, cfg)
        out3.index_copy_(0, bs["tok"], out_dec)
        _runtime.count_sparse(n_dec)
        return output

    # ---- KV write -----------------------------------------------------------------
    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
        """Store the step's K (already rotated by the model) and V rows with the
        library's write kernel; the call of the LAST layer then builds, in every
        layer, the summaries of the pages this step completed
        (``locks_rki4_build_slots``: decided on the device from the same
        ``slot_mapping``, fixed shape, so it sits inside a captured decode graph).
        The builder then has no tail refresh to do on steady decode steps."""
        st, K_layers = _runtime.get_state()
        cfg = _runtime.get_config()
        ok = (cfg is not None and cfg.variant == "fast" and st is not None
              and not _runtime.in_profiling()
              and isinstance(kv_cache, torch.Tensor) and kv_cache.numel() != 0
              and kv_cache.dtype == torch.bfloat16 and key is not None
              and key.dtype == torch.bfloat16 and value is not None
              and value.dtype == torch.bfloat16
              and slot_mapping.dtype == torch.int64
              and str(getattr(self, "kv_cache_dtype", "auto")) in ("auto", "bfloat16")
              and int(kv_cache.data_ptr()) in st._layer_of)
        if not ok:
            return super().do_kv_cache_update(layer, key, value, kv_cache,
                                              slot_mapping)
        from ..attention import rope_and_cache
        from ..selection import rki4_build_slots
        global _KV_ANNOUNCED
        if not _KV_ANNOUNCED:
            _KV_ANNOUNCED = True
            print("[locks] KV write ACTIVE (library write kernel; summaries of "
                  "completed pages built in the step that completes them)",
                  flush=True)
        n = int(slot_mapping.shape[0])
        k3 = key[:n].view(n, st.n_kv, st.d)
        v3 = value[:n].view(n, st.n_kv, st.d)
        rope_and_cache(k3, v3, kv_cache, slot_mapping, None, None)
        if st._layer_of[int(kv_cache.data_ptr())] == st.L - 1:
            rki4_build_slots(st, K_layers, slot_mapping)
            st._slots_built_in_forward = True
