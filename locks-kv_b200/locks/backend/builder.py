"""``LocksMetadataBuilder`` -- per-step host prologue of the decode hot path.

Keeps the page summaries valid under continuous batching and publishes the
selection state to the attention impl as ``md.locks``.  Same hooks and the same
refresh rules as the reference's ``backend/builder.py`` (state allocation
:658-787, ``build`` :1001-1136, refresh gate :1138-1282):

  steady step, no page boundary crossed       -> nothing
  steady step, some rows settled a full page  -> tail build for those rows
                                                 (one step AFTER the boundary:
                                                 the just-decoded token's K is
                                                 written by the forward that runs
                                                 after this prologue)
  anything else (first decode, arrivals,
  drain shuffles, preemption, slot reuse)     -> bulk build the first time, then
                                                 tag-scan delta builds

Lengths are SETTLED tokens = seq_lens - query_len.  The decision itself is the
host-only :class:`RefreshGate`; the vLLM-facing class is thin around it.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _runtime

try:  # vLLM is the plugin host; the gate below is usable without it
    from vllm.v1.attention.backends.flash_attn import \
        FlashAttentionMetadataBuilder
    _HAVE_VLLM = True
except Exception:  # pragma: no cover
    FlashAttentionMetadataBuilder = object
    _HAVE_VLLM = False


class RefreshGate:
    """Host-side decision of what the summary build has to do this step.

    ``decide(cur, cur_st)`` takes CPU int tensors of the rows' sequence lengths
    (including this step's query tokens) and settled lengths, and returns
    ``(action, rows, need_derive, max_fin)`` with ``action`` one of ``"skip"``,
    ``"tail"``, ``"delta"``, ``"bulk"``; ``rows`` (tail only) are the row
    indices whose last settled page just became complete.
    """

    def __init__(self, page: int):
        self.page = int(page)
        self.prev: Optional[torch.Tensor] = None
        self.prev_st: Optional[torch.Tensor] = None
        self.built_once = False
        # set by a step that left other rows' page parameters in the state (the
        # batch-split of a mixed step): the next decision asks for a derive
        self.derive_pending = False

    def reset(self) -> None:
        self.prev = self.prev_st = None

    def decide(self, cur: torch.Tensor, cur_st: torch.Tensor):
        page = self.page
        prev, prev_st = self.prev, self.prev_st
        full, crossed = True, None
        if (prev is not None and prev.shape == cur.shape
                and prev_st is not None and prev_st.shape == cur_st.shape):
            # steady = decoded exactly one token this step AND last step
            adv = (cur == prev + 1) & (cur_st == prev_st + 1)
            pad = (cur == 0) & (prev == 0)            # padded graph rows
            frozen = (cur == prev) & (cur_st == prev_st)   # drain replays
            if bool(torch.all(adv | pad | frozen)):
                full = False
                crossed = (cur_st % page == 0) & adv
        self.prev, self.prev_st = cur.clone(), cur_st.clone()
        pending, self.derive_pending = self.derive_pending, False
        if full:
            max_fin = int(cur_st.max().item()) // page if cur_st.numel() else 0
            action = "delta" if self.built_once else "bulk"
            self.built_once = True
            return action, None, True, max_fin
        if bool(crossed.any()):
            return "tail", torch.nonzero(crossed).squeeze(-1), True, 0
        return "skip", None, pending, 0


def settled_lengths(seq_lens_cpu: torch.Tensor, query_start_loc_cpu: torch.Tensor,
                    n_req: int):
    """(cur, cur_st): sequence lengths and settled lengths of the first
    ``n_req`` rows (reference ``builder.py:1363-1375``)."""
    cur = seq_lens_cpu[:n_req]
    qlen = (query_start_loc_cpu[1:n_req + 1] - query_start_loc_cpu[:n_req]).to(cur.dtype)
    return cur, (cur - qlen).clamp_(min=0)


class LocksMetadataBuilder(FlashAttentionMetadataBuilder):
    """FlashAttention metadata builder + LOCKS selection state.

    The state (:class:`locks.selection.Rki4State`) is allocated lazily at the
    first ``build`` that sees the engine's block count; its tensors never move
    afterwards, so the per-layer launches capture into the FULL decode graph.
    """

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        self._locks_cfg = _runtime.get_config()
        self._locks_state = None
        self._locks_ptrs = None          # data pointers the state was latched on
        self._locks_rows = None          # pinned + device row-index buffer pairs
        self._locks_rows_i = 0
        self._locks_settled = None
        self._locks_gate = RefreshGate(int(kv_cache_spec.block_size))
        self._locks_layers = list(layer_names)
        self._locks_vllm_config = vllm_config
        self._locks_device = device
        self._locks_spec = kv_cache_spec
        self._locks_caches = None

    @classmethod
    def get_cudagraph_support(cls, vllm_config, kv_cache_spec):
        """Pure single-token decode batches run the whole layer chain inside
        the captured graph (reference ``builder.py:526-541``)."""
        from vllm.v1.attention.backend import AttentionCGSupport
        return AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE

    # ---- state -------------------------------------------------------------
    def _layer_caches(self):
        """The engine's per-layer KV-cache tensors, or None while unbound."""
        ctx = self._locks_vllm_config.compilation_config.static_forward_context
        caches = []
        for name in self._locks_layers:
            kvc = getattr(ctx.get(name), "kv_cache", None)
            kvc = kvc[0] if isinstance(kvc, (list, tuple)) else kvc
            if not isinstance(kvc, torch.Tensor) or kvc.numel() == 0:
                return None
            caches.append(kvc)
        return caches

    def _ensure_state(self):
        if self._locks_cfg is None:
            return None
        # vLLM's graph-memory profiling runs against a throw-away minimal cache
        # (with num_gpu_blocks set): a state latched on it would key its
        # kv-cache -> layer map to pointers freed moments later (reference
        # backend/builder.py:658-672).  Two guards: the window register()
        # brackets, and a check that the latched pointers are still the engine's.
        if _runtime.in_profiling():
            return None
        if self._locks_state is not None:
            caches = self._layer_caches()
            if caches is not None and \
                    tuple(int(c.data_ptr()) for c in caches) == self._locks_ptrs:
                return self._locks_state
            print("[locks] the engine's KV caches moved (profiling cache "
                  "replaced): selection state rebuilt", flush=True)
            self._locks_state = None
            self._locks_gate = RefreshGate(int(self._locks_spec.block_size))
            _runtime.set_state(None, None)
        cfg, spec = self._locks_cfg, self._locks_spec
        vcfg = self._locks_vllm_config
        num_blocks = getattr(vcfg.cache_config, "num_gpu_blocks", None)
        if not num_blocks:
            return None                                   # cache not allocated yet
        caches = self._layer_caches()
        if caches is None:
            return None
        from ..attention import ensure_stage_b_buffers
        from ..attention.decode import _split_kv
        from ..selection import Rki4State
        n_kv, d, page = spec.num_kv_heads, spec.head_size, spec.block_size
        n_q = vcfg.model_config.get_num_attention_heads(vcfg.parallel_config)
        G = n_q // n_kv
        Rki4State.validate_geometry(head_dim=d, G=G, page=page)   # fail loudly
        max_reqs = vcfg.scheduler_config.max_num_seqs
        max_pages = -(-vcfg.model_config.max_model_len // page)
        nb_cache = int(_split_kv(caches[0])[0].shape[0])
        st = Rki4State(self._locks_device, num_layers=len(caches),
                       num_blocks=max(int(num_blocks), nb_cache), n_kv=n_kv, G=G,
                       head_dim=d, page=page, max_reqs=max_reqs,
                       max_pages=max_pages,
                       budget=cfg.budget if cfg.budget is not None else 0.1,
                       budget_pages=cfg.budget_pages, sink_pages=cfg.sink_pages,
                       window_pages=cfg.window_pages, combine=cfg.quad_combine,
                       zsplit=cfg.rki4_zsplit)
        st.scale = float(d) ** -0.5
        st._layer_of = {int(c.data_ptr()): i for i, c in enumerate(caches)}
        st._slots_built_in_forward = False
        ensure_stage_b_buffers(st, self._locks_device, 128)
        self._locks_caches = caches
        self._locks_ptrs = tuple(int(c.data_ptr()) for c in caches)
        self._locks_K = [_split_kv(c)[0] for c in caches]
        self._locks_state = st
        # row-index staging: two pinned + device pairs used in turn, so that the
        # copy of one step never waits for the replay of the step before
        # (reference builder ``_rows_to_device``)
        self._locks_rows = [
            (torch.zeros(max_reqs, dtype=torch.int64).pin_memory(),
             torch.zeros(max_reqs, dtype=torch.int64, device=self._locks_device))
            for _ in range(2)]
        self._locks_settled = torch.zeros(max_reqs, dtype=torch.int32,
                                          device=self._locks_device)
        _runtime.set_state(st, self._locks_K)
        print(f"[locks] state allocated: {len(caches)} layers, {num_blocks} blocks, "
              f"n_kv={n_kv} G={G} d={d} page={page}, "
              f"{st.bytes_per_layer() * len(caches) / 2**30:.2f} GiB summaries",
              flush=True)
        return st

    # ---- per step ------------------------------------------------------------
    def build(self, common_prefix_len, common_attn_metadata, fast_build=False):
        md = super().build(common_prefix_len, common_attn_metadata, fast_build)
        md.locks = None
        md.locks_qsl_cpu = md.locks_sl_cpu = None
        st = self._ensure_state()
        if st is None:
            return md
        cam = common_attn_metadata
        n_req = int(cam.num_reqs)
        sl_cpu = getattr(cam, "seq_lens_cpu_upper_bound", None)
        if sl_cpu is None:
            sl_cpu = getattr(cam, "_seq_lens_cpu", None)
        qs_cpu = getattr(cam, "query_start_loc_cpu", None)
        if sl_cpu is None or qs_cpu is None or sl_cpu.shape[0] < n_req or \
                qs_cpu.shape[0] < n_req + 1:
            sl_cpu = cam.seq_lens[:n_req].cpu()          # one sync, conservative
            qs_cpu = cam.query_start_loc[:n_req + 1].cpu()
        cur, cur_st = settled_lengths(sl_cpu, qs_cpu, n_req)
        pure_decode = int(cam.max_query_len) == 1
        if not pure_decode:
            # A mixed step: chunked prefill rides along with decode rows.  Those
            # rows are served by the attention impl's batch-split forward, which
            # reads the summaries, so this step refreshes them as a decode step
            # would and hands over the host views it needs (reference
            # backend/builder.py:1040-1066).  Pure-prefill steps need nothing.
            qlen = qs_cpu[1:n_req + 1] - qs_cpu[:n_req]
            if torch.cuda.is_current_stream_capturing() or \
                    not bool((qlen == 1).any()):
                self._locks_gate.reset()
                return md
            md.locks_qsl_cpu, md.locks_sl_cpu = qs_cpu, sl_cpu
        else:
            _runtime.dump_step_begin()
        self._refresh(st, md, cam, cur, cur_st, n_req, derive=pure_decode)
        if not pure_decode:
            self._locks_gate.derive_pending = True
        md.locks = st
        return md

    def _rows_to_device(self, rows: torch.Tensor) -> torch.Tensor:
        host, dev = self._locks_rows[self._locks_rows_i]
        self._locks_rows_i ^= 1
        n = int(rows.numel())
        host[:n].copy_(rows)
        dev[:n].copy_(host[:n], non_blocking=True)
        return dev[:n]

    def _refresh(self, st, md, cam, cur, cur_st, n_req, derive=True):
        from ..selection import (derive_page_params, rki4_build_bulk,
                                 rki4_build_delta, rki4_build_tail)
        action, rows, need_derive, max_fin = self._locks_gate.decide(cur, cur_st)
        if getattr(st, "_slots_built_in_forward", False):
            # the KV-write hook builds every page in the step that completes it:
            # a steady step has no tail to build, and the first decode step only
            # has to find what the hook did not see (a tag scan)
            if action == "tail":
                action = "skip"
            elif action == "bulk":
                action = "delta"
        bt, sl = md.block_table, md.seq_lens
        # settled tokens = those of earlier steps (this step's K is written by
        # the forward that runs after this prologue)
        settled = self._locks_settled[:n_req]
        qsl = md.query_start_loc
        torch.sub(sl[:n_req], (qsl[1:n_req + 1] - qsl[:n_req]).to(sl.dtype),
                  out=settled)
        settled.clamp_(min=0)
        if action == "bulk":
            rki4_build_bulk(st, self._locks_K, bt, settled, n_req, max_fin)
        elif action == "delta":
            rki4_build_delta(st, self._locks_K, bt, settled, n_req, max_fin)
        elif action == "tail":
            rki4_build_tail(st, self._locks_K, bt, settled, n_req,
                            self._rows_to_device(rows))
        if need_derive and derive:
            derive_page_params(st, sl, n_req)
