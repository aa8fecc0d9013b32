"""Attention-only driver of the decode hot path (what a model runner does
around the kernels, without the model).

``HotPath`` owns an :class:`Rki4State` for a set of per-layer paged KV caches,
keeps the summaries valid (bulk build at start, tail build when a page
finalises) and runs one decode step -- for every layer: score, select, sparse
decode, merge -- as a single CUDA-graph replay.  It calls exactly the functions
the vLLM hooks call (``backend/_runtime.py``).  Used by the benchmark, the
smoke test and the end-to-end tests.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import _cabi
from .attention import ResidentVSource, ensure_stage_b_buffers
from .backend import _runtime
from .config import LocksConfig
from .selection import (Rki4State, append_advance, derive_page_params,
                        rki4_build_bulk, rki4_build_slots, rki4_build_tail)


class HotPath:
    def __init__(self, kv_caches: List[torch.Tensor], block_table: torch.Tensor,
                 seq_lens: torch.Tensor, *, n_kv: int, G: int, scale: float,
                 cfg: LocksConfig, max_reqs: Optional[int] = None,
                 split_cap: int = 128, budget_pages_req=None,
                 launch_layers: Optional[int] = None):
        """``launch_layers``: run that many layer launches per step, cycling
        over the ``kv_caches`` given (layer launch l uses cache l % len): a
        benchmark whose full set of layer slabs would not fit in memory keeps
        a few distinct slabs -- each far larger than L2 -- and walks them in
        turn.  q / out are per launch."""
        dev = kv_caches[0].device
        self.device = dev
        self.cfg = cfg
        self.kv_caches = kv_caches
        self.block_table = block_table
        self.seq_lens = seq_lens
        self.n_req = int(seq_lens.shape[0])
        self.n_kv, self.G, self.scale = n_kv, G, float(scale)
        NB, _, page, _, d = kv_caches[0].shape
        self.page, self.d = int(page), int(d)
        L = len(kv_caches)
        self.launch_layers = int(launch_layers or L)
        st = Rki4State(dev, num_layers=L, num_blocks=int(NB), n_kv=n_kv, G=G,
                       head_dim=int(d), page=int(page),
                       max_reqs=max_reqs or self.n_req,
                       max_pages=int(block_table.shape[1]),
                       budget=cfg.budget if cfg.budget is not None else 0.1,
                       budget_pages=cfg.budget_pages,
                       sink_pages=cfg.sink_pages,
                       window_pages=cfg.window_pages,
                       combine=cfg.quad_combine, zsplit=cfg.rki4_zsplit)
        st.scale = self.scale
        st._layer_of = {int(c.data_ptr()): i for i, c in enumerate(kv_caches)}
        if budget_pages_req is not None:       # one page budget per request row
            st.set_request_budgets(budget_pages_req)
            st.budget_abs = max(int(max(budget_pages_req)), st.budget_abs)
        ensure_stage_b_buffers(st, dev, split_cap)
        self.st = st
        self.K_layers = [c[:, 0] for c in kv_caches]
        self.vsources = [ResidentVSource(c) for c in kv_caches]
        H = n_kv * G
        LL = self.launch_layers
        self.q = torch.zeros(LL, st.max_reqs, H, d, device=dev, dtype=torch.bfloat16)
        self.out = torch.zeros(LL, st.max_reqs, H, d, device=dev, dtype=torch.bfloat16)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_step = 0
        self.vtier = None

    # ---- summaries ---------------------------------------------------------
    def build_all(self) -> int:
        settled = self.seq_lens - 1
        max_fin = int((settled.max().item()) // self.page)
        return rki4_build_bulk(self.st, self.K_layers, self.block_table, settled,
                               self.n_req, max_fin)

    def build_tail(self, rows=None) -> int:
        return rki4_build_tail(self.st, self.K_layers, self.block_table,
                               self.seq_lens - 1, self.n_req, rows)

    def derive(self) -> None:
        derive_page_params(self.st, self.seq_lens, self.n_req)

    # ---- one decode step ---------------------------------------------------
    def _layers(self) -> None:
        st, R = self.st, self.n_req
        n = len(self.kv_caches)
        for l in range(self.launch_layers):
            kvc = self.kv_caches[l % n]
            q = self.q[l, :R]
            _runtime._rki4_select_adapter(q, kvc, self.block_table,
                                          self.seq_lens, st, R, self.scale,
                                          self.cfg)
            _runtime.decode_dispatch(q, kvc, self.block_table, self.seq_lens, st,
                                     self.out[l], self.vsources[l % n], self.scale,
                                     self.cfg)

    def step_eager(self) -> torch.Tensor:
        if self.vtier is not None:
            self.vtier.promote()         # last step's missed blocks come in
        self._layers()
        if self.vtier is not None:
            self.vtier.end_step()        # this step's residency notes go back
        return self.out

    def enable_vtier(self, n_slots: int, **kw):
        """Move V behind the two-level tier (``locks.attention.vtier``): the V
        planes are copied to pinned host memory, the decode reads selected pages
        from a staging buffer of ``n_slots`` blocks per layer or, on a miss, in
        place from the host; ``step_eager`` / ``step`` promote the misses
        between steps.  The resident V halves are no longer read."""
        from .attention.vtier import VTier
        assert self.launch_layers == len(self.kv_caches)
        self.vtier = VTier(self.kv_caches, n_slots, **kw)
        self.vsources = [self.vtier.vsource(l) for l in range(len(self.kv_caches))]
        self.graph = None
        return self.vtier

    def capture(self) -> None:
        """Warm up (first-launch attribute set-up must happen outside capture)
        and record the whole L-layer step into one CUDA graph."""
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._layers()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        n0 = _cabi.launches
        with torch.cuda.graph(g):
            self._layers()
        self.launches_per_step = _cabi.launches - n0
        self.graph = g

    def step(self) -> torch.Tensor:
        if self.graph is None:
            self.capture()
        if self.vtier is not None:       # the promotion copies stay outside the graph
            self.vtier.promote()
            self.vtier.wait_all()
        self.graph.replay()
        if self.vtier is not None:
            self.vtier.end_step()
        return self.out

    # ---- one step fed from, and read back to, host memory ----------------------
    def enable_host_io(self) -> None:
        """Pinned host staging for a caller whose tensors live in host memory:
        ``host_q`` (L, R, H, d), ``host_seq_lens``, ``host_block_table`` are
        written by the caller before ``step_host``; ``host_out`` holds the
        result after it."""
        R = self.n_req
        pin = lambda t: torch.empty(t.shape, dtype=t.dtype).pin_memory()
        self.host_q = pin(self.q[:, :R])
        self.host_seq_lens = pin(self.seq_lens)
        self.host_block_table = pin(self.block_table)
        self.host_out = pin(self.out[:, :R])
        self.io_graph: Optional[torch.cuda.CUDAGraph] = None

    def _io_step(self) -> None:
        R = self.n_req
        self.q[:, :R].copy_(self.host_q, non_blocking=True)
        self.seq_lens.copy_(self.host_seq_lens, non_blocking=True)
        self.block_table.copy_(self.host_block_table, non_blocking=True)
        self.derive()
        self._layers()
        self.host_out.copy_(self.out[:, :R], non_blocking=True)

    def step_host(self) -> torch.Tensor:
        """Host buffers in, host buffer out: the three host-to-device copies,
        the page parameters, the L-layer step and the device-to-host copy are
        ONE graph replay (copy nodes read and write the pinned buffers in
        place), followed by a stream synchronise -- ``host_out`` is valid on
        return."""
        if self.io_graph is None:
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._io_step()
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._io_step()
            self.io_graph = g
        self.io_graph.replay()
        torch.cuda.current_stream().synchronize()
        return self.host_out

    # ---- decode loop: append one token per request, then attend --------------
    def enable_append(self, cos_sin: Optional[torch.Tensor] = None,
                      neox: bool = True, fuse_write: bool = True) -> None:
        """Allocate what ``append_step`` needs: the new token's K/V per layer
        (``new_k`` / ``new_v``, (L, R, n_kv, d) bf16, filled by the caller
        before each step), the slot and position vectors it derives on the
        device, and the side stream of the summary build.  ``cos_sin`` is the
        (positions, rot_dim) cos|sin table of the rotation, or None for K that
        arrives rotated.  The block table must hold a block for every page the
        appended tokens reach.  ``fuse_write``: the selector's launch stores
        the token (no KV-write launch); otherwise ``locks_kv_write`` runs in
        front of every layer."""
        from .attention import kv_append_desc, rope_and_cache
        dev, R, L = self.device, self.n_req, len(self.kv_caches)
        self._rope_and_cache = rope_and_cache
        self._fuse_write = bool(fuse_write)
        self.cos_sin, self.neox = cos_sin, neox
        self.new_k = torch.zeros(L, R, self.n_kv, self.d, device=dev,
                                 dtype=torch.bfloat16)
        self.new_v = torch.zeros_like(self.new_k)
        self.pos = torch.zeros(R, dtype=torch.int64, device=dev)
        self.slot = torch.full((R,), -1, dtype=torch.int64, device=dev)
        self.slot_prev = torch.full((R,), -1, dtype=torch.int64, device=dev)
        self._side = torch.cuda.Stream(device=dev)
        self.append_graph: Optional[torch.cuda.CUDAGraph] = None
        pos = self.pos if cos_sin is not None else None
        self._append_desc = [
            kv_append_desc(self.new_k[l], self.new_v[l], kvc, self.slot, pos,
                           cos_sin, neox=neox)
            for l, kvc in enumerate(self.kv_caches)] if fuse_write else None

    def _append_step(self) -> None:
        """One decode step as a model runs it, every decision on the device:
        the token index is the current length; its slot comes from the block
        table; lengths grow by one and the page parameters follow; each layer
        rotates and stores the token, scores, selects and decodes.  Summaries
        of the pages the PREVIOUS step completed are built first.  With a
        recent window of two pages or more such a page is still inside the
        window during this step (no layer scores it), so the build runs on a
        forked branch and is joined at the end of the step.  With a window of
        one page (the default of ``LocksConfig``) the page completed by the
        previous step is scored by THIS step, so the build stays on the main
        stream in front of the first scorer -- the order the reference keeps
        (tail build before the forward of the step, ``backend/builder.py:
        1230-1245``)."""
        cur = torch.cuda.current_stream()
        append_advance(self.st, self.seq_lens, self.block_table, self.n_req,
                       self.slot, self.slot_prev, self.pos)
        forked = self.st.window_pages >= 2
        if forked:
            self._side.wait_stream(cur)
            with torch.cuda.stream(self._side):
                rki4_build_slots(self.st, self.K_layers, self.slot_prev)
        else:
            rki4_build_slots(self.st, self.K_layers, self.slot_prev)
        st, R = self.st, self.n_req
        for l, kvc in enumerate(self.kv_caches):
            if not self._fuse_write:
                self._rope_and_cache(self.new_k[l], self.new_v[l], kvc, self.slot,
                                     self.pos if self.cos_sin is not None else None,
                                     self.cos_sin, neox=self.neox)
            q = self.q[l, :R]
            _runtime._rki4_select_adapter(
                q, kvc, self.block_table, self.seq_lens, st, R, self.scale,
                self.cfg,
                append=self._append_desc[l] if self._fuse_write else None)
            _runtime.decode_dispatch(q, kvc, self.block_table, self.seq_lens, st,
                                     self.out[l], self.vsources[l], self.scale,
                                     self.cfg)
        if forked:
            cur.wait_stream(self._side)

    def append_step(self) -> torch.Tensor:
        """Replay the captured append-and-attend step (captured on first use;
        the capture's warm-up run is itself one real step)."""
        if self.append_graph is None:
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._append_step()
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._append_step()
            self.append_graph = g
            return self.out
        self.append_graph.replay()
        return self.out

    def flush_builds(self) -> None:
        """Build the summaries of pages completed by the last appended token
        (``append_step`` leaves them to the following step)."""
        rki4_build_slots(self.st, self.K_layers, self.slot)
        self.slot.fill_(-1)
