"""MLA (latent KV) page selection and decode -- host side.

DeepSeek-style MLA keeps ONE latent head (kv_lora_rank 512 + 64 rope channels)
shared by all query heads; the page score is the max over heads and tokens of
the logit reconstructed from a rank-8 factorisation of the page's latent block
plus the exact rope part (reference ``selection/mla_select.py``,
``selection/mla_score_torch.py``, ``backend/mla_attn.py:86-210``).

Differences from the reference's data layout, none in the algorithm:
  * factors are stored per PHYSICAL BLOCK as fp16 records (Rf 8x512, Lf 16x8 =
    8448 B; the reference keeps fp32 rank-16-padded factors, 37.9 KB per page)
    and the rope keys are read from the latent cache instead of being copied;
  * scoring, the keep rule, and the attention are kernels (no host sync, no
    per-row Python loops), so a decode step is graph-capturable.

``n_cache[row]`` = number of leading pages of the row that have factors; like
the reference, pages generated after the factors were built are scored -inf and
are attended only while they sit inside the recent window.
"""
from __future__ import annotations

import torch

from .. import _cabi

MLA_REC_BYTES = 8448
LKV, ROPE, HEADS, PAGE = 512, 64, 16, 16


class MlaState:
    """Factor records + per-step selection outputs of the MLA path."""

    def __init__(self, device, *, num_layers: int, num_blocks: int,
                 max_rows: int, max_pages: int, budget_pages: int,
                 sink_pages: int = 1, window_pages: int = 1, rank: int = 8):
        assert rank == 8, "the MLA factor rank is fixed at 8"
        assert budget_pages >= 1
        i32, f32 = torch.int32, torch.float32
        self.L, self.NB = num_layers, num_blocks
        self.max_rows, self.max_pages = max_rows, max_pages
        self.budget_pages = int(budget_pages)
        self.sink_pages, self.window_pages = int(sink_pages), int(window_pages)
        self.records = torch.zeros(num_layers, num_blocks, MLA_REC_BYTES,
                                   device=device, dtype=torch.uint8)
        self.n_cache = torch.zeros(max_rows, device=device, dtype=i32)
        self.n_pages = torch.zeros(max_rows, device=device, dtype=i32)
        self.n_sel_hi = torch.zeros(max_rows, device=device, dtype=i32)
        self.b_fix = torch.zeros(max_rows, device=device, dtype=i32)
        self.score = torch.zeros(max_rows, 1, max_pages, device=device, dtype=f32)
        self.page_table = torch.full((max_rows, 1, max_pages), -1, device=device,
                                     dtype=i32)
        self.page_cnt = torch.zeros(max_rows, 1, device=device, dtype=i32)
        self.status = torch.zeros(1, device=device, dtype=i32)
        # device-side factor bookkeeping (mla_refresh_rows): per layer and first
        # block id a content fingerprint and the pages its factors cover
        self.fp_tab = torch.zeros(num_layers, num_blocks, device=device, dtype=f32)
        self.nc_tab = torch.full((num_layers, num_blocks), -1, device=device,
                                 dtype=i32)
        self.need = torch.zeros(max_rows, device=device, dtype=i32)

    def factors(self, layer: int, blocks):
        """(Lf (n,16,8), Rf (n,8,512)) fp32 views of the listed blocks (tests)."""
        rec = self.records[layer][blocks.long()]
        Rf = rec[:, :8192].contiguous().view(torch.float16).view(-1, 8, LKV)
        Lf = rec[:, 8192:].contiguous().view(torch.float16).view(-1, PAGE, 8)
        return Lf.float(), Rf.float()

    def check_status(self) -> None:
        s = int(self.status.item())
        if s != 0:
            self.status.zero_()
            raise RuntimeError(f"a LOCKS kernel reported status {s}")


def _check_cache(cache):
    assert cache.dtype == torch.bfloat16 and cache.dim() == 3
    assert cache.shape[1] == PAGE and cache.shape[2] == LKV + ROPE, \
        f"latent cache must be (num_blocks, 16, 576), got {tuple(cache.shape)}"
    assert cache.stride(2) == 1


def build_page_factors(st: MlaState, layer: int, cache, blocks) -> int:
    """Rank-8 factors of the listed physical blocks of one layer (one launch)."""
    _check_cache(cache)
    if blocks.numel() == 0:
        return 0
    b32 = blocks.to(torch.int32).contiguous()
    _cabi.call("locks_mla_build_factors", _cabi.ptr(cache), cache.stride(0),
               cache.stride(1), _cabi.ptr(st.records[layer]), _cabi.ptr(b32),
               int(b32.numel()), int(min(st.NB, cache.shape[0])), _cabi.stream())
    return int(b32.numel())


def build_prompt_factors(st: MlaState, caches, block_table, seq_lens, rows=None):
    """Factors for every FULL page of the given rows in all layers and
    ``n_cache[row] = seq_len // 16`` (what the reference does at a row's first
    decode step, ``backend/mla_attn.py:212-239``)."""
    rows = list(range(int(seq_lens.shape[0]))) if rows is None else list(rows)
    sl = seq_lens.tolist()
    blocks = []
    for r in rows:
        nc = sl[r] // PAGE
        if nc > 0:
            blocks.append(block_table[r, :nc])
        st.n_cache[r] = nc
    if not blocks:
        return 0
    blocks = torch.cat(blocks)
    for l, cache in enumerate(caches):
        build_page_factors(st, l, cache, blocks)
    return int(blocks.numel()) * len(caches)


def mla_refresh_rows(st: MlaState, layer: int, cache, block_table, seq_lens,
                     n_rows: int) -> None:
    """Keep the factors of a decode batch valid with NO host synchronisation:
    a gate kernel flags the rows whose factors are missing or stale (first
    decode step, block ids reused by another request, a row that shrank) and
    sets ``st.n_cache``; the factor kernel rebuilds the flagged rows' pages.
    Fixed launch shapes: usable inside a captured graph.  What the reference's
    ``_factors`` does on the host with one ``.tolist()`` per step
    (``backend/mla_attn.py:118-133, 212-239``)."""
    _check_cache(cache)
    assert n_rows <= st.max_rows and block_table.shape[1] <= st.max_pages
    _cabi.call("locks_mla_refresh_rows", _cabi.ptr(cache), cache.stride(0),
               cache.stride(1), _cabi.ptr(st.records[layer]),
               _cabi.ptr(block_table), block_table.stride(0), _cabi.ptr(seq_lens),
               _cabi.ptr(st.fp_tab[layer]), _cabi.ptr(st.nc_tab[layer]),
               _cabi.ptr(st.need), _cabi.ptr(st.n_cache), int(n_rows),
               int(block_table.shape[1]), int(min(st.NB, cache.shape[0])),
               _cabi.stream())


def mla_derive(st: MlaState, seq_lens, n_rows: int) -> None:
    _cabi.call("locks_mla_derive", _cabi.ptr(seq_lens), int(n_rows),
               st.budget_pages, st.sink_pages, st.window_pages,
               _cabi.ptr(st.n_pages), _cabi.ptr(st.n_sel_hi), _cabi.ptr(st.b_fix),
               _cabi.stream())


def mla_page_score(st: MlaState, layer: int, q, cache, block_table, n_rows: int,
                   scale: float) -> None:
    """``st.score[row, 0, p]`` for every page with factors (-inf beyond)."""
    _check_cache(cache)
    assert q.dtype == torch.bfloat16 and q.shape[1] == HEADS \
        and q.shape[2] == LKV + ROPE and q.stride(2) == 1 and q.stride(1) == LKV + ROPE
    _cabi.call("locks_mla_score", _cabi.ptr(q), q.stride(0),
               _cabi.ptr(st.records[layer]), _cabi.ptr(cache), cache.stride(0),
               cache.stride(1), _cabi.ptr(block_table), block_table.stride(0),
               _cabi.ptr(st.n_cache), _cabi.ptr(st.n_pages), _cabi.ptr(st.score),
               int(n_rows), int(st.max_pages), int(min(st.NB, cache.shape[0])),
               float(scale), 0, _cabi.ptr(st.status), _cabi.stream())


def mla_select_pages(st: MlaState, n_rows: int) -> None:
    """Keep rule of ``topb_middle``: all pages when they fit the budget, else
    sink + recent window forced and the best-scored middle pages fill the rest
    (same exact-b kernel as the GQA selector, one "kv head")."""
    _cabi.call("locks_topb_select", 0, _cabi.ptr(None), _cabi.ptr(st.score),
               _cabi.ptr(None), _cabi.ptr(st.n_pages), _cabi.ptr(st.n_sel_hi),
               _cabi.ptr(st.b_fix), _cabi.ptr(st.page_table),
               _cabi.ptr(st.page_cnt), int(n_rows), 1, 1, int(st.max_pages),
               int(st.sink_pages), _cabi.stream())


def mla_decode(st: MlaState, q, cache, block_table, seq_lens, out, lse,
               n_rows: int, scale: float, tensor_core: bool = None) -> None:
    """o (rows,16,512) bf16 and lse (rows,16) f32 over the kept pages.
    ``tensor_core``: True = the tcgen05 kernel (tokens in the M dimension, TMA
    page gather; needs token rows evenly spaced across blocks), False = the
    warp-level kernel.  Default (None, or ``st.tensor_core`` when set): the
    tcgen05 kernel when a CTA of the cluster the library would launch
    (``locks_mla_decode_tc_cluster_size``) walks more than one 8-page tile, the
    warp-level kernel for the one-tile case.  Measured at config 3 (8 rows x
    128 kept pages): tcgen05 with two tiles per CTA in 8-CTA clusters 19.3 us,
    warp-level kernel 24.2 us; every page kept 3.5 against 4.2 ms per 4-layer
    step."""
    _check_cache(cache)
    if tensor_core is None:
        tensor_core = getattr(st, "tensor_core", None)
    can_tc = cache.stride(0) == PAGE * cache.stride(1)
    if tensor_core is None:
        pages = min(st.budget_pages, st.max_pages)
        cl = _cabi.lib().locks_mla_decode_tc_cluster_size(int(n_rows), int(pages))
        share = -(-pages // max(1, cl))
        tensor_core = share > 8
    tensor_core = bool(tensor_core) and can_tc
    if tensor_core:
        _cabi.call("locks_mla_decode_tc", _cabi.ptr(q), q.stride(0),
                   _cabi.ptr(cache), cache.stride(0), cache.stride(1),
                   _cabi.ptr(block_table), block_table.stride(0),
                   _cabi.ptr(st.page_table), _cabi.ptr(st.page_cnt),
                   _cabi.ptr(seq_lens), _cabi.ptr(out), _cabi.ptr(lse), int(n_rows),
                   int(st.max_pages), int(cache.shape[0]),
                   int(min(st.budget_pages, st.max_pages)), float(scale),
                   _cabi.ptr(st.status), _cabi.stream())
        return
    _cabi.call("locks_mla_decode", _cabi.ptr(q), q.stride(0), _cabi.ptr(cache),
               cache.stride(0), cache.stride(1), _cabi.ptr(block_table),
               block_table.stride(0), _cabi.ptr(st.page_table),
               _cabi.ptr(st.page_cnt), _cabi.ptr(seq_lens), _cabi.ptr(out),
               _cabi.ptr(lse), int(n_rows), int(st.max_pages), float(scale),
               _cabi.ptr(st.status), _cabi.stream())


def mla_forward(st: MlaState, layer: int, q, cache, block_table, seq_lens, out,
                lse, scale: float) -> None:
    """Score -> select -> decode of one layer (3 launches; the per-step
    ``mla_derive`` is done once by the caller)."""
    n_rows = int(seq_lens.shape[0])
    mla_page_score(st, layer, q, cache, block_table, n_rows, scale)
    mla_select_pages(st, n_rows)
    mla_decode(st, q, cache, block_table, seq_lens, out, lse, n_rows, scale)
