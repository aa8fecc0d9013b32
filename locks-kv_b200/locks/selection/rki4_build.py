"""Host side of the rki4 summary build: WHICH physical blocks to (re)build.

The arithmetic -- centroid, centred Gram, 16x16 eigen-decomposition, rank-8
factors, int4/int8 quantisation, pack -- is one CUDA kernel launch
(``locks_rki4_build``) over the cross product (layers x blocks x kv-heads); it
replaces the ~55-op torch chain and the cusolver call of the reference
(``selection/rki4_build.py:147-261``).  This module keeps the reference's entry
points and their block-selection rules:

  rki4_build_bulk     every finalized page of every request   (ref :293-303)
  rki4_build_tail     the last finalized page of chosen rows  (ref :264-290)
  rki4_build_delta    pages whose content tag went stale      (ref :306-316)
  rki4_build_refresh  single-layer, tag-gated or forced       (ref :320-364)

Only COMPLETE pages are summarised; lengths are settled lengths.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _cabi
from .rki4_state import Rki4State


def _k_ptr_array(st: Rki4State, K_layers) -> torch.Tensor:
    """Device array of the layers' K-plane base pointers (cached per set)."""
    key = tuple(int(k.data_ptr()) for k in K_layers)
    if st._k_ptrs_key != key:
        st._k_ptrs = torch.tensor(key, dtype=torch.int64, device=K_layers[0].device)
        st._k_ptrs_key = key
    return st._k_ptrs


def _check_k(st: Rki4State, K) -> None:
    assert K.dtype == torch.bfloat16, "K cache must be bf16"
    assert K.dim() == 4 and K.shape[1] == st.page and K.shape[2] == st.n_kv \
        and K.shape[3] == st.d, f"K plane must be (NB, page, n_kv, d), got {tuple(K.shape)}"
    assert K.stride(3) == 1


def _launch_build(st: Rki4State, K_layers, blocks: torch.Tensor, layer0: int,
                  n_layers: int) -> None:
    if blocks.numel() == 0 or n_layers == 0:
        return
    K0 = K_layers[0]
    for K in K_layers:
        _check_k(st, K)
        assert K.stride() == K0.stride() and K.shape == K0.shape
    blocks = blocks.to(torch.int32).contiguous()
    ptrs = _k_ptr_array(st, K_layers)
    _cabi.call("locks_rki4_build", _cabi.ptr(ptrs), K0.stride(0), K0.stride(1),
               K0.stride(2), _cabi.ptr(st.pp_rec), _cabi.ptr(st.pp_tag),
               _cabi.ptr(blocks), int(blocks.numel()), int(layer0),
               int(n_layers), int(st.NB), int(K0.shape[0]), int(st.n_kv),
               int(st.d), int(st.page), _cabi.stream())


def _bulk_blocks(block_table, seq_lens, n_req: int, page: int, max_fin: int):
    """All finalized (request, page) blocks, invalid slots -> block 0 (whose
    rebuild is harmless: a summary is a pure function of the page bytes).
    Fixed shapes, no sync (reference ``selection/build.py:414-426``)."""
    sl = seq_lens[:n_req].to(torch.int64)
    n_fin = sl // page
    pidx = torch.arange(max_fin, device=block_table.device)
    valid = pidx[None, :] < n_fin[:, None]
    return block_table[:n_req, :max_fin].to(torch.int64) \
        .masked_fill(~valid, 0).reshape(-1), valid.reshape(-1)


def _tail_blocks(block_table, seq_lens, n_req: int, page: int, rows):
    """Block of each (selected) request's last finalized page, clamped to page
    0 (reference ``selection/build.py:372-385``)."""
    if rows is None:
        sl = seq_lens[:n_req].to(torch.int64)
        bt = block_table[:n_req]
    else:
        sl = seq_lens[rows].to(torch.int64)
        bt = block_table[rows]
    fin1 = (sl // page - 1).clamp_(min=0)
    return bt.to(torch.int64).gather(1, fin1[:, None]).squeeze(1)


def rki4_build_tail(st: Rki4State, K_layers, block_table, seq_lens, n_req: int,
                    rows=None) -> int:
    """Rebuild the last finalized page of ``rows`` (or of every request) in all
    layers: ONE launch, no device sync, idempotent."""
    if n_req == 0:
        return 0
    blocks = _tail_blocks(block_table, seq_lens, n_req, st.page, rows)
    _launch_build(st, K_layers, blocks, 0, len(K_layers))
    return len(K_layers) * int(blocks.shape[0])


def rki4_build_slots(st: Rki4State, K_layers, slot_mapping: torch.Tensor) -> None:
    """Rebuild, in all layers, the pages that this step's cache writes completed:
    a token whose ``slot_mapping`` entry is the last slot of its block names the
    block; the decision is taken on the device, so the launch has a fixed shape,
    needs no host-side refresh gate and can be captured in the decode graph
    (the device-side form of the tail refresh, reference
    ``selection/rki4_tailgraph.py`` / ``selection/rki4_build.py:318-364``)."""
    assert slot_mapping.dtype == torch.int64 and slot_mapping.is_contiguous()
    n_tok = int(slot_mapping.numel())
    if n_tok == 0 or len(K_layers) == 0:
        return
    K0 = K_layers[0]
    for K in K_layers:
        _check_k(st, K)
        assert K.stride() == K0.stride() and K.shape == K0.shape
    ptrs = _k_ptr_array(st, K_layers)
    _cabi.call("locks_rki4_build_slots", _cabi.ptr(ptrs), K0.stride(0),
               K0.stride(1), K0.stride(2), _cabi.ptr(st.pp_rec),
               _cabi.ptr(st.pp_tag), _cabi.ptr(slot_mapping), n_tok, 0,
               len(K_layers), int(st.NB), int(K0.shape[0]), int(st.n_kv),
               int(st.d), int(st.page), _cabi.stream())


def rki4_build_bulk(st: Rki4State, K_layers, block_table, seq_lens, n_req: int,
                    max_fin: int, chunk_pairs: int = 8192) -> int:
    """Rebuild ALL finalized pages of ALL layers, no device sync.
    ``chunk_pairs`` is accepted for signature compatibility; the kernel needs
    no transient memory, so nothing is chunked."""
    if n_req == 0 or max_fin <= 0:
        return 0
    blocks, _ = _bulk_blocks(block_table, seq_lens, n_req, st.page, max_fin)
    _launch_build(st, K_layers, blocks, 0, len(K_layers))
    return len(K_layers) * int(blocks.shape[0])


def _delta_select(st: Rki4State, K_layers, block_table, seq_lens, n_req: int,
                  max_fin: int) -> torch.Tensor:
    """Blocks whose stored tag differs from the live keys in ANY layer (one
    scan launch + one boolean gather = the path's single device sync).
    Reference ``selection/build.py:475-488``."""
    blocks, valid = _bulk_blocks(block_table, seq_lens, n_req, st.page, max_fin)
    n = int(blocks.numel())
    b32 = blocks.to(torch.int32).contiguous()
    v8 = valid.to(torch.uint8).contiguous()
    stale = torch.zeros(n, dtype=torch.uint8, device=blocks.device)
    K0 = K_layers[0]
    ptrs = _k_ptr_array(st, K_layers)
    _cabi.call("locks_rki4_tag_scan", _cabi.ptr(ptrs), K0.stride(0),
               K0.stride(1), K0.stride(2), _cabi.ptr(st.pp_tag), _cabi.ptr(b32),
               _cabi.ptr(v8), _cabi.ptr(stale), n, len(K_layers), int(st.NB),
               int(st.n_kv), int(st.page), _cabi.stream())
    return blocks[stale.bool()]


def rki4_build_delta(st: Rki4State, K_layers, block_table, seq_lens,
                     n_req: int, max_fin: int, chunk_pairs: int = 8192) -> int:
    """Composition-change rebuild: only blocks whose content tag went stale,
    in all layers."""
    if n_req == 0 or max_fin <= 0:
        return 0
    blocks = _delta_select(st, K_layers, block_table, seq_lens, n_req, max_fin)
    _launch_build(st, K_layers, blocks, 0, len(K_layers))
    return len(K_layers) * int(blocks.shape[0])


def rki4_build_refresh(st: Rki4State, layer: int, K, block_table, seq_lens,
                       n_req: int, *, force: bool = False) -> int:
    """(Re)build every STALE finalized page of the batch for ONE layer
    (``force`` ignores the tags).  Returns the number of blocks rebuilt."""
    if n_req == 0:
        return 0
    page = st.page
    sl = seq_lens[:n_req].to(torch.int64)
    n_fin = sl // page
    max_fin = int(n_fin.max().item())
    if max_fin == 0:
        return 0
    pidx = torch.arange(max_fin, device=K.device)
    fin_mask = pidx[None, :] < n_fin[:, None]
    blocks = block_table[:n_req, :max_fin].to(torch.int64)[fin_mask]
    nb = min(int(st.NB), int(K.shape[0]))
    blocks = blocks[(blocks >= 0) & (blocks < nb)]
    if blocks.numel() == 0:
        return 0
    if not force:
        tag_cur = K[blocks, page - 1, :, :st.tagw].float()
        tag_old = st.pp_tag[layer, blocks].float()
        blocks = blocks[(tag_cur != tag_old).any(dim=(1, 2))]
    blocks = torch.unique(blocks)
    if blocks.numel() == 0:
        return 0
    # a one-layer pointer array whose entry 0 is this layer's K plane
    _check_k(st, K)
    ptrs = torch.zeros(st.L, dtype=torch.int64, device=K.device)
    ptrs[layer] = int(K.data_ptr())
    b32 = blocks.to(torch.int32).contiguous()
    _cabi.call("locks_rki4_build", _cabi.ptr(ptrs), K.stride(0), K.stride(1),
               K.stride(2), _cabi.ptr(st.pp_rec), _cabi.ptr(st.pp_tag),
               _cabi.ptr(b32), int(b32.numel()), int(layer), 1, int(st.NB),
               int(K.shape[0]), int(st.n_kv), int(st.d), int(st.page),
               _cabi.stream())
    return int(blocks.numel())
