"""Stage B: sparse paged decode over the pages Stage A selected.

Host wrappers with the reference's names and argument meaning
(``attention/decode.py``): ``ResidentVSource`` / ``_split_kv`` (:64-100),
``ensure_stage_b_buffers`` (:130-156), ``_pps_min`` (:162-203),
``_adaptive_split`` (:103-127) and ``sparse_paged_decode_batched`` (:328-387).
K and V are read straight from the engine's paged cache (no gather); every call
is fixed-shape, allocation-free and sync-free.
"""
from __future__ import annotations

import os

import math
from typing import Protocol, Tuple

import torch

from .. import _cabi


class VSource(Protocol):
    """Injected V provider: ``args()`` returns the V plane and its (block,
    token, head) element strides."""
    SRC_ID: int

    def args(self) -> Tuple[torch.Tensor, int, int, int]:
        ...


def _split_kv(kv_cache: torch.Tensor):
    """(K, V) views ``(num_blocks, page, n_kv, d)`` for either engine layout:
    ``(2, NB, page, n_kv, d)`` or ``(NB, 2, page, n_kv, d)``; a K-only cache
    ``(NB, 1, ...)`` yields V = None."""
    if kv_cache.shape[0] == 2:
        return kv_cache[0], kv_cache[1]
    if kv_cache.shape[1] == 1:
        return kv_cache.select(1, 0), None
    return kv_cache.select(1, 0), kv_cache.select(1, 1)


class ResidentVSource:
    """V lives in the engine cache next to K (the ``fast`` variant)."""
    SRC_ID = 0

    def __init__(self, kv_cache: torch.Tensor):
        _, v = _split_kv(kv_cache)
        if v is None:
            raise ValueError("ResidentVSource needs a resident V half; this "
                             "cache is K-only")
        self._v = v

    def args(self):
        v = self._v
        return v, v.stride(0), v.stride(1), v.stride(2)


class PinnedHostVSource:
    """V lives in pinned host memory and is read IN PLACE by the decode kernel
    over the host link (the memory-saving variant: the GPU keeps K and the
    summaries, which selection needs for every page, while V -- needed only for
    the ~b selected pages of a step -- stays in DRAM).  The plane has the K
    plane's strides, so the kernels address both alike; the KV-write kernel can
    store new V rows through the same pointer.  This is the seam of the
    reference's V tier (``attention/decode.py:52-100``, ``tier/pool.py:104-184``)
    without its staging pool: no copy engine, no residency map."""
    SRC_ID = 1

    def __init__(self, kv_cache: torch.Tensor):
        k, v = _split_kv(kv_cache)
        if v is None:
            raise ValueError("PinnedHostVSource copies the V half of a cache "
                             "that has one")
        # smallest buffer that holds a plane with K's strides
        span = 1 + sum((n - 1) * st for n, st in zip(k.shape, k.stride()))
        self._buf = torch.empty(span, dtype=v.dtype, pin_memory=True)
        self._v = torch.as_strided(self._buf, tuple(k.shape), tuple(k.stride()))
        self._v.copy_(v)

    @property
    def plane(self) -> torch.Tensor:
        return self._v

    def args(self):
        v = self._v
        return v, v.stride(0), v.stride(1), v.stride(2)


def _next_pow2(x: int) -> int:
    return 1 << max(0, int(x) - 1).bit_length()


def _pps_min(n_req: int, n_kv: int = 8) -> int:
    """Minimum page-table entries per split program (amortises the q load and
    the partial store)."""
    if n_kv == 1 and 4 < n_req <= 16:
        return 4
    if n_req == 1:
        return 2
    return 8 if n_req < 16 else 16


def _adaptive_split(max_reqs: int, max_pages: int, budget: float,
                    hard_cap: int) -> int:
    """Allocation-time split count: about the number of ACTIVE split programs
    at low batch, the fixed cap otherwise."""
    if int(max_reqs) > 4:
        return hard_cap
    pps_min = _pps_min(int(max_reqs))
    est = math.ceil(1.5 * float(budget) * int(max_pages) / max(1, pps_min))
    return int(min(hard_cap, max(16, _next_pow2(max(1, est)))))


def ensure_stage_b_buffers(st, device, split: int, *, adapt: bool = True) -> None:
    """Attach the split-K partial buffers to the state (once, outside any
    graph): ``m_part, l_part (R, n_kv, split, G)``, ``acc_part (.., G, d)``."""
    if getattr(st, "m_part", None) is not None:
        return
    R, n_kv, G, D = st.max_reqs, st.n_kv, st.G, st.d
    if adapt:
        if st.budget_abs > 0:
            est_frac = (st.budget_abs + st.sink_pages + st.window_pages) \
                / max(1, st.max_pages)
        else:
            est_frac = float(st.budget or 0.1)
        split = _adaptive_split(R, st.max_pages, est_frac, split)
    st.split = int(split)
    f32 = torch.float32
    st.m_part = torch.empty(R, n_kv, split, G, device=device, dtype=f32)
    st.l_part = torch.empty(R, n_kv, split, G, device=device, dtype=f32)
    st.acc_part = torch.empty(R, n_kv, split, G, D, device=device, dtype=f32)


def _kv_args(kv_cache, vsource):
    k, _ = _split_kv(kv_cache)
    v, svb, svt, svh = vsource.args()
    assert k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
    assert (k.stride(0), k.stride(1), k.stride(2)) == (svb, svt, svh), \
        "K and V planes must share strides"
    assert k.stride(3) == 1 and v.stride(3) == 1
    return k, v


def sparse_paged_decode_batched(q, kv_cache, block_table, seq_lens, st, out,
                                vsource, *, scale: float = None) -> None:
    """Split-K decode + merge (2 launches) for the whole batch; writes rows
    [0, n_req) of ``out (T, H, d)`` in place."""
    if scale is None:
        scale = st.scale
    n_req = int(seq_lens.shape[0])
    k, v = _kv_args(kv_cache, vsource)
    pps_min = _pps_min(n_req, st.n_kv)
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(1) == st.d and out.stride(1) == st.d
    _cabi.call("locks_decode_split", _cabi.ptr(q), q.stride(0), _cabi.ptr(k),
               _cabi.ptr(v), k.stride(0), k.stride(1), k.stride(2),
               _cabi.ptr(block_table), block_table.stride(0),
               _cabi.ptr(st.page_table), _cabi.ptr(st.page_cnt),
               _cabi.ptr(seq_lens), _cabi.ptr(st.m_part), _cabi.ptr(st.l_part),
               _cabi.ptr(st.acc_part), n_req, int(st.n_kv), int(st.G),
               int(st.d), int(st.page), int(st.max_pages), int(st.split),
               int(pps_min), float(scale), _cabi.ptr(st.status), _cabi.stream())
    _cabi.call("locks_merge_splits", _cabi.ptr(st.m_part), _cabi.ptr(st.l_part),
               _cabi.ptr(st.acc_part), _cabi.ptr(st.page_cnt), _cabi.ptr(out),
               out.stride(0), n_req, int(st.n_kv), int(st.G), int(st.d),
               int(st.split), int(pps_min), _cabi.stream())


# Page staging of the fused decode: False = 16-byte cp.async copies (any cache
# strides, V may live in pinned host memory), True = tiled tensor-map copies
# (cp.async.bulk.tensor.2d; needs both planes resident as (num_blocks, 16, n_kv,
# 128) matrices).  LOCKS_DECODE_TMA=0/1 overrides for A/B timing.
FUSED_TMA_DEFAULT = False


def _tma_layout_ok(k, v, vsource) -> bool:
    return (isinstance(vsource, ResidentVSource) and v.is_cuda
            and k.stride(1) > 0 and k.stride(0) % k.stride(1) == 0
            and k.stride(0) >= 16 * k.stride(1) and k.stride(2) % 64 == 0
            and k.stride(2) >= 128
            and (k.shape[2] - 1) * k.stride(2) + 128 <= k.stride(1))


def sparse_paged_decode_fused(q, kv_cache, block_table, seq_lens, st, out,
                              vsource, *, scale: float = None,
                              tma: bool = None) -> None:
    """One-launch decode: a CTA per (kv-head, request) walks every selected
    page and writes the final output (the reference's ``locks_decode_fused``,
    ``attention/decode_cuda.py:587-884``; preferred at large batch).  ``tma``
    picks the page staging (see ``FUSED_TMA_DEFAULT``)."""
    if scale is None:
        scale = st.scale
    if hasattr(vsource, "tier"):    # V behind the two-level tier (vtier.py)
        vsource.tier.decode(vsource.layer, q, kv_cache, block_table, seq_lens, st,
                            out, scale)
        return
    n_req = int(seq_lens.shape[0])
    k, v = _kv_args(kv_cache, vsource)
    if tma is None:                 # by default only where the layout allows it
        env = os.environ.get("LOCKS_DECODE_TMA")
        tma = (FUSED_TMA_DEFAULT if env is None else env == "1") and \
            _tma_layout_ok(k, v, vsource)
    if tma:
        _cabi.call("locks_decode_fused_tma", _cabi.ptr(q), q.stride(0),
                   _cabi.ptr(k), _cabi.ptr(v), k.stride(0), k.stride(1),
                   k.stride(2), _cabi.ptr(block_table), block_table.stride(0),
                   _cabi.ptr(st.page_table), _cabi.ptr(st.page_cnt),
                   _cabi.ptr(seq_lens), _cabi.ptr(out), out.stride(0), n_req,
                   int(st.n_kv), int(st.G), int(st.d), int(st.page),
                   int(st.max_pages), int(k.shape[0]), float(scale),
                   _cabi.ptr(st.status), _cabi.stream())
        return
    if getattr(st, "row_order_n", 0) == n_req:      # large batch: longest row first
        _cabi.call("locks_decode_fused_rows", _cabi.ptr(q), q.stride(0),
                   _cabi.ptr(k), _cabi.ptr(v), k.stride(0), k.stride(1),
                   k.stride(2), _cabi.ptr(block_table), block_table.stride(0),
                   _cabi.ptr(st.page_table), _cabi.ptr(st.page_cnt),
                   _cabi.ptr(seq_lens), _cabi.ptr(out), out.stride(0), n_req,
                   int(st.n_kv), int(st.G), int(st.d), int(st.page),
                   int(st.max_pages), _cabi.ptr(st.order_dec), float(scale),
                   _cabi.ptr(st.status), _cabi.stream())
        return
    _cabi.call("locks_decode_fused", _cabi.ptr(q), q.stride(0), _cabi.ptr(k),
               _cabi.ptr(v), k.stride(0), k.stride(1), k.stride(2),
               _cabi.ptr(block_table), block_table.stride(0),
               _cabi.ptr(st.page_table), _cabi.ptr(st.page_cnt),
               _cabi.ptr(seq_lens), _cabi.ptr(out), out.stride(0), n_req,
               int(st.n_kv), int(st.G), int(st.d), int(st.page),
               int(st.max_pages), float(scale), _cabi.ptr(st.status),
               _cabi.stream())


class DenseDecodeBuffers:
    """Partial buffers of the dense full-KV baseline decode."""

    def __init__(self, device, max_reqs, n_kv, G, d, split):
        f32 = torch.float32
        self.split = int(split)
        self.m = torch.empty(max_reqs, n_kv, split, G, device=device, dtype=f32)
        self.l = torch.empty(max_reqs, n_kv, split, G, device=device, dtype=f32)
        self.acc = torch.empty(max_reqs, n_kv, split, G, d, device=device,
                               dtype=f32)


def dense_paged_decode(q, kv_cache, block_table, seq_lens, buf, out, *, n_kv,
                       G, scale, status=None) -> None:
    """Full-KV paged decode with the same kernels (baseline for the
    sparse/dense crossover)."""
    k, v = _split_kv(kv_cache)
    n_req = int(seq_lens.shape[0])
    d, page = int(k.shape[3]), int(k.shape[1])
    _cabi.call("locks_dense_decode", _cabi.ptr(q), q.stride(0), _cabi.ptr(k),
               _cabi.ptr(v), k.stride(0), k.stride(1), k.stride(2),
               _cabi.ptr(block_table), block_table.stride(0),
               _cabi.ptr(seq_lens), _cabi.ptr(buf.m), _cabi.ptr(buf.l),
               _cabi.ptr(buf.acc), _cabi.ptr(out), out.stride(0), n_req,
               int(n_kv), int(G), d, page, int(buf.split), float(scale),
               _cabi.ptr(status), _cabi.stream())


NOALLOC_MAX_ROWS = 16384


def sparse_paged_decode_noalloc(q, kv_cache, block_table, seq_lens, st, out,
                                vsource, *, split: int, scale: float = None) -> None:
    """Split decode + merge whose partial buffers live inside the library.

    For integrations that are not allowed to allocate device memory (they can
    only hand over the tensors they were given): nothing is taken from
    ``st.m_part / l_part / acc_part``; the partials go to a fixed ~8.5 MB array
    that is part of the loaded library on every GPU.  Limits: ``n_req * n_kv *
    split * G <= 16384`` (a ``RuntimeError`` otherwise); make the first call on
    a device outside stream capture (it looks up the array's address once);
    calls share the array, so do not let two of them overlap on the GPU.
    Results equal ``sparse_paged_decode_batched`` with the same ``split``.
    """
    if scale is None:
        scale = st.scale
    n_req = int(seq_lens.shape[0])
    k, v = _kv_args(kv_cache, vsource)
    _cabi.call("locks_decode_split_noalloc", _cabi.ptr(q), q.stride(0),
               _cabi.ptr(k), _cabi.ptr(v), k.stride(0), k.stride(1), k.stride(2),
               _cabi.ptr(block_table), block_table.stride(0),
               _cabi.ptr(st.page_table), _cabi.ptr(st.page_cnt),
               _cabi.ptr(seq_lens), _cabi.ptr(out), out.stride(0), n_req,
               int(st.n_kv), int(st.G), int(st.d), int(st.page),
               int(st.max_pages), int(split), int(_pps_min(n_req, st.n_kv)),
               float(scale), _cabi.ptr(st.status), _cabi.stream())
