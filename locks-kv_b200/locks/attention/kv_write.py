"""KV-write neighbour of the hot path (host wrapper of ``locks_kv_write``).

``rope_and_cache`` keeps the argument meaning of the reference's
``tier/k5_cuda.py::rope_and_cache_fixc`` (:689-730): un-rotated K and V rows of
the step's tokens, the paged cache, ``slot_mapping`` and ``positions`` (int64),
the (P, rot_dim) cos|sin table.  Passing the selection state and the layer index
additionally rebuilds, in the same launch, the summary of every page a token
completes -- what the reference does with a separate tail refresh one step
later (``selection/rki4_tailgraph.py``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi
from .decode import _split_kv


def rope_and_cache(key: torch.Tensor, val: torch.Tensor, kv_cache: torch.Tensor,
                   slot_mapping: torch.Tensor, positions: Optional[torch.Tensor],
                   cos_sin: Optional[torch.Tensor], *, neox: bool = True,
                   st=None, lidx: Optional[int] = None) -> None:
    """key, val: bf16 (n_tok, n_kv, d); kv_cache: (NB, 2, page, n_kv, d) or
    (2, NB, page, n_kv, d)."""
    k, v = _split_kv(kv_cache)
    assert key.dtype == torch.bfloat16 and val.dtype == torch.bfloat16
    assert key.stride(2) == 1 and val.stride(2) == 1
    assert slot_mapping.dtype == torch.int64
    assert (k.stride(0), k.stride(1), k.stride(2)) == \
        (v.stride(0), v.stride(1), v.stride(2)), "K and V planes must share strides"
    n_tok, n_kv, d = key.shape
    rot = 0
    if cos_sin is not None:
        assert positions is not None and positions.dtype == torch.int64
        assert cos_sin.dtype == torch.bfloat16 and cos_sin.stride(1) == 1
        rot = int(cos_sin.shape[1])
    rec = tag = None
    if st is not None:
        rec, tag = st.pp_rec[lidx], st.pp_tag[lidx]
        assert int(k.shape[0]) <= st.NB
    _cabi.call("locks_kv_write", _cabi.ptr(key), key.stride(0), key.stride(1),
               _cabi.ptr(val), val.stride(0), val.stride(1), _cabi.ptr(k),
               _cabi.ptr(v), k.stride(0), k.stride(1), k.stride(2),
               _cabi.ptr(slot_mapping), _cabi.ptr(positions), _cabi.ptr(cos_sin),
               int(cos_sin.stride(0)) if cos_sin is not None else 0, rot,
               1 if neox else 0, _cabi.ptr(rec), _cabi.ptr(tag), int(n_tok),
               int(n_kv), int(d), int(k.shape[1]), int(k.shape[0]),
               _cabi.stream())



def kv_append_desc(key: torch.Tensor, val: torch.Tensor, kv_cache: torch.Tensor,
                   slot_mapping: torch.Tensor, positions: Optional[torch.Tensor],
                   cos_sin: Optional[torch.Tensor], *, neox: bool = True):
    """Description of one layer's decode-step KV write (one token per request
    row; same arguments as :func:`rope_and_cache`) for the selector to carry:
    ``rki4_select_only(st, n_req, append=desc)`` stores the token in the launch
    that selects the pages, so the step has no KV-write launch of its own.  The
    description holds raw addresses: the tensors must outlive its use."""
    k, v = _split_kv(kv_cache)
    assert key.dtype == torch.bfloat16 and val.dtype == torch.bfloat16
    assert key.stride(2) == 1 and val.stride(2) == 1
    assert slot_mapping.dtype == torch.int64
    assert (k.stride(0), k.stride(1), k.stride(2)) == \
        (v.stride(0), v.stride(1), v.stride(2)), "K and V planes must share strides"
    rot = 0
    if cos_sin is not None:
        assert positions is not None and positions.dtype == torch.int64
        assert cos_sin.dtype == torch.bfloat16 and cos_sin.stride(1) == 1
        rot = int(cos_sin.shape[1])
    d = _cabi.KvAppendDesc()
    d.key, d.k_row_stride, d.k_head_stride = key.data_ptr(), key.stride(0), key.stride(1)
    d.val, d.v_row_stride, d.v_head_stride = val.data_ptr(), val.stride(0), val.stride(1)
    d.k_cache, d.v_cache = k.data_ptr(), v.data_ptr()
    d.kv_stride_block, d.kv_stride_tok, d.kv_stride_head = \
        k.stride(0), k.stride(1), k.stride(2)
    d.slot_mapping = slot_mapping.data_ptr()
    d.positions = positions.data_ptr() if positions is not None else None
    d.cos_sin = cos_sin.data_ptr() if cos_sin is not None else None
    d.cos_sin_row_stride = int(cos_sin.stride(0)) if cos_sin is not None else 0
    d.rot_dim, d.neox, d.head_dim = rot, 1 if neox else 0, int(key.shape[2])
    d.page, d.num_blocks = int(k.shape[1]), int(k.shape[0])
    for t in (key, val, k, v, slot_mapping):
        if not t.is_cuda:
            raise RuntimeError("LOCKS B200 kernels need CUDA tensors: there is no "
                               "CPU path")
    return d
