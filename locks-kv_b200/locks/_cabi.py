"""ctypes binding of ``liblocks_b200.so`` (the C ABI of include/locks_b200.h).

This is the only way the Python host code reaches a kernel.  There is no
fallback: if the library has not been built, or a call reports an error, a
``RuntimeError`` is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, c_char_p, c_double, c_float, c_int, c_int64,
                    c_void_p)

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "_lib", "liblocks_b200.so")

_P, _I, _L, _F, _D = c_void_p, c_int, c_int64, c_float, c_double

# name -> (argtypes, kernel launches per call)
_SIGNATURES = {
    "locks_version": ([], 0),
    "locks_set_pdl": ([_I], 0),
    "locks_record_bytes": ([_I, _I], 0),
    "locks_rki4_build": ([_P, _L, _L, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                          _I, _I, _P], 1),
    "locks_rki4_tag_scan": ([_P, _L, _L, _L, _P, _P, _P, _P, _I, _I, _I, _I,
                             _I, _P], 1),
    "locks_derive_page_params": ([_P, _I, _I, _I, _I, _I, _D, _P, _P, _P, _P], 1),
    "locks_derive_page_params_req": ([_P, _I, _I, _I, _I, _P, _D, _P, _P, _P,
                                      _P], 1),
    "locks_append_advance_req": ([_P, _P, _L, _I, _I, _I, _I, _I, _P, _D, _P, _P,
                                  _P, _P, _P, _P, _P], 1),
    "locks_rki4_score_bt": ([_P, _L, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I,
                             _I, _I, _I, _I, _F, _I, _P, _P], 1),
    "locks_topb_select": ([_I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I,
                           _I, _P], 1),
    "locks_append_advance": ([_P, _P, _L, _I, _I, _I, _I, _I, _I, _D, _P, _P, _P,
                              _P, _P, _P, _P], 1),
    "locks_topb_select_append": ([_I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I,
                                  _I, _I, _P, _P], 1),
    "locks_decode_split": ([_P, _L, _P, _P, _L, _L, _L, _P, _L, _P, _P, _P, _P,
                            _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P,
                            _P], 1),
    "locks_merge_splits": ([_P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I,
                            _P], 1),
    "locks_rki4_build_slots": ([_P, _L, _L, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                                _I, _I, _P], 1),
    "locks_kv_write": ([_P, _L, _L, _P, _L, _L, _P, _P, _L, _L, _L, _P, _P, _P,
                        _L, _I, _I, _P, _P, _I, _I, _I, _I, _I, _P], 1),
    "locks_cp_pack": ([_P, _P, _P, _I, _I, _I, _I, _I, _I, _P], 1),
    "locks_cp_select": ([_P, _L, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P], 1),
    "locks_cp_region_bytes": ([_I, _P], 0),
    "locks_cp_alloc": ([_L, _P], 0),
    "locks_cp_free": ([_P], 0),
    "locks_cp_ipc_export": ([_P, _P], 0),
    "locks_cp_ipc_open": ([_P, _P], 0),
    "locks_cp_ipc_close": ([_P], 0),
    "locks_cp_exchange": ([_P, _I, _I, _P, _I, _I, _P, _I, _P, _P], 1),
    "locks_cp_link_bytes": ([_I, _I, _I, _P], 0),
    "locks_cp_begin_step": ([_P, _P], 1),
    "locks_cp_link_reset": ([_P, _L, ctypes.c_uint32, _P], 1),
    "locks_topb_select_cp": ([_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P,
                              _P, _P], 1),
    "locks_decode_fused_cp": ([_P, _L, _P, _P, _L, _L, _L, _P, _L, _P, _P, _P, _P,
                               _L, _I, _I, _I, _I, _I, _F, _P, _P, _P], 1),
    "locks_merge_gathered": ([_P, _L, _I, _P, _L, _I, _I, _I, _I, _I, _P], 1),
    "locks_decode_fused": ([_P, _L, _P, _P, _L, _L, _L, _P, _L, _P, _P, _P, _P,
                            _L, _I, _I, _I, _I, _I, _I, _F, _P, _P], 1),
    "locks_vtier_copy_run": ([_P, _L, _P, _L, _L, _I, _P], 0),
    "locks_decode_fused_vtier": ([_P, _L, _P, _P, _L, _L, _L, _P, _L, _P, _P, _P,
                                  _P, _P, _I, _P, _P, _L, _P, _P, _P, _P, _L, _I,
                                  _I, _I, _I, _I, _I, _F, _P, _P], 1),
    "locks_decode_fused_rows": ([_P, _L, _P, _P, _L, _L, _L, _P, _L, _P, _P, _P, _P,
                                 _L, _I, _I, _I, _I, _I, _I, _P, _F, _P, _P], 1),
    "locks_rki4_score_bt_rows": ([_P, _L, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I,
                                  _I, _I, _I, _I, _F, _I, _P, _P, _P], 1),
    "locks_topb_select_rows": ([_I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I,
                                _I, _P, _P], 1),
    "locks_mla_decode_tc_cluster_size": ([_I, _I], 0),
    "locks_row_order": ([_P, _P, _P, _I, _I, _P, _P, _P], 1),
    "locks_decode_fused_tma": ([_P, _L, _P, _P, _L, _L, _L, _P, _L, _P, _P, _P, _P,
                                _L, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P], 1),
    "locks_dense_decode": ([_P, _L, _P, _P, _L, _L, _L, _P, _L, _P, _P, _P, _P,
                            _P, _L, _I, _I, _I, _I, _I, _I, _F, _P, _P], 2),
    "locks_decode_split_noalloc": ([_P, _L, _P, _P, _L, _L, _L, _P, _L, _P, _P,
                                    _P, _P, _L, _I, _I, _I, _I, _I, _I, _I, _I,
                                    _F, _P, _P], 2),
    "locks_mla_build_factors": ([_P, _L, _L, _P, _P, _I, _I, _P], 1),
    "locks_mla_refresh_rows": ([_P, _L, _L, _P, _P, _L, _P, _P, _P, _P, _P, _I, _I,
                                _I, _P], 2),
    "locks_mla_derive": ([_P, _I, _I, _I, _I, _P, _P, _P, _P], 1),
    "locks_mla_score": ([_P, _L, _P, _P, _L, _L, _P, _L, _P, _P, _P, _I, _I,
                         _I, _F, _I, _P, _P], 1),
    "locks_mla_decode_tc": ([_P, _L, _P, _L, _L, _P, _L, _P, _P, _P, _P, _P, _I,
                             _I, _I, _I, _F, _P, _P], 1),
    "locks_mla_decode": ([_P, _L, _P, _L, _L, _P, _L, _P, _P, _P, _P, _P, _I,
                          _I, _F, _P, _P], 1),
}

_lib = None
launches = 0          # kernels launched through this binding (bench evidence)


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it is missing (no CPU fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with "
                "`python -m locks._build` (needs nvcc); the LOCKS B200 ops "
                "have no other implementation")
        L = ctypes.CDLL(LIB_PATH)
        L.locks_last_error.restype = c_char_p
        L.locks_last_error.argtypes = []
        for name, (args, _) in _SIGNATURES.items():
            if not hasattr(L, name):
                continue                       # optional entry points
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = c_int
        _lib = L
    return _lib


def register_signature(name, argtypes, n_launch=1):
    """Declare an additional entry point (used by optional modules)."""
    _SIGNATURES[name] = (argtypes, n_launch)
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int


def call(name: str, *args) -> None:
    """Invoke an entry point; non-zero return codes become RuntimeError."""
    global launches
    L = lib()
    rc = getattr(L, name)(*args)
    if rc != 0:
        raise RuntimeError(
            f"{name} failed ({rc}): {L.locks_last_error().decode()}")
    launches += _SIGNATURES[name][1]


def ptr(t) -> c_void_p:
    """Device pointer of a CUDA tensor, or of a pinned host tensor (unified
    addressing: the GPU reads it over the host link); None -> NULL."""
    if t is None:
        return c_void_p(0)
    if not t.is_cuda and not t.is_pinned():
        raise RuntimeError("LOCKS B200 kernels need CUDA tensors (or pinned host "
                           f"memory the GPU reads in place), got {t.device}: "
                           "there is no CPU path")
    return c_void_p(t.data_ptr())


class KvAppendDesc(ctypes.Structure):
    """``locks_kv_append_t`` of the header, field for field."""
    _fields_ = [("key", _P), ("k_row_stride", _L), ("k_head_stride", _L),
                ("val", _P), ("v_row_stride", _L), ("v_head_stride", _L),
                ("k_cache", _P), ("v_cache", _P), ("kv_stride_block", _L),
                ("kv_stride_tok", _L), ("kv_stride_head", _L),
                ("slot_mapping", _P), ("positions", _P), ("cos_sin", _P),
                ("cos_sin_row_stride", _L), ("rot_dim", ctypes.c_int32),
                ("neox", ctypes.c_int32), ("head_dim", ctypes.c_int32),
                ("page", ctypes.c_int32), ("num_blocks", ctypes.c_int32)]


class CpLinkDesc(ctypes.Structure):
    """``locks_cp_link_t`` of the header, field for field."""
    _fields_ = [("regions", _P * 8), ("world", ctypes.c_int32),
                ("rank", ctypes.c_int32), ("layer", ctypes.c_int32),
                ("n_layers", ctypes.c_int32), ("p0", ctypes.c_int32),
                ("cap", ctypes.c_int32), ("b_global", ctypes.c_int32),
                ("sink_loc", ctypes.c_int32), ("nsh_loc", ctypes.c_int32)]


def stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)
