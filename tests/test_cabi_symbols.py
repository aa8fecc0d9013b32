"""The shared library builds (nvcc cross-compile), loads without a GPU and
exports every symbol that include/locks_b200.h declares."""
from __future__ import annotations

import ctypes
import os
import re

import pytest

from conftest import ROOT


@pytest.fixture(scope="session")
def libpath():
    from locks._build import build_library
    return build_library()


def _declared():
    hdr = open(os.path.join(ROOT, "include", "locks_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b(locks_[a-z0-9_]+)\s*\(", hdr)))


def test_header_symbols_exported(libpath):
    lib = ctypes.CDLL(libpath)
    names = _declared()
    assert "locks_rki4_score_bt" in names and "locks_decode_split" in names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_covers_header(libpath):
    from locks import _cabi
    import locks.attention  # noqa: F401  (registers optional signatures)
    import locks.selection  # noqa: F401
    declared = set(_declared()) - {"locks_last_error"}
    assert declared <= set(_cabi._SIGNATURES), declared - set(_cabi._SIGNATURES)
    assert _cabi.lib().locks_version() == 1


def test_argument_errors_without_gpu(libpath):
    """Validation happens before any CUDA call, so it is testable on CPU."""
    from locks import _cabi
    lib = _cabi.lib()
    assert lib.locks_record_bytes(128, 16) == 832
    assert lib.locks_record_bytes(64, 16) == -2
    assert b"head_dim 128" in lib.locks_last_error()
    null = ctypes.c_void_p(0)
    rc = lib.locks_derive_page_params(null, 1, 16, 1, 1, 0, 0.1, null, null,
                                      null, null)
    assert rc == -1 and b"null pointer" in lib.locks_last_error()
    with pytest.raises(RuntimeError, match="null pointer"):
        _cabi.call("locks_topb_select", 0, null, null, null, null, null, null,
                   null, null, 1, 1, 1, 1, 1, null)


def test_cpu_tensors_are_rejected():
    import torch
    from locks import _cabi
    with pytest.raises(RuntimeError, match="no CPU path"):
        _cabi.ptr(torch.zeros(4))
