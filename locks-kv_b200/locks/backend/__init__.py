"""vLLM integration -- the plugin boundary.

``register()`` patches ``CudaPlatform.get_attn_backend_cls`` so that the
FlashAttention backend is replaced by ``LocksAttentionBackend`` and any MLA
backend by ``LocksMLABackend``.  The vLLM-dependent modules are imported
lazily so that the kernels are usable without vLLM installed.
"""
from __future__ import annotations

__all__ = ["register", "LocksAttentionBackend", "LocksAttentionImpl",
           "LocksMetadataBuilder"]


def __getattr__(name):
    if name in ("register", "LocksAttentionBackend"):
        from . import register as _r
        return getattr(_r, name)
    if name == "LocksAttentionImpl":
        from .attn import LocksAttentionImpl
        return LocksAttentionImpl
    if name == "LocksMetadataBuilder":
        from .builder import LocksMetadataBuilder
        return LocksMetadataBuilder
    raise AttributeError(name)
