"""LOCKS decode hot path for NVIDIA B200 (sm_100a).

Drop-in for the ``locks`` package of Js-Hwang1/locks-kv on its decode path:
same ``LocksConfig`` / ``LOCKS_CONFIG`` surface, same ``register()`` vLLM
general-plugin hook, same selection / attention module layout -- with every
hot-path stage running as a hand-written CUDA kernel reached through a C-ABI
shared library (``liblocks_b200.so``).

  from locks import LocksConfig, register
"""
from __future__ import annotations

from .config import LocksConfig  # noqa: F401

__all__ = ["LocksConfig", "register"]

__version__ = "0.1.0"


def register() -> None:
    """vLLM general-plugin entry point (reference: ``__init__.py:26-31``)."""
    from .backend.register import register as _register
    _register()
