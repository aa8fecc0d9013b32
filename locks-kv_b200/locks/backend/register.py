"""``register()`` -- the vLLM general-plugin entry point.

Builds the one :class:`LocksConfig` (``LOCKS_CONFIG`` + overrides) and patches
``CudaPlatform.get_attn_backend_cls`` so that the FlashAttention backend is
replaced by :class:`LocksAttentionBackend` and any MLA backend by
``LocksMLABackend``.  Inert without a config or with ``LOCKS_DISABLE`` set, as
the reference (``backend/register.py:123-184``).
"""
from __future__ import annotations

import os

from vllm.v1.attention.backends.flash_attn import FlashAttentionBackend

from ..config import LocksConfig
from . import _runtime
from .attn import LocksAttentionImpl
from .builder import LocksMetadataBuilder

_APPLIED = False
_FA_PATH = "vllm.v1.attention.backends.flash_attn.FlashAttentionBackend"
_OUR_PATH = f"{__name__}.LocksAttentionBackend"
_MLA_PATH = __name__.rsplit(".", 1)[0] + ".mla_attn.LocksMLABackend"


class LocksAttentionBackend(FlashAttentionBackend):
    """FlashAttention backend with the LOCKS impl and builder swapped in.
    ``get_name()`` is inherited ("FLASH_ATTN") so vLLM's backend enum still
    resolves; the KV-cache shape is the stock one (K and V resident)."""

    @staticmethod
    def get_impl_cls():
        return LocksAttentionImpl

    @staticmethod
    def get_builder_cls():
        return LocksMetadataBuilder


def _swap_path(path):
    """The backend path LOCKS substitutes for ``path`` (or ``path`` itself)."""
    if path == _FA_PATH:
        return _OUR_PATH
    if isinstance(path, str) and ".mla." in path and path != _MLA_PATH:
        return _MLA_PATH
    return path


def _bracket_profiling_runs() -> None:
    """Mark the engine's memory-profiling dummy runs (they use a throw-away
    minimal KV cache) so that the builder does not latch its state on them:
    ``GPUModelRunner.profile_cudagraph_memory`` and ``_dummy_run(is_profile=
    True)`` are wrapped to raise the runtime's profiling flag for their
    duration (reference ``backend/register.py:340-393``).  Absent methods are
    skipped: the builder also re-checks the latched cache pointers itself."""
    try:
        from vllm.v1.worker.gpu_model_runner import GPUModelRunner as MR
    except Exception as exc:                       # pragma: no cover
        print(f"[locks] profiling-window bracket skipped ({exc})", flush=True)
        return

    def wrap(name, only_if=None):
        orig = getattr(MR, name, None)
        if orig is None or getattr(orig, "_locks_wrapped", False):
            return

        def wrapped(self, *args, **kwargs):
            if only_if is not None and not only_if(args, kwargs):
                return orig(self, *args, **kwargs)
            _runtime.set_profiling(True)
            try:
                return orig(self, *args, **kwargs)
            finally:
                _runtime.set_profiling(False)
        wrapped._locks_wrapped = True
        setattr(MR, name, wrapped)

    wrap("profile_cudagraph_memory")
    wrap("_dummy_run", only_if=lambda a, kw: bool(kw.get("is_profile")))


def register(overrides: dict | None = None) -> None:
    """Runs in every engine / worker process; no device work."""
    global _APPLIED
    if _APPLIED or os.environ.get("LOCKS_DISABLE"):
        return
    if overrides is None and not os.environ.get("LOCKS_CONFIG"):
        print("[locks] register: no LOCKS_CONFIG and no overrides -> plugin "
              "INERT (stock vLLM). Set LOCKS_CONFIG to activate.", flush=True)
        return
    cfg = LocksConfig.load(overrides)
    if cfg.is_mem:
        raise ValueError(
            f"locks (B200 build): variant {cfg.variant!r} is not available; only "
            "'fast' (K and V resident in HBM) has sm_100a kernels")
    _runtime.set_config(cfg)

    from vllm.platforms import cuda
    target = next(k for k in cuda.CudaPlatform.__mro__
                  if "get_attn_backend_cls" in k.__dict__)
    orig = target.__dict__["get_attn_backend_cls"].__func__

    def get_attn_backend_cls(cls, *args, **kwargs):
        path = orig(cls, *args, **kwargs)
        new = _swap_path(path)
        if new != path:
            print(f"[locks] ACTIVE variant={cfg.variant} budget={cfg.budget} "
                  f"budget_pages={cfg.budget_pages} sink={cfg.sink_pages} "
                  f"window={cfg.window_pages}: {path} -> {new}", flush=True)
        return new

    target.get_attn_backend_cls = classmethod(get_attn_backend_cls)
    _bracket_profiling_runs()
    _APPLIED = True
    print("[locks] registered (patched CudaPlatform.get_attn_backend_cls)",
          flush=True)
