"""Stage B -- sparse paged attention over the selected pages."""
from __future__ import annotations

from .decode import (DenseDecodeBuffers, PinnedHostVSource,  # noqa: F401
                     ResidentVSource, VSource,
                     dense_paged_decode, ensure_stage_b_buffers,
                     sparse_paged_decode_batched, sparse_paged_decode_fused)
from .kv_write import kv_append_desc, rope_and_cache  # noqa: F401
from .merge import merge_splits  # noqa: F401

__all__ = ["sparse_paged_decode_batched", "sparse_paged_decode_fused",
           "dense_paged_decode", "DenseDecodeBuffers", "ResidentVSource",
           "PinnedHostVSource",
           "VSource", "ensure_stage_b_buffers", "merge_splits", "rope_and_cache",
           "kv_append_desc"]
