"""Host logic of the plugin boundary: refresh gate, settled lengths, backend
path substitution, plugin inertness.  No GPU needed."""
from __future__ import annotations

import pytest
import torch

from locks.backend.builder import RefreshGate, settled_lengths


def T(*v):
    return torch.tensor(v, dtype=torch.int32)


def test_gate_first_step_is_bulk_then_delta_on_composition_change():
    g = RefreshGate(16)
    a, rows, nd, mf = g.decide(T(100, 40), T(99, 39))
    assert (a, nd, mf) == ("bulk", True, 99 // 16)
    # a new request replaces row 1 -> not steady -> tag-scan delta
    a, rows, nd, mf = g.decide(T(101, 300), T(100, 299))
    assert (a, nd, mf) == ("delta", True, 299 // 16)
    # different batch size -> delta again
    a, *_ = g.decide(T(102, 301, 7), T(101, 300, 6))
    assert a == "delta"


def test_gate_steady_steps_skip_and_tail_one_step_after_boundary():
    g = RefreshGate(16)
    g.decide(T(110, 30), T(109, 29))
    seen = []
    for step in range(1, 8):
        cur = T(110 + step, 30 + step)
        a, rows, nd, _ = g.decide(cur, cur - 1)
        seen.append((a, None if rows is None else rows.tolist(), nd))
    # row 0: settled 112 (= 7*16) at cur 113 (step 3); row 1: settled 32 at cur 33
    assert seen[0] == ("skip", None, False)
    assert seen[1] == ("skip", None, False)
    assert seen[2] == ("tail", [0, 1], True)
    assert all(s[0] == "skip" for s in seen[3:])


def test_gate_padded_and_frozen_rows_are_steady():
    g = RefreshGate(16)
    g.decide(T(50, 0, 0), T(49, 0, 0))
    a, rows, nd, _ = g.decide(T(51, 0, 0), T(50, 0, 0))
    assert a == "skip"
    a, *_ = g.decide(T(51, 0, 0), T(50, 0, 0))        # drain replay: frozen
    assert a == "skip"


def test_gate_prefill_to_decode_transition_is_full():
    """A row leaving chunked prefill advances seq_len by one but its settled
    length jumps by the last chunk: must not be treated as steady."""
    g = RefreshGate(16)
    g.decide(T(512), T(0))            # prefill step: 512 query tokens
    a, *_ = g.decide(T(513), T(512))
    assert a == "delta"               # built_once is already set by the first


def test_settled_lengths():
    cur, st = settled_lengths(T(100, 50, 9), T(0, 1, 2, 3), 3)
    assert st.tolist() == [99, 49, 8]
    cur, st = settled_lengths(T(100, 600), T(0, 1, 513), 2)   # mixed step
    assert st.tolist() == [99, 88]


def test_backend_substitution_and_inert_register(monkeypatch, capsys):
    reg = pytest.importorskip("locks.backend.register")
    assert reg._swap_path(reg._FA_PATH).endswith("LocksAttentionBackend")
    assert reg._swap_path("vllm.v1.attention.backends.mla.triton_mla.TritonMLABackend") \
        .endswith("mla_attn.LocksMLABackend")
    assert reg._swap_path("something.else.Backend") == "something.else.Backend"
    assert reg.LocksAttentionBackend.get_impl_cls().__name__ == "LocksAttentionImpl"
    assert reg.LocksAttentionBackend.get_builder_cls().__name__ == "LocksMetadataBuilder"
    assert reg.LocksAttentionBackend.get_name() == "FLASH_ATTN"
    monkeypatch.delenv("LOCKS_CONFIG", raising=False)
    monkeypatch.delenv("LOCKS_DISABLE", raising=False)
    reg.register()
    assert "INERT" in capsys.readouterr().out and not reg._APPLIED
    monkeypatch.setenv("LOCKS_DISABLE", "1")
    reg.register({"budget_pages": 8})
    assert not reg._APPLIED
    monkeypatch.delenv("LOCKS_DISABLE")
    with pytest.raises(ValueError, match="not available"):
        reg.register({"variant": "mem-v"})


def test_mla_backend_class():
    m = pytest.importorskip("locks.backend.mla_attn")
    assert m.LocksMLABackend.get_impl_cls() is m.LocksMLAImpl
    assert hasattr(m.LocksMLAImpl, "forward_mqa")
