"""LocksConfig: defaults, validation and LOCKS_CONFIG loading follow the
reference's config.py."""
from __future__ import annotations

import json

import pytest

from locks import LocksConfig


def test_defaults():
    c = LocksConfig()
    assert c.variant == "fast" and c.coverage == 0.95 and c.budget is None
    assert c.budget_pages is None and c.table == "kv-union"
    assert c.sink_pages == 1 and c.window_pages == 1
    assert c.quad_combine == "nrm" and c.rki4_zsplit is None
    assert c.r8_rank == 8 and c.use_cuda and not c.force_eager
    assert not c.is_mem and not c.offload_k
    with pytest.raises(Exception):
        c.variant = "mem-v"            # frozen


@pytest.mark.parametrize("kw", [
    dict(variant="bogus"), dict(coverage=0.0), dict(coverage=1.5),
    dict(budget=0.0), dict(budget=1.1), dict(rki4_zsplit=0),
    dict(rki4_zsplit=70000), dict(quad_combine="sum"), dict(hot_ratio=0.0),
    dict(mem_summary_cache=True),
    dict(variant="mem-kv", mem_summary_cache=True, mem_k_only=False)])
def test_validation(kw):
    with pytest.raises(ValueError):
        LocksConfig(**kw)


def test_mem_kv_forces_screen():
    c = LocksConfig(variant="mem-kv")
    assert c.r8_screen and c.is_mem and c.offload_k


def test_load_env_inline_file_and_overrides(monkeypatch, tmp_path):
    monkeypatch.delenv("LOCKS_CONFIG", raising=False)
    assert LocksConfig.load() == LocksConfig()
    monkeypatch.setenv("LOCKS_CONFIG", '{"budget_pages": 128, "window_pages": 8}')
    c = LocksConfig.load()
    assert c.budget_pages == 128 and c.window_pages == 8
    c = LocksConfig.load({"window_pages": 4, "sink_pages": None})
    assert c.window_pages == 4 and c.sink_pages == 1
    p = tmp_path / "cfg.json"
    p.write_text(json.dumps({"budget": 0.2}))
    monkeypatch.setenv("LOCKS_CONFIG", str(p))
    assert LocksConfig.load().budget == 0.2
    y = tmp_path / "cfg.yaml"
    y.write_text("budget_pages: 64\nquad_combine: max\n")
    monkeypatch.setenv("LOCKS_CONFIG", str(y))
    c = LocksConfig.load()
    assert c.budget_pages == 64 and c.quad_combine == "max"
    monkeypatch.setenv("LOCKS_CONFIG", '{"nonsense": 1}')
    with pytest.raises(ValueError, match="unknown LocksConfig keys"):
        LocksConfig.load()


def test_single_knob_env_escapes(monkeypatch):
    monkeypatch.delenv("LOCKS_CONFIG", raising=False)
    monkeypatch.setenv("LOCKS_RKI4_Z", "24")
    assert LocksConfig.load().rki4_zsplit == 24
    assert LocksConfig.load({"rki4_zsplit": 8}).rki4_zsplit == 8
