"""The allocation-free decode entry point.

``locks_decode_split_noalloc`` serves callers that may not allocate device
memory themselves (they can only pass on buffers they were handed), so its
split partials sit in a fixed array inside the library instead of in
caller-owned scratch.  This file checks, through the C ABI, that it returns what
the ordinary split + merge pair returns -- twice in a row with different inputs,
because the shared array keeps the previous call's contents -- and that sizes
beyond the built-in scratch are refused.  It is collected last on purpose.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from cases import make_gqa
from conftest import t2n

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_noalloc_decode_matches_split_merge_twice():
    from locks.attention import (ResidentVSource, ensure_stage_b_buffers,
                                 sparse_paged_decode_batched)
    from locks.attention.decode import sparse_paged_decode_noalloc
    from locks.selection import (Rki4State, derive_page_params,
                                 rki4_build_bulk, rki4_score_state)
    cpu, c = make_gqa("gqa_ragged")
    sh = c["shape"]
    caches = [k.to(DEV) for k in cpu.kv_caches]
    bt, sl = cpu.block_table.to(DEV), cpu.seq_lens.to(DEV)
    R, H = cpu.n_req, sh.n_kv * sh.G
    st = Rki4State(DEV, num_layers=sh.n_layers, num_blocks=cpu.num_blocks,
                   n_kv=sh.n_kv, G=sh.G, head_dim=sh.d, page=sh.page, max_reqs=R,
                   max_pages=cpu.max_pages, budget_pages=sh.budget_pages,
                   sink_pages=sh.sink_pages, window_pages=sh.window_pages)
    st.scale = cpu.scale
    ensure_stage_b_buffers(st, DEV, 32, adapt=False)
    rki4_build_bulk(st, [k[:, 0] for k in caches], bt, sl - 1, R,
                    int((t2n(sl).max() - 1) // sh.page))
    derive_page_params(st, sl, R)
    for l in range(sh.n_layers):          # two calls in a row, different inputs
        q = cpu.q[l].to(DEV).contiguous()
        rki4_score_state(st, l, q, bt, sl, R, cpu.scale)
        want = torch.full((R, H, sh.d), float("nan"), device=DEV, dtype=torch.bfloat16)
        got = torch.full_like(want, float("nan"))
        vs = ResidentVSource(caches[l])
        sparse_paged_decode_batched(q, caches[l], bt, sl, st, want, vs,
                                    scale=cpu.scale)
        sparse_paged_decode_noalloc(q, caches[l], bt, sl, st, got, vs,
                                    split=st.split, scale=cpu.scale)
        torch.cuda.synchronize()
        st.check_status()
        a, b = t2n(want), t2n(got)
        assert np.isfinite(b).all()
        # same kernels, same split: the decode tolerance (2e-2 abs, 1e-2 rel)
        # is far wider than needed, the results are expected to be identical
        np.testing.assert_allclose(b, a, atol=2e-2, rtol=1e-2)
        assert np.abs(a - b).max() == 0.0


def test_noalloc_at_the_exact_row_limit_g16():
    """n_req * n_kv * split * G == 16384 exactly, with 16 query heads per KV
    head: the last partial row sits on the boundary between the m, l and acc
    parts of the in-library array.  Bit-identical to the caller-owned pair."""
    from locks import synth
    from locks.attention import (ResidentVSource, ensure_stage_b_buffers,
                                 sparse_paged_decode_batched)
    from locks.attention.decode import (NOALLOC_MAX_ROWS,
                                        sparse_paged_decode_noalloc)
    from locks.selection import (Rki4State, derive_page_params,
                                 rki4_build_bulk, rki4_score_state)
    sh = synth.GqaShape(n_layers=1, n_kv=2, G=16, budget_pages=150,
                        sink_pages=1, window_pages=2, n_needles=2)
    lens = [3100, 2049, 1500, 40]
    split = 128
    assert len(lens) * sh.n_kv * split * sh.G == NOALLOC_MAX_ROWS
    cpu = synth.make_gqa_case(17, sh, lens)
    cache = cpu.kv_caches[0].to(DEV)
    bt, sl = cpu.block_table.to(DEV), cpu.seq_lens.to(DEV)
    R, H = cpu.n_req, sh.n_kv * sh.G
    st = Rki4State(DEV, num_layers=1, num_blocks=cpu.num_blocks, n_kv=sh.n_kv,
                   G=sh.G, head_dim=sh.d, page=sh.page, max_reqs=R,
                   max_pages=cpu.max_pages, budget_pages=sh.budget_pages,
                   sink_pages=sh.sink_pages, window_pages=sh.window_pages)
    st.scale = cpu.scale
    ensure_stage_b_buffers(st, DEV, split, adapt=False)
    assert st.split == split
    rki4_build_bulk(st, [cache[:, 0]], bt, sl - 1, R,
                    int((t2n(sl).max() - 1) // sh.page))
    derive_page_params(st, sl, R)
    q = cpu.q[0].to(DEV).contiguous()
    rki4_score_state(st, 0, q, bt, sl, R, cpu.scale)
    want = torch.full((R, H, sh.d), float("nan"), device=DEV, dtype=torch.bfloat16)
    got = torch.full_like(want, float("nan"))
    vs = ResidentVSource(cache)
    sparse_paged_decode_batched(q, cache, bt, sl, st, want, vs, scale=cpu.scale)
    sparse_paged_decode_noalloc(q, cache, bt, sl, st, got, vs, split=split,
                                scale=cpu.scale)
    torch.cuda.synchronize()
    st.check_status()
    assert np.isfinite(t2n(got)).all()
    assert torch.equal(got, want)


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from locks import _cabi
    z = torch.zeros(64, device=DEV, dtype=torch.int32)
    x = torch.zeros(4096, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="exceeds the built-in scratch"):
        _cabi.call("locks_decode_split_noalloc", _cabi.ptr(x), 512, _cabi.ptr(x),
                   _cabi.ptr(x), 4096, 256, 128, _cabi.ptr(z), 8, _cabi.ptr(z),
                   _cabi.ptr(z), _cabi.ptr(z), _cabi.ptr(x), 512,
                   8, 8, 16, 128, 16, 8, 128, 1, 0.1, _cabi.ptr(None),
                   _cabi.stream())
    # one row past the limit: 5 * 29 * 113 * 1 = 16385
    with pytest.raises(RuntimeError, match="exceeds the built-in scratch"):
        _cabi.call("locks_decode_split_noalloc", _cabi.ptr(x), 512, _cabi.ptr(x),
                   _cabi.ptr(x), 4096, 256, 128, _cabi.ptr(z), 8, _cabi.ptr(z),
                   _cabi.ptr(z), _cabi.ptr(z), _cabi.ptr(x), 512,
                   5, 29, 1, 128, 16, 8, 113, 1, 0.1, _cabi.ptr(None),
                   _cabi.stream())
