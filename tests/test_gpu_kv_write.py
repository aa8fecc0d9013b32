"""GPU parity of the KV-write neighbour: rotated K and V land in the paged cache
bit-exactly as the oracle's restatement of the reference kernel says, and the
summary of a page completed by the write equals the stand-alone builder's."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import locks_oracle as orc
from conftest import t2n

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _table(P, rot, seed):
    g = torch.Generator().manual_seed(seed)
    ang = torch.rand(P, rot // 2, generator=g) * 6.28
    return torch.cat([ang.cos(), ang.sin()], 1).to(torch.bfloat16)


@pytest.mark.parametrize("neox", [True, False])
@pytest.mark.parametrize("rot", [128, 64])
def test_rope_and_cache_bit_exact(neox, rot):
    from locks.attention import rope_and_cache
    n_tok, n_kv, d, page, NB, P = 7, 8, 128, 16, 12, 4096
    g = torch.Generator().manual_seed(5 + rot + int(neox))
    key = torch.randn(n_tok, n_kv, d, generator=g).to(torch.bfloat16)
    val = torch.randn(n_tok, n_kv, d, generator=g).to(torch.bfloat16)
    cache = torch.randn(NB, 2, page, n_kv, d, generator=g).to(torch.bfloat16)
    cs = _table(P, rot, 9)
    slots = torch.tensor([3 * page + 5, 0, -1, 11 * page + 15, 7 * page + 1,
                          2 * page + 9, 5 * page + 4], dtype=torch.int64)
    pos = torch.tensor([100, 0, 7, 4095, 17, 2049, 333], dtype=torch.int64)
    kc = cache[:, 0].float().numpy().copy()
    vc = cache[:, 1].float().numpy().copy()
    orc.rope_and_cache(key.float().numpy(), val.float().numpy(), kc, vc,
                       slots.numpy(), pos.numpy(), cs.float().numpy(), rot, neox,
                       page)
    dev_cache = cache.to(DEV)
    rope_and_cache(key.to(DEV), val.to(DEV), dev_cache, slots.to(DEV),
                   pos.to(DEV), cs.to(DEV), neox=neox)
    torch.cuda.synchronize()
    got_k, got_v = t2n(dev_cache[:, 0].float()), t2n(dev_cache[:, 1].float())
    assert np.array_equal(got_k, kc)
    assert np.array_equal(got_v, vc)


def test_plain_copy_without_table_and_strided_rows():
    from locks.attention import rope_and_cache
    n_tok, n_kv, d, page, NB = 3, 2, 128, 16, 4
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(n_tok, 3 * n_kv, d, generator=g).to(torch.bfloat16).to(DEV)
    key, val = qkv[:, n_kv:2 * n_kv], qkv[:, 2 * n_kv:]       # strided views
    cache = torch.zeros(2, NB, page, n_kv, d, dtype=torch.bfloat16, device=DEV)
    slots = torch.tensor([17, 2, 63], dtype=torch.int64, device=DEV)
    rope_and_cache(key, val, cache, slots, None, None)
    torch.cuda.synchronize()
    for r, s in enumerate([17, 2, 63]):
        assert torch.equal(cache[0, s // page, s % page], key[r])
        assert torch.equal(cache[1, s // page, s % page], val[r])
    assert int((cache != 0).any(-1).any(-1).sum()) == 2 * n_tok


def test_page_completion_builds_the_summary():
    """The write that lands on token 15 of a block leaves the block's records
    and tags exactly as a stand-alone build of that block does."""
    from locks.attention import rope_and_cache
    from locks.selection import Rki4State, rki4_build_bulk
    n_kv, G, d, page, NB = 8, 4, 128, 16, 6
    g = torch.Generator().manual_seed(21)
    cache = torch.randn(NB, 2, page, n_kv, d, generator=g).to(torch.bfloat16).to(DEV)

    def state():
        return Rki4State(DEV, num_layers=1, num_blocks=NB, n_kv=n_kv, G=G,
                         head_dim=d, page=page, max_reqs=2, max_pages=NB)
    st = state()
    key = torch.randn(2, n_kv, d, generator=g).to(torch.bfloat16).to(DEV)
    val = torch.randn(2, n_kv, d, generator=g).to(torch.bfloat16).to(DEV)
    cs = _table(64, d, 4).to(DEV)
    # row 0 completes block 4, row 1 lands mid-page in block 2
    slots = torch.tensor([4 * page + 15, 2 * page + 3], dtype=torch.int64, device=DEV)
    pos = torch.tensor([31, 9], dtype=torch.int64, device=DEV)
    rope_and_cache(key, val, cache, slots, pos, cs, neox=True, st=st, lidx=0)
    torch.cuda.synchronize()
    # stand-alone build of block 4 from the cache as it is now
    ref = state()
    bt = torch.tensor([[4, 2]], dtype=torch.int32, device=DEV)
    settled = torch.tensor([2 * page], dtype=torch.int32, device=DEV)
    rki4_build_bulk(ref, [cache[:, 0]], bt, settled, 1, 1)      # page 0 -> block 4
    torch.cuda.synchronize()
    assert torch.equal(st.pp_rec[0, 4], ref.pp_rec[0, 4])
    assert torch.equal(st.pp_tag[0, 4].view(torch.int16),
                       ref.pp_tag[0, 4].view(torch.int16))
    # nothing else was built: block 2 still carries the never-built NaN tag
    assert bool(torch.isnan(st.pp_tag[0, 2].float()).all())
    assert int(st.pp_rec[0, 2].abs().sum()) == 0


def test_rows_of_one_page_in_one_launch():
    """A launch that stores SEVERAL rows of the same page (a prefill chunk): the
    CTA of the row that completes the page must not summarise it before its
    siblings' rows are in the cache.  All 16 rows of a block arrive in one
    launch (the completing row first, so that its CTA is scheduled first); the
    summary equals a stand-alone build of the final cache."""
    from locks.attention import rope_and_cache
    from locks.selection import Rki4State, rki4_build_bulk
    n_kv, G, d, page, NB = 8, 4, 128, 16, 5
    g = torch.Generator().manual_seed(314)
    cache = torch.zeros(NB, 2, page, n_kv, d, dtype=torch.bfloat16, device=DEV)

    def state():
        return Rki4State(DEV, num_layers=1, num_blocks=NB, n_kv=n_kv, G=G,
                         head_dim=d, page=page, max_reqs=1, max_pages=NB)
    for trial in range(8):
        st = state()
        cache.zero_()
        key = torch.randn(page, n_kv, d, generator=g).to(torch.bfloat16).to(DEV)
        val = torch.randn(page, n_kv, d, generator=g).to(torch.bfloat16).to(DEV)
        order = [15] + list(range(15))
        slots = torch.tensor([3 * page + t for t in order], dtype=torch.int64,
                             device=DEV)
        rope_and_cache(key, val, cache, slots, None, None, st=st, lidx=0)
        ref = state()
        bt = torch.tensor([[3]], dtype=torch.int32, device=DEV)
        settled = torch.tensor([page], dtype=torch.int32, device=DEV)
        rki4_build_bulk(ref, [cache[:, 0]], bt, settled, 1, 1)
        torch.cuda.synchronize()
        for r, t in enumerate(order):
            assert torch.equal(cache[3, 0, t], key[r])
        assert torch.equal(st.pp_rec[0, 3], ref.pp_rec[0, 3]), trial
        assert torch.equal(st.pp_tag[0, 3].view(torch.int16),
                           ref.pp_tag[0, 3].view(torch.int16))


def test_slot_driven_build_matches_block_list_build():
    """locks_rki4_build_slots builds exactly the blocks whose last slot was
    written this step, in every layer, and leaves the others alone."""
    from locks.selection import Rki4State, rki4_build_bulk, rki4_build_slots
    n_kv, G, d, page, NB, L = 2, 16, 128, 16, 8, 3
    g = torch.Generator().manual_seed(77)
    caches = [torch.randn(NB, 2, page, n_kv, d, generator=g).to(torch.bfloat16).to(DEV)
              for _ in range(L)]
    K_layers = [c[:, 0] for c in caches]

    def state():
        return Rki4State(DEV, num_layers=L, num_blocks=NB, n_kv=n_kv, G=G,
                         head_dim=d, page=page, max_reqs=4, max_pages=NB)
    st = state()
    # tokens: completes block 5, mid-page in block 1, skipped row, completes block 2
    slots = torch.tensor([5 * page + 15, 1 * page + 7, -1, 2 * page + 15],
                         dtype=torch.int64, device=DEV)
    rki4_build_slots(st, K_layers, slots)
    ref = state()
    bt = torch.tensor([[5], [2]], dtype=torch.int32, device=DEV)
    settled = torch.tensor([page, page], dtype=torch.int32, device=DEV)
    rki4_build_bulk(ref, K_layers, bt, settled, 2, 1)
    torch.cuda.synchronize()
    for blk in (5, 2):
        assert torch.equal(st.pp_rec[:, blk], ref.pp_rec[:, blk])
        assert torch.equal(st.pp_tag[:, blk].view(torch.int16),
                           ref.pp_tag[:, blk].view(torch.int16))
    for blk in (0, 1, 3, 4, 6, 7):
        assert bool(torch.isnan(st.pp_tag[:, blk].float()).all())
        assert int(st.pp_rec[:, blk].abs().sum()) == 0


@pytest.mark.parametrize("MP,R,n_kv", [(48, 3, 2),       # one CTA per row
                                       (8200, 1, 8),     # owner CTA + helper CTAs
                                       (40000, 2, 2)])   # a cluster of slices
def test_selector_carries_the_kv_write(MP, R, n_kv):
    """``rki4_select_only(..., append=desc)`` leaves the cache exactly as
    ``rope_and_cache`` does (and as the oracle says), for every way the selector
    spreads a row over CTAs, and selects exactly what it selects without the
    write.  One row carries slot -1: nothing may be stored for it."""
    from locks.attention import kv_append_desc, rope_and_cache
    from locks.selection import Rki4State, derive_page_params, rki4_select_only
    G, d, page, NB = 4, 128, 16, 9
    g = torch.Generator().manual_seed(MP + R)
    cache = torch.randn(NB, 2, page, n_kv, d, generator=g).to(torch.bfloat16)
    key = torch.randn(R, n_kv, d, generator=g).to(torch.bfloat16)
    val = torch.randn(R, n_kv, d, generator=g).to(torch.bfloat16)
    cs = _table(512, 64, 3)
    slots = torch.tensor([5 * page + 15, -1, 2 * page + 4][:R], dtype=torch.int64)
    pos = torch.tensor([300, 7, 511][:R], dtype=torch.int64)
    kc = cache[:, 0].float().numpy().copy()
    vc = cache[:, 1].float().numpy().copy()
    orc.rope_and_cache(key.float().numpy(), val.float().numpy(), kc, vc,
                       slots.numpy(), pos.numpy(), cs.float().numpy(), 64, False,
                       page)
    st = Rki4State(DEV, num_layers=1, num_blocks=NB, n_kv=n_kv, G=G, head_dim=d,
                   page=page, max_reqs=R, max_pages=MP, budget_pages=20,
                   sink_pages=1, window_pages=2)
    sl = torch.tensor([MP * 16 - 3, 40, (MP // 2) * 16 + 1][:R], dtype=torch.int32)
    derive_page_params(st, sl.to(DEV), R)
    st.score_h.copy_(torch.randn(R, n_kv, G, MP, generator=g).to(DEV))
    rki4_select_only(st, R, has_hmax=False)
    torch.cuda.synchronize()
    tab0, cnt0 = st.page_table.clone(), st.page_cnt.clone()
    st.page_table.fill_(-7)
    dev_key, dev_val, dev_cache = key.to(DEV), val.to(DEV), cache.to(DEV)
    dev_slots, dev_pos, dev_cs = slots.to(DEV), pos.to(DEV), cs.to(DEV)
    desc = kv_append_desc(dev_key, dev_val, dev_cache, dev_slots, dev_pos, dev_cs,
                          neox=False)
    rki4_select_only(st, R, has_hmax=False, append=desc)
    torch.cuda.synchronize()
    assert torch.equal(st.page_table, tab0) and torch.equal(st.page_cnt, cnt0)
    assert np.array_equal(t2n(dev_cache[:, 0].float()), kc)
    assert np.array_equal(t2n(dev_cache[:, 1].float()), vc)
    # and the stand-alone kernel agrees
    ref_cache = cache.to(DEV)
    rope_and_cache(dev_key, dev_val, ref_cache, dev_slots, dev_pos, dev_cs,
                   neox=False)
    torch.cuda.synchronize()
    assert torch.equal(ref_cache, dev_cache)
