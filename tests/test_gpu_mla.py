"""GPU parity of the MLA (latent KV) path against the numpy oracle and the
reference's golden outputs."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import locks_oracle as orc
from cases import MLA_CASES, make_mla
from conftest import load_golden, t2n

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _setup(name):
    from locks.selection import MlaState, build_prompt_factors, mla_derive
    cpu, c = make_mla(name)
    sh = c["shape"]
    cache = cpu.caches[0].to(DEV)
    bt = cpu.block_table.to(DEV)
    sl = cpu.seq_lens.to(DEV)
    q = cpu.q[0].to(DEV).contiguous()
    B = len(c["seq_lens"])
    st = MlaState(DEV, num_layers=1, num_blocks=cache.shape[0], max_rows=B,
                  max_pages=bt.shape[1], budget_pages=sh.budget_pages,
                  sink_pages=sh.sink_pages, window_pages=sh.window_pages)
    build_prompt_factors(st, [cache], bt, sl)
    mla_derive(st, sl, B)
    return cpu, c, sh, cache, bt, sl, q, st, B


@pytest.mark.parametrize("name", list(MLA_CASES))
def test_mla_factors_score_select_decode(name):
    from locks.selection import (mla_decode, mla_forward, mla_page_score,
                                 mla_select_pages)
    cpu, c, sh, cache, bt, sl, q, st, B = _setup(name)
    g = load_golden(name)
    page, Lkv = sh.page, sh.kv_lora_rank
    cache_np, bt_np, sl_np = t2n(cpu.caches[0]), t2n(cpu.block_table), t2n(cpu.seq_lens)
    ref = orc.mla_decode_step(t2n(cpu.q[0]), cache_np, bt_np, sl_np, cpu.scale,
                              Lkv=Lkv, rank=c["rank"],
                              budget_pages=sh.budget_pages, sink=sh.sink_pages,
                              window=sh.window_pages)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(t2n(st.n_cache), sl_np // page)

    # ---- factors: Lf Rf (gauge-free) against the oracle and the reference -----
    L0 = c["seq_lens"][0]
    blks = cpu.block_table[0, :L0 // page]
    Lf, Rf = st.factors(0, blks.to(DEV))
    rec = t2n(Lf @ Rf)
    kv_c = cache_np[t2n(blks).astype(np.int64)][:, :, :Lkv]
    Lo, Ro = orc.mla_build_page_factors(kv_c.reshape(-1, Lkv), L0 // page, page,
                                        c["rank"])
    want = Lo @ Ro
    denom = np.abs(want).max()
    assert np.abs(rec - want).max() <= 3e-3 * denom          # fp16 factors
    n = g["Lf0"].shape[0]
    assert np.abs(rec[:n] - g["Lf0"] @ g["Rf0"]).max() <= 3e-3 * denom

    # ---- scores ------------------------------------------------------------------
    mla_page_score(st, 0, q, cache, bt, B, cpu.scale)
    torch.cuda.synchronize()
    st.check_status()
    sc = t2n(st.score[:, 0])
    for bi in range(B):
        P = -(-int(sl_np[bi]) // page)
        nc = int(sl_np[bi]) // page
        if P > sh.budget_pages:
            want_s = ref["page_score"][bi]
            np.testing.assert_allclose(sc[bi, :nc], want_s[:nc], rtol=3e-3, atol=3e-3)
            np.testing.assert_allclose(sc[bi, :nc], g[f"score{bi}"][:nc], rtol=3e-3,
                                       atol=3e-3)
        assert np.isneginf(sc[bi, nc:P]).all()

    # ---- keep rule ---------------------------------------------------------------
    mla_select_pages(st, B)
    torch.cuda.synchronize()
    tab, cnt = t2n(st.page_table[:, 0]), t2n(st.page_cnt[:, 0])
    for bi in range(B):
        keep_ref = g[f"keep{bi}"]
        got = tab[bi, :cnt[bi]]
        assert cnt[bi] == keep_ref.shape[0]
        assert (np.diff(got) > 0).all()
        diff = set(got.tolist()) ^ set(keep_ref.tolist())
        if diff:                       # only pages tied with the threshold
            s_ref = g[f"score{bi}"]
            mid = [p for p in keep_ref.tolist()
                   if sh.sink_pages <= p < s_ref.shape[0] - sh.window_pages]
            tau = min(s_ref[p] for p in mid)
            for p in diff:
                assert abs(s_ref[p] - tau) <= 3e-3 * abs(tau) + 3e-3

    # ---- decode on the reference's kept pages -------------------------------------
    st.page_table.fill_(-1)
    for bi in range(B):
        k = g[f"keep{bi}"]
        st.page_table[bi, 0, :len(k)] = torch.from_numpy(k.astype(np.int32)).to(DEV)
        st.page_cnt[bi, 0] = len(k)
    out = torch.full((B, 16, Lkv), float("nan"), device=DEV, dtype=torch.bfloat16)
    lse = torch.full((B, 16), float("nan"), device=DEV, dtype=torch.float32)
    mla_decode(st, q, cache, bt, sl, out, lse, B, cpu.scale)
    torch.cuda.synchronize()
    st.check_status()
    for bi in range(B):
        # stated tolerance of the path: 2e-2 max-abs, 1e-2 relative (bf16 output)
        np.testing.assert_allclose(t2n(out[bi]), g[f"o{bi}"], atol=2e-2, rtol=1e-2)
        np.testing.assert_allclose(t2n(lse[bi]), g[f"lse{bi}"], atol=2e-3, rtol=2e-3)
        np.testing.assert_allclose(t2n(out[bi]), ref["o"][bi], atol=2e-2, rtol=1e-2)

    # ---- whole layer in three launches ----------------------------------------------
    out2 = torch.empty_like(out)
    lse2 = torch.empty_like(lse)
    mla_forward(st, 0, q, cache, bt, sl, out2, lse2, cpu.scale)
    torch.cuda.synchronize()
    for bi in range(B):
        np.testing.assert_allclose(t2n(out2[bi]), ref["o"][bi], atol=2e-2, rtol=1e-2)


def test_mla_full_size_properties():
    """Config 3 at full size -- batch 8 x 131072 tokens, 16 heads on one latent
    head of 576 -- for one of its 27 layers: counts, ascending tables, the exact
    keep rule against a torch sort of the DEVICE scores (forced sink + recent
    pages, best-scored middle pages up to the budget), scores of a page sample
    against the fp32 product the factors approximate, and o / lse against a
    plain torch attention over the kept pages."""
    from locks import synth
    from locks.selection import mla_select as ms
    sh = synth.CONFIG3
    dev = torch.device("cuda", 0)
    B, seq_len = 8, 131072 + 1
    case = synth.make_mla_case(77, sh, [seq_len] * B, device=dev, n_layers=1)
    MP, NB = int(case.block_table.shape[1]), int(case.caches[0].shape[0])
    st = ms.MlaState(dev, num_layers=1, num_blocks=NB, max_rows=B, max_pages=MP,
                     budget_pages=sh.budget_pages, sink_pages=sh.sink_pages,
                     window_pages=sh.window_pages)
    ms.mla_derive(st, case.seq_lens, B)
    ms.build_prompt_factors(st, case.caches, case.block_table, case.seq_lens)
    out = torch.zeros(B, sh.n_heads, sh.kv_lora_rank, device=dev, dtype=torch.bfloat16)
    lse = torch.zeros(B, sh.n_heads, device=dev)
    ms.mla_forward(st, 0, case.q[0], case.caches[0], case.block_table,
                   case.seq_lens, out, lse, case.scale)
    torch.cuda.synchronize()
    st.check_status()
    npg = -(-seq_len // sh.page)
    n_cache = seq_len // sh.page
    assert (st.n_pages[:B] == npg).all() and (st.n_cache[:B] == n_cache).all()
    A = sh.budget_pages                       # the MLA budget includes forced pages
    assert (st.page_cnt[:B, 0] == A).all()
    tab = st.page_table[:B, 0]
    assert (tab[:, A:] == -1).all()
    assert (tab[:, 1:A] > tab[:, :A - 1]).all()
    score = st.score[:B, 0]
    assert torch.isfinite(score[:, :n_cache]).all()
    nsh = npg - sh.window_pages
    forced = list(range(sh.sink_pages)) + list(range(nsh, npg))
    n_mid = A - len(forced)
    for r in range(B):
        mid = score[r, sh.sink_pages:nsh]
        order = torch.sort(mid, descending=True, stable=True).indices[:n_mid] \
            + sh.sink_pages
        assert tab[r, :A].tolist() == sorted(order.tolist() + forced), r
    # scores of a sample of pages against the oracle's factored scorer on the
    # same pages (fp16 factors: the 3e-3 band of the small-case test)
    cache, q = case.caches[0], case.q[0].float()
    g = torch.Generator().manual_seed(1)
    for r in (0, B - 1):
        pages = torch.randint(0, n_cache, (64,), generator=g)
        blks = case.block_table[r, pages.to(dev)].long()
        kv = t2n(cache[blks])                                      # (64, 16, 576)
        Lf, Rf = orc.mla_build_page_factors(
            kv[:, :, :sh.kv_lora_rank].reshape(-1, sh.kv_lora_rank), 64, sh.page, 8)
        qr = t2n(case.q[0][r])
        want = orc.mla_page_score(qr[:, :sh.kv_lora_rank], qr[:, sh.kv_lora_rank:],
                                  Lf, Rf, kv[:, :, sh.kv_lora_rank:],
                                  np.full(64, sh.page), case.scale)
        np.testing.assert_allclose(t2n(score[r, pages.to(dev)]), want, rtol=3e-3,
                                   atol=3e-3)
    out_tc = torch.zeros_like(out)
    lse_tc = torch.zeros_like(lse)
    ms.mla_decode(st, case.q[0], case.caches[0], case.block_table, case.seq_lens,
                  out_tc, lse_tc, B, case.scale, tensor_core=True)
    torch.cuda.synchronize()
    st.check_status()
    # attention over the kept pages, plain torch fp32
    for r in (0, 3, B - 1):
        pg = tab[r, :A].long()
        blks = case.block_table[r, pg].long()
        kv = cache[blks].reshape(-1, sh.width).float()
        pos = (pg[:, None] * sh.page + torch.arange(sh.page, device=dev)[None]).reshape(-1)
        s_ = (q[r] @ kv.T) * case.scale
        s_ = s_.masked_fill(~(pos < seq_len)[None], float("-inf"))
        o_ref = torch.softmax(s_, -1) @ kv[:, :sh.kv_lora_rank]
        torch.testing.assert_close(out[r].float(), o_ref, atol=2e-2, rtol=1e-2)
        torch.testing.assert_close(lse[r], torch.logsumexp(s_, -1), atol=2e-2,
                                   rtol=1e-2)
        # the tcgen05 kernel on the same kept pages
        torch.testing.assert_close(out_tc[r].float(), o_ref, atol=2e-2, rtol=1e-2)
        torch.testing.assert_close(lse_tc[r], torch.logsumexp(s_, -1), atol=2e-2,
                                   rtol=1e-2)


@pytest.mark.parametrize("lens", [[777, 2053, 300, 16, 5000], [130, 4096 + 7]])
def test_mla_tensor_core_decode_equals_warp_level_decode(lens):
    """The tcgen05 decode (tokens in M, TMA page gather, accumulators in tensor
    memory) against the warp-level kernel on the same kept pages: rows shorter
    than a tile, partial last pages, several tiles per CTA (a dense selection:
    budget >= pages) and the sparse selection of the path."""
    from locks import synth
    from locks.selection import mla_select as ms
    sh = synth.MlaShape(n_layers=1, budget_pages=24, sink_pages=1, window_pages=4)
    case = synth.make_mla_case(5, sh, lens, device=DEV, n_layers=1)
    B = len(lens)
    MP, NB = int(case.block_table.shape[1]), int(case.caches[0].shape[0])
    for budget in (24, MP):
        st = ms.MlaState(DEV, num_layers=1, num_blocks=NB, max_rows=B, max_pages=MP,
                         budget_pages=budget, sink_pages=1, window_pages=4)
        ms.mla_derive(st, case.seq_lens, B)
        ms.build_prompt_factors(st, case.caches, case.block_table, case.seq_lens)
        ms.mla_page_score(st, 0, case.q[0], case.caches[0], case.block_table, B,
                          case.scale)
        ms.mla_select_pages(st, B)
        outs = []
        for tc in (False, True):
            out = torch.full((B, 16, 512), float("nan"), device=DEV,
                             dtype=torch.bfloat16)
            lse = torch.full((B, 16), float("nan"), device=DEV)
            ms.mla_decode(st, case.q[0], case.caches[0], case.block_table,
                          case.seq_lens, out, lse, B, case.scale, tensor_core=tc)
            torch.cuda.synchronize()
            st.check_status()
            outs.append((out.float(), lse))
        (o0, l0), (o1, l1) = outs
        assert torch.isfinite(o1).all() and torch.isfinite(l1).all()
        # both within the decode tolerance of each other (bf16 P in the tensor-core
        # kernel, hi+lo split P in the warp-level one)
        torch.testing.assert_close(o1, o0, atol=2e-2, rtol=1e-2)
        torch.testing.assert_close(l1, l0, atol=2e-3, rtol=2e-3)


def test_mla_factor_bookkeeping_on_the_device():
    """``mla_refresh_rows`` (no host synchronisation): first decode step builds
    every row's factors; steady decode steps (the sequences grow, new tokens land
    in later pages) flag nothing and keep n_cache; a finished request's block
    ids handed to a new request are caught by the content fingerprint and
    rebuilt; a row that shrank (preemption) is rebuilt."""
    from locks import synth
    from locks.selection import mla_select as ms
    sh = synth.MlaShape(n_layers=1, budget_pages=24, sink_pages=1, window_pages=4)
    lens = [777, 2053, 300, 40]
    case = synth.make_mla_case(9, sh, lens, device=DEV, n_layers=1, max_pages=160)
    cache, bt = case.caches[0], case.block_table
    B, MP, NB = len(lens), int(bt.shape[1]), int(cache.shape[0])

    def state():
        return ms.MlaState(DEV, num_layers=1, num_blocks=NB, max_rows=8, max_pages=MP,
                           budget_pages=24, sink_pages=1, window_pages=4)
    st = state()
    sl = case.seq_lens.clone()
    ms.mla_refresh_rows(st, 0, cache, bt, sl, B)
    torch.cuda.synchronize()
    assert st.need[:B].tolist() == [1, 1, 1, 1]
    assert st.n_cache[:B].tolist() == [n // 16 for n in lens]
    ref = state()
    ms.build_prompt_factors(ref, [cache], bt, sl)
    torch.cuda.synchronize()
    used = torch.cat([bt[r, :lens[r] // 16] for r in range(B)]).long()
    assert torch.equal(st.records[0][used], ref.records[0][used])
    # steady decode: 20 more tokens per row, written into the tail pages
    g = torch.Generator().manual_seed(3)
    for step in range(20):
        for r in range(B):
            tok = lens[r] + step
            blk = int(bt[r, tok // 16]) if tok // 16 < -(-lens[r] // 16) else None
            if blk is not None:
                cache[blk, tok % 16] = torch.randn(576, generator=g).to(torch.bfloat16).to(DEV)
        sl += 1
        ms.mla_refresh_rows(st, 0, cache, bt, sl, B)
    torch.cuda.synchronize()
    assert st.need[:B].tolist() == [0, 0, 0, 0]
    assert st.n_cache[:B].tolist() == [n // 16 for n in lens]      # entries as built
    # row 2 finishes; a new request gets its block ids with other content
    n2 = 300 // 16
    cache[bt[2, :n2 + 1].long()] = torch.randn(n2 + 1, 16, 576, generator=g) \
        .to(torch.bfloat16).to(DEV)
    sl[2] = 290
    ms.mla_refresh_rows(st, 0, cache, bt, sl, B)
    torch.cuda.synchronize()
    assert st.need[:B].tolist() == [0, 0, 1, 0]
    assert int(st.n_cache[2]) == 290 // 16
    ref = state()
    ms.build_prompt_factors(ref, [cache], bt, sl, rows=[2])
    torch.cuda.synchronize()
    b2 = bt[2, :290 // 16].long()
    assert torch.equal(st.records[0][b2], ref.records[0][b2])
    # row 1 is preempted and resumes shorter than its entry
    sl[1] = 1000
    ms.mla_refresh_rows(st, 0, cache, bt, sl, B)
    torch.cuda.synchronize()
    assert st.need[:B].tolist() == [0, 1, 0, 0]
    assert int(st.n_cache[1]) == 1000 // 16
    st.check_status()
