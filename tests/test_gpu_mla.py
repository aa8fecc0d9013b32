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
