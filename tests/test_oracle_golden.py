"""Pin the numpy oracle against outputs of the reference's own code
(tests/golden/*.npz, produced by tests/golden/make_golden.py)."""
from __future__ import annotations

import numpy as np
import pytest

import locks_oracle as orc
from cases import GQA_CASES, MLA_CASES, make_gqa, make_mla
from conftest import load_golden, t2n


def _layer_slabs(case, l, page):
    """Oracle summaries of every physical block of layer ``l``."""
    K = t2n(case.kv_caches[l][:, 0])                  # (NB, page, n_kv, d)
    return orc.rki4_build_pages(K)


def _code_mismatch(ref, new):
    Vr, Vn, Cr, Cn = orc.align_signs(ref, new)
    dv, dc = np.abs(Vr - Vn), np.abs(Cr - Cn)
    return dv, dc


@pytest.mark.parametrize("name", list(GQA_CASES))
def test_build_codes_match_reference(name):
    g = load_golden(name)
    case, c = make_gqa(name)
    page = c["shape"].page
    nb = g["slab_v4"].shape[0]
    blk = t2n(case.block_table[0, :nb]).astype(np.int64)
    new = orc.rki4_build_pages(t2n(case.kv_caches[0][:, 0])[blk])
    ref = {"v4": g["slab_v4"], "c8": g["slab_c8"]}
    dv, dc = _code_mismatch(ref, new)
    # bit-exact except at rounding ties: <= 0.1% of codes, <= 1 LSB
    assert dv.max() <= 1 and (dv > 0).mean() <= 1e-3
    assert dc.max() <= 1 and (dc > 0).mean() <= 1e-3
    dm = np.abs(g["slab_mu8"].astype(np.int16) - new["mu8"].astype(np.int16))
    assert dm.max() <= 1 and (dm > 0).mean() <= 1e-3
    for k in ("vs", "cs", "mus"):
        rel = np.abs(g["slab_" + k] - new[k]) / np.maximum(np.abs(g["slab_" + k]), 1e-12)
        assert rel.max() <= 2 ** -7, k               # at most one bf16 ulp
        assert (rel > 0).mean() <= 2e-3, k
    np.testing.assert_array_equal(g["slab_tag"], new["tag"])


@pytest.mark.parametrize("name", list(GQA_CASES))
def test_gqa_step_matches_reference(name):
    g = load_golden(name)
    case, c = make_gqa(name)
    sh = c["shape"]
    R = case.n_req
    bt, sl = t2n(case.block_table), t2n(case.seq_lens)
    npg, nsh, b = orc.derive_page_params(
        sl, sh.page, sh.window_pages, sh.sink_pages,
        0 if c["budget"] else sh.budget_pages, c["budget"] or 0.1)
    np.testing.assert_array_equal(npg, g["n_pages"])
    np.testing.assert_array_equal(nsh, g["n_sel_hi"])
    np.testing.assert_array_equal(b, g["b_fix"])
    hi_max = g["score_h"].shape[-1]
    for l in range(sh.n_layers):
        slabs = _layer_slabs(case, l, sh.page)
        res = orc.gqa_decode_step(
            slabs, t2n(case.q[l]), t2n(case.kv_caches[l][:, 0]),
            t2n(case.kv_caches[l][:, 1]), bt, sl, case.scale, n_kv=sh.n_kv,
            G=sh.G, page=sh.page, window=sh.window_pages, sink=sh.sink_pages,
            budget_pages=0 if c["budget"] else sh.budget_pages,
            budget=c["budget"] or 0.1, combine=c["combine"],
            split=int(g["split"]), pps_min=orc.pps_min_default(R, sh.n_kv))
        sh_ref = g["score_h"][l]
        # scores: the oracle's summaries differ from the reference's only by
        # the rare 1-LSB code flips of eigensolver rounding (a flip touches all G
        # scores of its page): all but 2% agree to 1e-4, the rest stay within 5e-2
        err = np.abs(res["score_h"][..., :hi_max] - sh_ref)
        assert (err > 1e-4 + 1e-4 * np.abs(sh_ref)).mean() <= 2e-2
        assert err.max() <= 5e-2
        # top-b on the REFERENCE's combined score must be bit-identical
        tab, cnt = orc.topb_select(
            np.pad(g["score"][l], ((0, 0), (0, 0), (0, case.max_pages - hi_max))),
            npg, nsh, b, sh.sink_pages)
        cm = g["page_table"].shape[-1]
        np.testing.assert_array_equal(cnt, g["page_cnt"][l])
        np.testing.assert_array_equal(tab[..., :cm], g["page_table"][l])
        # the oracle's own end-to-end selection: identical away from ties
        _assert_sets_match(res["page_table"], res["page_cnt"],
                           g["page_table"][l], g["page_cnt"][l],
                           g["score"][l], nsh, sh.sink_pages)
        # decode on the reference's page set vs the reference kernel output
        m, lp, acc = orc.sparse_decode_split(
            t2n(case.q[l]), t2n(case.kv_caches[l][:, 0]),
            t2n(case.kv_caches[l][:, 1]), bt,
            np.pad(g["page_table"][l], ((0, 0), (0, 0), (0, case.max_pages - cm)),
                   constant_values=-1),
            g["page_cnt"][l], sl, case.scale, sh.n_kv, sh.G, int(g["split"]),
            orc.pps_min_default(R, sh.n_kv))
        out = orc.merge_splits(m, lp, acc, g["page_cnt"][l], int(g["split"]),
                               orc.pps_min_default(R, sh.n_kv))
        np.testing.assert_allclose(out, g["out"][l], atol=2e-3, rtol=2e-3)
        ref64, _ = orc.attention_over_pages(
            t2n(case.q[l]), t2n(case.kv_caches[l][:, 0]),
            t2n(case.kv_caches[l][:, 1]), bt,
            np.pad(g["page_table"][l], ((0, 0), (0, 0), (0, case.max_pages - cm)),
                   constant_values=-1),
            g["page_cnt"][l], sl, case.scale, sh.n_kv, sh.G)
        np.testing.assert_allclose(out, ref64, atol=2e-3, rtol=2e-3)


def _assert_sets_match(tab, cnt, tab_ref, cnt_ref, score_ref, nsh, sink,
                       tol=1e-3):
    """Selected sets equal, except pages whose reference score is within
    ``tol`` (relative) of the reference threshold."""
    R, n_kv = cnt.shape
    np.testing.assert_array_equal(cnt, cnt_ref)
    for r in range(R):
        for kh in range(n_kv):
            a = set(tab[r, kh, :cnt[r, kh]].tolist())
            bset = set(tab_ref[r, kh, :cnt_ref[r, kh]].tolist())
            if a == bset:
                continue
            hi = int(nsh[r])
            sel = [p for p in bset if sink <= p < hi]
            tau = min(score_ref[r, kh, p] for p in sel)
            for p in a ^ bset:
                assert sink <= p < hi
                assert abs(score_ref[r, kh, p] - tau) <= tol * abs(tau), \
                    (r, kh, p, score_ref[r, kh, p], tau)


def test_topb_known_answers():
    g = load_golden("topb_kat")
    npg, nsh, b = orc.derive_page_params(g["seq_lens"], 16, 3, 2, 12)
    np.testing.assert_array_equal(npg, g["n_pages"])
    np.testing.assert_array_equal(nsh, g["n_sel_hi"])
    np.testing.assert_array_equal(b, g["b_fix"])
    tab, cnt = orc.topb_select(g["score"], npg, nsh, b, 2)
    np.testing.assert_array_equal(cnt, g["page_cnt"])
    np.testing.assert_array_equal(tab, g["page_table"])
    npg2, nsh2, b2 = orc.derive_page_params(g["seq_lens"], 16, 3, 2, 0, 0.07)
    np.testing.assert_array_equal(npg2, g["frac_n_pages"])
    np.testing.assert_array_equal(nsh2, g["frac_n_sel_hi"])
    np.testing.assert_array_equal(b2, g["frac_b_fix"])


@pytest.mark.parametrize("name", list(MLA_CASES))
def test_mla_matches_reference(name):
    g = load_golden(name)
    case, c = make_mla(name)
    sh = c["shape"]
    res = orc.mla_decode_step(
        t2n(case.q[0]), t2n(case.caches[0]), t2n(case.block_table),
        t2n(case.seq_lens), case.scale, Lkv=sh.kv_lora_rank, rank=c["rank"],
        budget_pages=sh.budget_pages, sink=sh.sink_pages,
        window=sh.window_pages)
    for bi in range(len(c["seq_lens"])):
        ref_s = g[f"score{bi}"]
        fin = np.isfinite(ref_s)
        if ref_s.shape[0] > sh.budget_pages:     # short rows are not scored
            np.testing.assert_allclose(res["page_score"][bi][fin], ref_s[fin],
                                       rtol=1e-4, atol=1e-4)
        np.testing.assert_array_equal(res["keep"][bi], g[f"keep{bi}"])
        np.testing.assert_allclose(res["o"][bi], g[f"o{bi}"], atol=1e-4, rtol=1e-4)
        np.testing.assert_allclose(res["lse"][bi], g[f"lse{bi}"], atol=1e-4,
                                   rtol=1e-4)
    # factors: Lf @ Rf is gauge-free
    page, Lkv = sh.page, sh.kv_lora_rank
    L0 = c["seq_lens"][0]
    blks = t2n(case.block_table[0, :L0 // page]).astype(np.int64)
    kv_c = t2n(case.caches[0])[blks].reshape(-1, sh.width)[:, :Lkv]
    Lf, Rf = orc.mla_build_page_factors(kv_c, L0 // page, page, c["rank"])
    n = g["Lf0"].shape[0]
    np.testing.assert_allclose(Lf[:n] @ Rf[:n], g["Lf0"] @ g["Rf0"], atol=2e-3)
