"""GPU parity: every GQA stage, called through the C ABI, against the numpy
oracle on the same seeded inputs and against the reference's golden outputs."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import locks_oracle as orc
from cases import GQA_CASES, make_gqa
from conftest import load_golden, t2n

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _state(case, c, max_reqs=None):
    from locks.attention import ensure_stage_b_buffers
    from locks.selection import Rki4State
    sh = c["shape"]
    st = Rki4State(DEV, num_layers=sh.n_layers, num_blocks=case.num_blocks,
                   n_kv=sh.n_kv, G=sh.G, head_dim=sh.d, page=sh.page,
                   max_reqs=max_reqs or c["max_reqs"], max_pages=case.max_pages,
                   budget=c["budget"] or 0.1,
                   budget_pages=None if c["budget"] else sh.budget_pages,
                   sink_pages=sh.sink_pages, window_pages=sh.window_pages,
                   combine=c["combine"])
    st.scale = case.scale
    ensure_stage_b_buffers(st, DEV, 128)
    return st


def _gpu_case(name):
    case, c = make_gqa(name)
    g = make_gqa(name)[0]            # CPU copy for the oracle
    case.kv_caches = [k.to(DEV) for k in case.kv_caches]
    case.q = case.q.to(DEV)
    case.block_table = case.block_table.to(DEV)
    case.seq_lens = case.seq_lens.to(DEV)
    return case, g, c


def _slabs_from_state(st, layer):
    v4, vs, c8, cs, mu8, mus, tag = st.layer_state(layer)
    return {"v4": t2n(v4), "vs": t2n(vs), "c8": t2n(c8), "cs": t2n(cs),
            "mu8": t2n(mu8), "mus": t2n(mus), "tag": t2n(tag)}


def _upload_slabs(st, layer, slabs):
    st.pp_v4[layer].copy_(torch.from_numpy(slabs["v4"]).to(DEV))
    st.pp_vs[layer].copy_(torch.from_numpy(slabs["vs"]).to(DEV).bfloat16())
    st.pp_c8[layer].copy_(torch.from_numpy(slabs["c8"]).to(DEV))
    st.pp_cs[layer].copy_(torch.from_numpy(slabs["cs"]).to(DEV).bfloat16())
    st.pp_mu8[layer].copy_(torch.from_numpy(slabs["mu8"]).to(DEV))
    st.pp_mus[layer].copy_(torch.from_numpy(slabs["mus"]).to(DEV).bfloat16())


def _finalized_blocks(cpu_case, page):
    bt, sl = t2n(cpu_case.block_table), t2n(cpu_case.seq_lens) - 1
    out = []
    for r in range(bt.shape[0]):
        out.extend(bt[r, :sl[r] // page].tolist())
    return np.array(sorted(set(out)), dtype=np.int64)


def _few(mask, frac):
    """At most `frac` of the entries (but always allow 2: tiny samples)."""
    return int(mask.sum()) <= max(2, int(np.ceil(frac * mask.size)))


def _check_codes(ref, new, idx):
    """<= 0.1 % of codes differ, each by <= 1 LSB, after sign alignment."""
    Vr, Vn, Cr, Cn = orc.align_signs({k: v[idx] for k, v in ref.items()},
                                     {k: v[idx] for k, v in new.items()})
    dv, dc = np.abs(Vr - Vn), np.abs(Cr - Cn)
    assert dv.max() <= 1 and _few(dv > 0, 1e-3), ((dv > 0).mean(), dv.max())
    assert dc.max() <= 1 and _few(dc > 0, 1e-3), ((dc > 0).mean(), dc.max())
    dm = np.abs(ref["mu8"][idx].astype(np.int16) - new["mu8"][idx].astype(np.int16))
    assert dm.max() <= 1 and _few(dm > 0, 1e-3)
    for k in ("vs", "cs", "mus"):
        a, b = ref[k][idx], new[k][idx]
        rel = np.abs(a - b) / np.maximum(np.abs(a), 1e-12)
        # stored scales are bf16: at most one ulp apart, and rarely
        assert rel.max() <= 2 ** -7 and _few(rel > 0, 5e-3), (k, rel.max())


@pytest.mark.parametrize("name", list(GQA_CASES))
def test_build_matches_oracle_and_reference(name):
    from locks.selection import rki4_build_bulk
    case, cpu, c = _gpu_case(name)
    sh = c["shape"]
    st = _state(case, c)
    K_layers = [kc[:, 0] for kc in case.kv_caches]
    settled = case.seq_lens - 1
    max_fin = int((t2n(settled) // sh.page).max())
    n = rki4_build_bulk(st, K_layers, case.block_table, settled, case.n_req,
                        max_fin)
    torch.cuda.synchronize()
    g = load_golden(name)
    assert n == int(g["n_built"])
    fin = _finalized_blocks(cpu, sh.page)
    for l in range(sh.n_layers):
        new = _slabs_from_state(st, l)
        ref = orc.rki4_build_pages(t2n(cpu.kv_caches[l][:, 0]))
        _check_codes(ref, new, fin)
        np.testing.assert_array_equal(ref["tag"][fin], new["tag"][fin])
    # the reference's own slabs (first pages of request 0, layer 0)
    nb = g["slab_v4"].shape[0]
    blk = t2n(cpu.block_table[0, :nb]).astype(np.int64)
    new0 = _slabs_from_state(st, 0)
    refg = {"v4": g["slab_v4"], "c8": g["slab_c8"], "mu8": g["slab_mu8"],
            "vs": g["slab_vs"], "cs": g["slab_cs"], "mus": g["slab_mus"]}
    _check_codes(refg, {k: v[blk] for k, v in new0.items() if k != "tag"},
                 np.arange(nb))
    # never-built blocks keep their NaN tag
    unbuilt = np.setdiff1d(np.arange(case.num_blocks), np.append(fin, 0))
    if unbuilt.size:
        assert np.isnan(new0["tag"][unbuilt]).all()


@pytest.mark.parametrize("name", list(GQA_CASES))
def test_derive_score_select_decode(name):
    from locks.attention import (ResidentVSource, sparse_paged_decode_batched,
                                 sparse_paged_decode_fused)
    from locks.attention.decode import _pps_min
    from locks.selection import (derive_page_params, rki4_score_only,
                                 rki4_select_only, topb_select)
    case, cpu, c = _gpu_case(name)
    sh = c["shape"]
    g = load_golden(name)
    st = _state(case, c)
    R, MR = case.n_req, c["max_reqs"]
    H = sh.n_kv * sh.G
    bt_np, sl_np = t2n(cpu.block_table), t2n(cpu.seq_lens)

    derive_page_params(st, case.seq_lens, R)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(t2n(st.n_pages[:R]), g["n_pages"])
    np.testing.assert_array_equal(t2n(st.n_sel_hi[:R]), g["n_sel_hi"])
    np.testing.assert_array_equal(t2n(st.b_fix[:R]), g["b_fix"])
    npg, nsh, b = g["n_pages"], g["n_sel_hi"], g["b_fix"]
    hi_max = g["score_h"].shape[-1]

    for l in range(sh.n_layers):
        # ---- scorer on the ORACLE's summaries: tight comparison -------------
        slabs = orc.rki4_build_pages(t2n(cpu.kv_caches[l][:, 0]))
        _upload_slabs(st, l, slabs)
        q = torch.zeros(MR, H, sh.d, device=DEV, dtype=torch.bfloat16)
        q[:R] = case.q[l]
        st.score_h.fill_(float("nan"))
        rki4_score_only(st, l, q, case.block_table, case.seq_lens, R, case.scale)
        torch.cuda.synchronize()
        st.check_status()
        ref_sh = orc.rki4_score(slabs, t2n(cpu.q[l]), bt_np, nsh, case.scale,
                                sh.n_kv, sh.G, case.max_pages)
        got_sh = t2n(st.score_h[:R])
        for r in range(R):
            hi = max(int(nsh[r]), 0)
            np.testing.assert_allclose(got_sh[r, :, :, :hi], ref_sh[r, :, :, :hi],
                                       rtol=2e-4, atol=2e-4)
            # pages >= n_sel_hi are not written
            assert np.isnan(got_sh[r, :, :, hi:]).all()
        # and within the statistical band of the reference's own scores
        err = np.abs(np.nan_to_num(got_sh[..., :hi_max]) - g["score_h"][l])
        valid = np.arange(hi_max)[None, None, None, :] < nsh[:, None, None, None]
        assert (err[np.broadcast_to(valid, err.shape)] > 2e-4 + 2e-4 * 5).mean() <= 2e-2
        assert err[np.broadcast_to(valid, err.shape)].max() <= 5e-2

        # ---- combine + top-b --------------------------------------------------
        st.score_h[:R] = torch.from_numpy(ref_sh).to(DEV)
        st.score.zero_()
        rki4_select_only(st, R, has_hmax=False)
        torch.cuda.synchronize()
        ref_score = orc.nrm_combine(ref_sh, nsh) if c["combine"] == "nrm" \
            else orc.max_combine(ref_sh)
        got_score = t2n(st.score[:R])
        for r in range(R):
            hi = max(int(nsh[r]), 0)
            np.testing.assert_allclose(got_score[r, :, :hi], ref_score[r, :, :hi],
                                       rtol=1e-5, atol=1e-6)
        tab_o, cnt_o = orc.topb_select(ref_score, npg, nsh, b, sh.sink_pages)
        _assert_sets(t2n(st.page_table[:R]), t2n(st.page_cnt[:R]), tab_o, cnt_o,
                     ref_score, nsh, sh.sink_pages)
        # with the score kernel's published per-head maxima (hmax handshake)
        if c["combine"] == "nrm":
            st.hmax.zero_()
            rki4_score_only(st, l, q, case.block_table, case.seq_lens, R,
                            case.scale)
            rki4_select_only(st, R, has_hmax=True)
            torch.cuda.synchronize()
            assert int(st.hmax.abs().sum()) == 0          # reset after use
            _assert_sets(t2n(st.page_table[:R]), t2n(st.page_cnt[:R]), tab_o,
                         cnt_o, ref_score, nsh, sh.sink_pages)
        # top-b on the REFERENCE's combined score: bit-exact table
        st.score.zero_()
        st.score[:R, :, :hi_max] = torch.from_numpy(g["score"][l]).to(DEV)
        topb_select(st, R)
        torch.cuda.synchronize()
        cm = g["page_table"].shape[-1]
        np.testing.assert_array_equal(t2n(st.page_cnt[:R]), g["page_cnt"][l])
        tab = t2n(st.page_table[:R])
        np.testing.assert_array_equal(tab[..., :cm], g["page_table"][l])
        for r in range(R):
            for kh in range(sh.n_kv):
                assert (tab[r, kh, g["page_cnt"][l][r, kh]:] == -1).all()

        # ---- decode on the reference's page set -------------------------------
        out = torch.full((MR, H, sh.d), float("nan"), device=DEV,
                         dtype=torch.bfloat16)
        vs = ResidentVSource(case.kv_caches[l])
        sparse_paged_decode_batched(q[:R], case.kv_caches[l], case.block_table,
                                    case.seq_lens, st, out, vs, scale=case.scale)
        torch.cuda.synchronize()
        st.check_status()
        ref64, _ = orc.attention_over_pages(
            t2n(cpu.q[l]), t2n(cpu.kv_caches[l][:, 0]), t2n(cpu.kv_caches[l][:, 1]),
            bt_np, tab, g["page_cnt"][l], sl_np, case.scale, sh.n_kv, sh.G)
        got = t2n(out[:R])
        # tolerance stated for this path: 2e-2 max-abs, 1e-2 relative (bf16 out)
        np.testing.assert_allclose(got, ref64, atol=2e-2, rtol=1e-2)
        np.testing.assert_allclose(got, g["out"][l], atol=2e-2, rtol=1e-2)
        assert np.abs(got - ref64).max() <= 8e-3          # what bf16 output allows
        # split partials against the oracle's split restatement
        pps_min = _pps_min(R, sh.n_kv)
        m_o, l_o, a_o = orc.sparse_decode_split(
            t2n(cpu.q[l]), t2n(cpu.kv_caches[l][:, 0]), t2n(cpu.kv_caches[l][:, 1]),
            bt_np, tab, g["page_cnt"][l], sl_np, case.scale, sh.n_kv, sh.G,
            st.split, pps_min)
        o_o = orc.merge_splits(m_o, l_o, a_o, g["page_cnt"][l], st.split, pps_min)
        np.testing.assert_allclose(got, o_o, atol=2e-2, rtol=1e-2)
        # one-launch variant
        out2 = torch.full_like(out, float("nan"))
        sparse_paged_decode_fused(q[:R], case.kv_caches[l], case.block_table,
                                  case.seq_lens, st, out2, vs, scale=case.scale)
        torch.cuda.synchronize()
        np.testing.assert_allclose(t2n(out2[:R]), ref64, atol=2e-2, rtol=1e-2)
        # the same with the pages staged by tensor-map copies: same arithmetic
        # in the same order, so the rows are bit-equal
        out3 = torch.full_like(out, float("nan"))
        sparse_paged_decode_fused(q[:R], case.kv_caches[l], case.block_table,
                                  case.seq_lens, st, out3, vs, scale=case.scale,
                                  tma=True)
        torch.cuda.synchronize()
        st.check_status()
        assert torch.equal(out3[:R], out2[:R])


def _assert_sets(tab, cnt, tab_ref, cnt_ref, score_ref, nsh, sink, tol=1e-3):
    np.testing.assert_array_equal(cnt, cnt_ref)
    R, n_kv = cnt.shape
    for r in range(R):
        for kh in range(n_kv):
            a = tab[r, kh, :cnt[r, kh]]
            assert (np.diff(a) > 0).all()                 # ascending, unique
            sa, sb = set(a.tolist()), set(tab_ref[r, kh, :cnt_ref[r, kh]].tolist())
            if sa == sb:
                continue
            hi = int(nsh[r])
            tau = min(score_ref[r, kh, p] for p in sb if sink <= p < hi)
            for p in sa ^ sb:
                assert sink <= p < hi
                assert abs(score_ref[r, kh, p] - tau) <= tol * abs(tau)


def test_topb_known_answers_gpu():
    """Ties at the threshold, all-equal scores, +0 underflow, short rows."""
    from locks.selection import Rki4State, derive_page_params, topb_select
    g = load_golden("topb_kat")
    R, n_kv, MP = g["score"].shape
    st = Rki4State(DEV, num_layers=1, num_blocks=4, n_kv=n_kv, G=2,
                   head_dim=128, page=16, max_reqs=R, max_pages=MP,
                   budget_pages=12, sink_pages=2, window_pages=3)
    sl = torch.from_numpy(g["seq_lens"]).to(DEV)
    derive_page_params(st, sl, R)
    st.score.copy_(torch.from_numpy(g["score"]).to(DEV))
    topb_select(st, R)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(t2n(st.b_fix), g["b_fix"])
    np.testing.assert_array_equal(t2n(st.page_cnt), g["page_cnt"])
    np.testing.assert_array_equal(t2n(st.page_table), g["page_table"])
    st2 = Rki4State(DEV, num_layers=1, num_blocks=4, n_kv=n_kv, G=2,
                    head_dim=128, page=16, max_reqs=R, max_pages=MP,
                    budget=0.07, sink_pages=2, window_pages=3)
    derive_page_params(st2, sl, R)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(t2n(st2.b_fix), g["frac_b_fix"])
    np.testing.assert_array_equal(t2n(st2.n_sel_hi), g["frac_n_sel_hi"])


def test_padded_rows_and_dense_decode():
    """Padded request rows (seq_len 0) give zeros, never NaN; the dense
    baseline equals full attention."""
    from locks.attention import (DenseDecodeBuffers, ResidentVSource,
                                 dense_paged_decode,
                                 sparse_paged_decode_batched)
    from locks.selection import (derive_page_params, rki4_build_bulk,
                                 rki4_score_state)
    case, cpu, c = _gpu_case("gqa_ragged")
    sh = c["shape"]
    MR = c["max_reqs"]
    st = _state(case, c)
    R = case.n_req
    H = sh.n_kv * sh.G
    sl_pad = torch.zeros(MR, dtype=torch.int32, device=DEV)
    sl_pad[:R] = case.seq_lens
    bt_pad = torch.zeros(MR, case.max_pages, dtype=torch.int32, device=DEV)
    bt_pad[:R] = case.block_table
    K_layers = [kc[:, 0] for kc in case.kv_caches]
    rki4_build_bulk(st, K_layers, bt_pad, sl_pad - 1, MR,
                    int((t2n(case.seq_lens).max() - 1) // sh.page))
    derive_page_params(st, sl_pad, MR)
    q = torch.zeros(MR, H, sh.d, device=DEV, dtype=torch.bfloat16)
    q[:R] = case.q[0]
    rki4_score_state(st, 0, q, bt_pad, sl_pad, MR, case.scale)
    out = torch.full((MR, H, sh.d), float("nan"), device=DEV, dtype=torch.bfloat16)
    sparse_paged_decode_batched(q, case.kv_caches[0], bt_pad, sl_pad, st, out,
                                ResidentVSource(case.kv_caches[0]),
                                scale=case.scale)
    torch.cuda.synchronize()
    st.check_status()
    assert (t2n(st.page_cnt[R:]) == 0).all()
    o = t2n(out)
    assert np.isfinite(o).all() and (o[R:] == 0).all()
    # dense baseline
    buf = DenseDecodeBuffers(DEV, MR, sh.n_kv, sh.G, sh.d, 8)
    outd = torch.full_like(out, float("nan"))
    dense_paged_decode(q, case.kv_caches[0], bt_pad, sl_pad, buf, outd,
                       n_kv=sh.n_kv, G=sh.G, scale=case.scale, status=st.status)
    torch.cuda.synchronize()
    ref, _ = orc.dense_decode(t2n(cpu.q[0]), t2n(cpu.kv_caches[0][:, 0]),
                              t2n(cpu.kv_caches[0][:, 1]), t2n(cpu.block_table),
                              t2n(cpu.seq_lens), case.scale, sh.n_kv, sh.G)
    od = t2n(outd)
    np.testing.assert_allclose(od[:R], ref, atol=2e-2, rtol=1e-2)
    assert (od[R:] == 0).all()


@pytest.mark.parametrize("MP,combine", [(40000, "nrm"), (70001, "max"),
                                        (20000, "none")])
def test_topb_long_context(MP, combine):
    """Page counts beyond one CTA's shared memory: the selector spreads over a
    thread-block cluster; tables must equal the oracle's bit for bit (scores are
    coarse so that ties at the threshold are common)."""
    from locks.selection import (Rki4State, derive_page_params,
                                 rki4_select_only, topb_select)
    rng = np.random.default_rng(MP)
    n_kv, G, R = 2, 3, 2
    st = Rki4State(DEV, num_layers=1, num_blocks=4, n_kv=n_kv, G=G,
                   head_dim=128, page=16, max_reqs=R, max_pages=MP,
                   budget_pages=200, sink_pages=3, window_pages=5,
                   combine="max" if combine == "max" else "nrm")
    sl = np.array([MP * 16 - 7, (MP // 3) * 16 + 1], dtype=np.int32)
    derive_page_params(st, torch.from_numpy(sl).to(DEV), R)
    npg, nsh, b = orc.derive_page_params(sl, 16, 5, 3, 200)
    sh = (np.round(rng.standard_normal((R, n_kv, G, MP)) * 8) / 8).astype(np.float32)
    if combine == "none":
        score = (np.round(rng.random((R, n_kv, MP)) * 512) / 512).astype(np.float32)
        st.score.copy_(torch.from_numpy(score).to(DEV))
        topb_select(st, R)
    else:
        st.score_h.copy_(torch.from_numpy(sh).to(DEV))
        rki4_select_only(st, R, has_hmax=False)
        score = orc.nrm_combine(sh, nsh) if combine == "nrm" else orc.max_combine(sh)
    torch.cuda.synchronize()
    if combine == "nrm":
        # the device exp differs in the last bits: compare on the device score
        score = t2n(st.score)
    tab_o, cnt_o = orc.topb_select(score, npg, nsh, b, 3)
    np.testing.assert_array_equal(t2n(st.page_cnt), cnt_o)
    np.testing.assert_array_equal(t2n(st.page_table), tab_o)


@pytest.mark.parametrize("MP,kind,budget", [
    (65536, "equal", 128), (65536, "one_slice", 128), (40000, "coarse", 1),
    (131072, "coarse", 200), (20000, "equal", 500), (65536, "fine", 230)])
def test_topb_long_rows_small_budget(MP, kind, budget):
    """Long rows (kept as per-CTA slices) with a small page budget: all-equal
    scores (ties across slice borders: the lowest pages win), the best pages all
    in one slice, budget 1, a second row that fills only part of the slices;
    tables equal the oracle's bit for bit."""
    from locks.selection import Rki4State, derive_page_params, topb_select
    rng = np.random.default_rng(MP + budget)
    n_kv, R = 2, 2
    st = Rki4State(DEV, num_layers=1, num_blocks=4, n_kv=n_kv, G=1,
                   head_dim=128, page=16, max_reqs=R, max_pages=MP,
                   budget_pages=budget, sink_pages=2, window_pages=4,
                   combine="nrm")
    sl = np.array([MP * 16 - 3, (MP // 2 + 7) * 16], dtype=np.int32)
    derive_page_params(st, torch.from_numpy(sl).to(DEV), R)
    npg, nsh, b = orc.derive_page_params(sl, 16, 4, 2, budget)
    if kind == "equal":
        score = np.full((R, n_kv, MP), 0.25, np.float32)
    elif kind == "coarse":
        score = (np.round(rng.random((R, n_kv, MP)) * 64) / 64).astype(np.float32)
    elif kind == "one_slice":
        score = rng.random((R, n_kv, MP)).astype(np.float32)
        score[..., MP // 2 - 300:MP // 2 - 300 + 2 * budget] += 5.0
    else:
        score = rng.standard_normal((R, n_kv, MP)).astype(np.float32)
    st.score.copy_(torch.from_numpy(score).to(DEV))
    topb_select(st, R)
    torch.cuda.synchronize()
    tab_o, cnt_o = orc.topb_select(score, npg, nsh, b, 2)
    np.testing.assert_array_equal(t2n(st.page_cnt), cnt_o)
    np.testing.assert_array_equal(t2n(st.page_table), tab_o)


@pytest.mark.parametrize("MP,kind", [(40000, "equal"), (131072, "coarse"),
                                     (16385, "equal"), (65536, "fine"),
                                     (200000, "coarse")])
def test_topb_sliced_rows_ties_and_fraction_budget(MP, kind):
    """Rows kept as per-CTA slices: a 10 % budget (thousands of pages), all-equal
    scores (every page ties: the lowest pages win, across slice borders) and
    coarse scores; tables equal the oracle's bit for bit."""
    from locks.selection import Rki4State, derive_page_params, topb_select
    rng = np.random.default_rng(MP + 1)
    n_kv, R = 2, 2
    st = Rki4State(DEV, num_layers=1, num_blocks=4, n_kv=n_kv, G=1,
                   head_dim=128, page=16, max_reqs=R, max_pages=MP,
                   budget=0.1, sink_pages=2, window_pages=4, combine="nrm")
    sl = np.array([MP * 16 - 3, (MP // 2 + 7) * 16], dtype=np.int32)
    derive_page_params(st, torch.from_numpy(sl).to(DEV), R)
    npg, nsh, b = orc.derive_page_params(sl, 16, 4, 2, 0, 0.1)
    if kind == "equal":
        score = np.full((R, n_kv, MP), 0.25, np.float32)
    elif kind == "coarse":
        score = (np.round(rng.random((R, n_kv, MP)) * 64) / 64).astype(np.float32)
    else:
        score = rng.standard_normal((R, n_kv, MP)).astype(np.float32)
    st.score.copy_(torch.from_numpy(score).to(DEV))
    topb_select(st, R)
    torch.cuda.synchronize()
    tab_o, cnt_o = orc.topb_select(score, npg, nsh, b, 2)
    np.testing.assert_array_equal(t2n(st.page_cnt), cnt_o)
    np.testing.assert_array_equal(t2n(st.page_table), tab_o)
