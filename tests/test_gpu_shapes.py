"""Parity at the other benchmark shapes and size-independent properties at the
full benchmark sizes (where the CPU oracle would take minutes)."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import locks_oracle as orc
from conftest import t2n

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _hot(case, shape, max_reqs=None):
    from locks import LocksConfig
    from locks.hotpath import HotPath
    cfg = LocksConfig(budget_pages=shape.budget_pages, sink_pages=shape.sink_pages,
                      window_pages=shape.window_pages)
    hp = HotPath([c.to(DEV) for c in case.kv_caches], case.block_table.to(DEV),
                 case.seq_lens.to(DEV), n_kv=shape.n_kv, G=shape.G, scale=case.scale,
                 cfg=cfg, max_reqs=max_reqs)
    hp.build_all()
    hp.derive()
    hp.q[:, :case.n_req].copy_(case.q.to(DEV))
    return hp


def test_g16_group_matches_oracle():
    """32 query heads on 2 KV heads (G = 16, the 1M-context config as written;
    beyond the reference's own G <= 8 limit, so the oracle is the only check)."""
    from locks import synth
    shape = synth.GqaShape(n_layers=1, n_kv=2, G=16, budget_pages=16,
                           sink_pages=1, window_pages=3, n_needles=4)
    cpu = synth.make_gqa_case(11, shape, [2500, 900], device="cpu")
    hp = _hot(cpu, shape)
    out = t2n(hp.step()[0])
    torch.cuda.synchronize()
    hp.st.check_status()
    f = lambda t: t.float().numpy()
    slabs = {k: t2n(v) for k, v in zip(("v4", "vs", "c8", "cs", "mu8", "mus", "tag"),
                                       hp.st.layer_state(0))}
    ref = orc.gqa_decode_step(
        slabs, f(cpu.q[0]), f(cpu.kv_caches[0][:, 0]), f(cpu.kv_caches[0][:, 1]),
        cpu.block_table.numpy(), cpu.seq_lens.numpy(), cpu.scale, n_kv=2, G=16,
        page=16, window=3, sink=1, budget_pages=16, split=8)
    nsh = ref["n_sel_hi"]
    got_sh = t2n(hp.st.score_h)
    for r in range(2):
        np.testing.assert_allclose(got_sh[r, :, :, :nsh[r]],
                                   ref["score_h"][r, :, :, :nsh[r]], rtol=2e-4, atol=2e-4)
    np.testing.assert_array_equal(t2n(hp.st.page_cnt), ref["page_cnt"])
    tab, tab_ref = t2n(hp.st.page_table), ref["page_table"]
    for r in range(2):
        for kh in range(2):
            a = set(tab[r, kh, :ref["page_cnt"][r, kh]].tolist())
            b = set(tab_ref[r, kh, :ref["page_cnt"][r, kh]].tolist())
            if a != b:             # only pages tied with the threshold (1e-3)
                sel = [p for p in b if 1 <= p < nsh[r]]
                tau = min(ref["score"][r, kh, p] for p in sel)
                assert all(abs(ref["score"][r, kh, p] - tau) <= 1e-3 * abs(tau)
                           for p in a ^ b)
    # decode tolerance of the path: 2e-2 max-abs, 1e-2 relative
    ref64, _ = orc.attention_over_pages(
        f(cpu.q[0]), f(cpu.kv_caches[0][:, 0]), f(cpu.kv_caches[0][:, 1]),
        cpu.block_table.numpy(), tab, t2n(hp.st.page_cnt), cpu.seq_lens.numpy(),
        cpu.scale, 2, 16)
    np.testing.assert_allclose(out, ref64, atol=2e-2, rtol=1e-2)


def _expected_tables(score, n_sel_hi, n_pages, b, sink):
    """Independent device-side statement of the keep rule for ONE row: top-b by
    (score desc, page asc) over [sink, n_sel_hi) + forced pages."""
    n_kv = score.shape[0]
    sel = score[:, sink:n_sel_hi]
    order = torch.sort(sel, dim=1, descending=True, stable=True).indices[:, :b] + sink
    out = []
    forced = list(range(sink)) + list(range(n_sel_hi, n_pages))
    for kh in range(n_kv):
        out.append(sorted(order[kh].tolist() + forced))
    return out


@pytest.mark.parametrize("cfgname", ["c1", "c4"])
def test_full_size_properties(cfgname):
    """One layer at the full benchmark context (131072 tokens, 8 KV heads, G 4;
    1048576 tokens, 2 KV heads, G 16): counts, order, exact top-b against a
    torch sort of the device scores, needle recall, sparse ~ dense attention,
    build idempotence."""
    import dataclasses
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    from locks import LocksConfig, synth
    from locks.attention import DenseDecodeBuffers, dense_paged_decode
    from locks.hotpath import HotPath
    sh, ctx = bench.workload(cfgname, None)
    sh = dataclasses.replace(sh, n_layers=1)
    seq_len = ctx + 1
    dev = torch.device("cuda", 0)
    caches, q, bt, sl, needles = bench.make_device_case(sh, seq_len, dev, seed=77,
                                                        return_needles=True)
    cfg = LocksConfig(budget_pages=sh.budget_pages, sink_pages=sh.sink_pages,
                      window_pages=sh.window_pages)
    hp = HotPath(caches, bt, sl, n_kv=sh.n_kv, G=sh.G, scale=1 / math.sqrt(sh.d), cfg=cfg)
    hp.build_all()
    rec1 = hp.st.pp_rec.clone()
    hp.build_all()                                   # idempotent: same bytes
    assert torch.equal(rec1, hp.st.pp_rec)
    del rec1
    hp.derive()
    hp.q.copy_(q)
    out = hp.step()[0, 0].float()
    torch.cuda.synchronize()
    hp.st.check_status()
    st = hp.st
    npg = -(-seq_len // sh.page)
    nsh = npg - sh.window_pages
    A = sh.budget_pages + sh.sink_pages + sh.window_pages
    assert int(st.n_pages[0]) == npg and int(st.n_sel_hi[0]) == nsh
    assert (st.page_cnt[0] == A).all()
    tab = st.page_table[0]
    assert (tab[:, A:] == -1).all()
    assert (tab[:, 1:A] > tab[:, :A - 1]).all()                 # ascending
    assert torch.isfinite(st.score_h[0, :, :, :nsh]).all()
    want = _expected_tables(st.score[0], nsh, npg, sh.budget_pages, sh.sink_pages)
    for kh in range(sh.n_kv):
        assert tab[kh, :A].tolist() == want[kh], kh
    # every planted needle page is selected
    for kh in range(sh.n_kv):
        assert set(needles[0][kh].tolist()) <= set(tab[kh, :A].tolist())
    # decode against a plain torch fp32 attention over the same selected pages
    kvc = caches[0]
    ref = torch.empty(sh.n_kv * sh.G, sh.d, device=dev)
    for kh in range(sh.n_kv):
        blks = bt[0, tab[kh, :A].long()].long()
        K = kvc[blks, 0, :, kh].reshape(-1, sh.d).float()
        V = kvc[blks, 1, :, kh].reshape(-1, sh.d).float()
        pos = (tab[kh, :A].long()[:, None] * sh.page
               + torch.arange(sh.page, device=dev)[None]).reshape(-1)
        s_ = (hp.q[0, 0, kh * sh.G:(kh + 1) * sh.G].float() @ K.T) * hp.scale
        s_ = s_.masked_fill(~(pos < seq_len)[None], float("-inf"))
        ref[kh * sh.G:(kh + 1) * sh.G] = torch.softmax(s_, -1) @ V
    # tolerance of the path: 2e-2 max-abs, 1e-2 relative
    torch.testing.assert_close(out, ref, atol=2e-2, rtol=1e-2)
    # dense baseline kernel against torch on a slice of heads (full KV)
    buf = DenseDecodeBuffers(dev, 1, sh.n_kv, sh.G, sh.d, 64)
    dense = torch.empty_like(hp.out[0])
    dense_paged_decode(hp.q[0], caches[0], bt, sl, buf, dense, n_kv=sh.n_kv,
                       G=sh.G, scale=hp.scale, status=st.status)
    torch.cuda.synchronize()
    st.check_status()
    kh = sh.n_kv - 1
    blks = bt[0, :npg].long()
    K = kvc[blks, 0, :, kh].reshape(-1, sh.d)[:seq_len].float()
    V = kvc[blks, 1, :, kh].reshape(-1, sh.d)[:seq_len].float()
    s_ = (hp.q[0, 0, kh * sh.G:(kh + 1) * sh.G].float() @ K.T) * hp.scale
    dref = torch.softmax(s_, -1) @ V
    torch.testing.assert_close(dense[0, kh * sh.G:(kh + 1) * sh.G].float(), dref,
                               atol=2e-2, rtol=1e-2)
    if cfgname == "c1":
        # on this data the planted pages carry almost all of the softmax mass,
        # so sparse and dense attention agree
        assert (out - dense[0].float()).abs().max().item() <= 5e-2


def test_decode_reads_v_from_pinned_host_memory():
    """V kept in pinned host memory (read in place over the host link) gives the
    same output as V resident next to K, for the fused and the split decode."""
    import math
    from locks import LocksConfig, synth
    from locks.attention import (PinnedHostVSource, sparse_paged_decode_batched,
                                 sparse_paged_decode_fused)
    from locks.hotpath import HotPath
    sh = synth.GqaShape(n_layers=1, n_kv=8, G=4, d=128, page=16, budget_pages=32,
                        sink_pages=1, window_pages=4, n_needles=4, n_outlier=4)
    case = synth.make_gqa_case(5, sh, [3000, 517], device="cuda")
    cfg = LocksConfig(budget_pages=32, sink_pages=1, window_pages=4)
    hp = HotPath(case.kv_caches, case.block_table, case.seq_lens, n_kv=8, G=4,
                 scale=1 / math.sqrt(128), cfg=cfg)
    hp.build_all(); hp.derive(); hp.q.copy_(case.q)
    ref = hp.step_eager()[0].clone()                 # resident V, fused decode
    host_v = PinnedHostVSource(case.kv_caches[0])
    assert not host_v.plane.is_cuda and host_v.plane.is_pinned()
    # wipe the resident V half: the kernels must not be reading it
    case.kv_caches[0][:, 1].zero_()
    out = torch.zeros_like(ref)
    sparse_paged_decode_fused(hp.q[0, :2], case.kv_caches[0], case.block_table,
                              case.seq_lens, hp.st, out, host_v, scale=hp.scale)
    torch.cuda.synchronize()
    assert torch.equal(out[:2], ref[:2])
    out2 = torch.zeros_like(ref)
    sparse_paged_decode_batched(hp.q[0, :2], case.kv_caches[0], case.block_table,
                                case.seq_lens, hp.st, out2, host_v, scale=hp.scale)
    torch.cuda.synchronize()
    assert (out2[:2].float() - ref[:2].float()).abs().max().item() <= 2e-2


def test_fused_decode_with_tensor_map_copies_ignores_stale_rows():
    """The tensor-map variant copies whole 16-row pages; rows past the sequence
    end (here filled with NaN and huge values) must not reach the output.  G = 4
    and G = 16, ragged lengths with partial last pages, against the cp.async
    variant (bit-equal) and the fp64 oracle."""
    from locks import LocksConfig, synth
    from locks.attention import ResidentVSource, sparse_paged_decode_fused
    from locks.hotpath import HotPath
    for n_kv, G in ((8, 4), (2, 16)):
        sh = synth.GqaShape(n_layers=1, n_kv=n_kv, G=G, d=128, page=16,
                            budget_pages=24, sink_pages=1, window_pages=3,
                            n_needles=4, n_outlier=4)
        lens = [3001, 517, 16 * 40, 33]
        case = synth.make_gqa_case(21, sh, lens, device="cuda")
        cache = case.kv_caches[0]
        bt = case.block_table.cpu().numpy()
        for r, n in enumerate(lens):          # poison the tail of the last page
            if n % 16:
                blk = int(bt[r, n // 16])
                cache[blk, 0, n % 16:] = float("nan")
                cache[blk, 1, n % 16:] = float("inf")
        cfg = LocksConfig(budget_pages=24, sink_pages=1, window_pages=3)
        hp = HotPath(case.kv_caches, case.block_table, case.seq_lens, n_kv=n_kv,
                     G=G, scale=1 / math.sqrt(128), cfg=cfg)
        hp.build_all(); hp.derive(); hp.q.copy_(case.q)
        ref = hp.step_eager()[0].clone()              # cp.async staging
        R = len(lens)
        out = torch.full_like(ref, float("nan"))
        sparse_paged_decode_fused(hp.q[0, :R], cache, case.block_table,
                                  case.seq_lens, hp.st, out,
                                  ResidentVSource(cache), scale=hp.scale, tma=True)
        torch.cuda.synchronize()
        hp.st.check_status()
        assert torch.isfinite(out[:R].float()).all()
        assert torch.equal(out[:R], ref[:R])
        c = cache.float().cpu().numpy()
        ref64, _ = orc.attention_over_pages(
            hp.q[0, :R].float().cpu().numpy(), c[:, 0], c[:, 1], bt,
            hp.st.page_table[:R].cpu().numpy(), hp.st.page_cnt[:R].cpu().numpy(),
            case.seq_lens.cpu().numpy(), hp.scale, n_kv, G)
        np.testing.assert_allclose(out[:R].float().cpu().numpy(), ref64,
                                   atol=2e-2, rtol=1e-2)


def test_large_batch_rows_launched_longest_first_give_the_same_result():
    """More (request, kv-head) rows than resident CTAs: the selector and the
    decode handle the rows longest first (``locks_row_order``).  The orders are
    permutations sorted as documented, and tables and outputs equal those of the
    grid-order launch bit for bit."""
    from locks import LocksConfig, synth
    from locks.hotpath import HotPath
    sh = synth.GqaShape(n_layers=1, n_kv=8, G=4, d=128, page=16, budget_pages=16,
                        sink_pages=1, window_pages=2, n_needles=2, n_outlier=2)
    rng = np.random.default_rng(3)
    lens = [int(x) for x in rng.integers(40, 2500, size=40)]
    budgets = [int(x) for x in rng.choice([4, 8, 16, 32], size=40)]
    case = synth.make_gqa_case(17, sh, lens, device="cuda")
    cfg = LocksConfig(budget_pages=32, sink_pages=1, window_pages=2)
    hp = HotPath(case.kv_caches, case.block_table, case.seq_lens, n_kv=8, G=4,
                 scale=1 / math.sqrt(128), cfg=cfg, budget_pages_req=budgets)
    hp.build_all(); hp.derive(); hp.q.copy_(case.q)
    st, R = hp.st, len(lens)
    assert st.row_order_n == R
    torch.cuda.synchronize()
    npg, nsh, b = (t2n(x[:R]) for x in (st.n_pages, st.n_sel_hi, st.b_fix))
    o_sel, o_dec = t2n(st.order_sel[:R]), t2n(st.order_dec[:R])
    assert sorted(o_sel.tolist()) == list(range(R)) == sorted(o_dec.tolist())
    assert (np.diff(nsh[o_sel]) <= 0).all()
    att = np.minimum(b, np.maximum(nsh - 1, 0)) + (npg - nsh)
    assert (np.diff(att[o_dec]) <= 0).all()
    out_a = hp.step_eager()[0].clone()
    tab_a, cnt_a = st.page_table[:R].clone(), st.page_cnt[:R].clone()
    st.row_order_n = 0                               # grid order
    out_b = hp.step_eager()[0].clone()
    torch.cuda.synchronize()
    assert torch.equal(tab_a, st.page_table[:R]) and torch.equal(cnt_a, st.page_cnt[:R])
    assert torch.equal(out_a[:R], out_b[:R])


def test_ragged_batch_scores_equal_single_request_scores():
    """The scorer deals the CTAs of a kv-head to the requests of a batch by
    length; whatever the split, a request's scores must be bit-identical to the
    ones it gets when it is scored alone."""
    from locks import synth
    from locks.selection import Rki4State, derive_page_params, rki4_build_bulk, \
        rki4_score_only
    sh = synth.GqaShape(n_layers=1, n_kv=8, G=4, d=128, page=16, budget_pages=32,
                        sink_pages=1, window_pages=4, n_needles=0, n_outlier=4)
    lens = [40, 5000, 300, 70001, 129, 16 * 700]
    case = synth.make_gqa_case(9, sh, lens, device=DEV)
    R, MP, NB = len(lens), int(case.block_table.shape[1]), int(case.kv_caches[0].shape[0])

    def state(n):
        st = Rki4State(DEV, num_layers=1, num_blocks=NB, n_kv=8, G=4, head_dim=128,
                       page=16, max_reqs=n, max_pages=MP, budget_pages=32,
                       sink_pages=1, window_pages=4)
        st.scale = case.scale
        return st
    st = state(R)
    K = [case.kv_caches[0][:, 0]]
    rki4_build_bulk(st, K, case.block_table, case.seq_lens - 1, R, MP)
    derive_page_params(st, case.seq_lens, R)
    rki4_score_only(st, 0, case.q[0], case.block_table, case.seq_lens, R, case.scale)
    torch.cuda.synchronize()
    batch = st.score_h.clone()
    nsh = t2n(st.n_sel_hi)
    for r in range(R):
        one = state(1)
        one.pp_rec.copy_(st.pp_rec)
        sl = case.seq_lens[r:r + 1].contiguous()
        bt = case.block_table[r:r + 1].contiguous()
        derive_page_params(one, sl, 1)
        rki4_score_only(one, 0, case.q[0, r:r + 1].contiguous(), bt, sl, 1, case.scale)
        torch.cuda.synchronize()
        n = max(int(nsh[r]), 0)
        assert torch.equal(one.score_h[0, :, :, :n], batch[r, :, :, :n]), r
        # the published per-head maxima agree as well
        assert torch.equal(one.hmax[0], st.hmax[r]), r


def test_ragged_batch_with_per_request_budgets_matches_oracle():
    """A continuous batch whose requests carry their own page budgets (the
    ragged-batch benchmark draws them from {32, 64, 128, 256}): page
    parameters, selected sets and outputs of every request against the oracle
    run with the same per-request budgets.  One request is shorter than its
    budget (keeps every page), one uses the fractional fallback (entry 0)."""
    from locks import LocksConfig, synth
    from locks.hotpath import HotPath
    shape = synth.GqaShape(n_layers=1, n_kv=4, G=4, budget_pages=64,
                           sink_pages=1, window_pages=2, n_needles=3)
    lens = [3000, 700, 5200, 260, 1900]
    budgets = [32, 64, 128, 256, 0]
    cpu = synth.make_gqa_case(23, shape, lens, device="cpu")
    cfg = LocksConfig(budget_pages=shape.budget_pages, sink_pages=1, window_pages=2)
    hp = HotPath([c.to(DEV) for c in cpu.kv_caches], cpu.block_table.to(DEV),
                 cpu.seq_lens.to(DEV), n_kv=shape.n_kv, G=shape.G, scale=cpu.scale,
                 cfg=cfg, budget_pages_req=budgets)
    hp.build_all()
    hp.derive()
    hp.q[:, :cpu.n_req].copy_(cpu.q.to(DEV))
    out = t2n(hp.step()[0])
    torch.cuda.synchronize()
    hp.st.check_status()
    f = lambda t: t.float().numpy()
    slabs = {k: t2n(v) for k, v in zip(("v4", "vs", "c8", "cs", "mu8", "mus", "tag"),
                                       hp.st.layer_state(0))}
    ref = orc.gqa_decode_step(
        slabs, f(cpu.q[0]), f(cpu.kv_caches[0][:, 0]), f(cpu.kv_caches[0][:, 1]),
        cpu.block_table.numpy(), cpu.seq_lens.numpy(), cpu.scale, n_kv=shape.n_kv,
        G=shape.G, page=16, window=2, sink=1, budget_pages=np.array(budgets),
        budget=hp.st.budget, split=8)
    R = len(lens)
    np.testing.assert_array_equal(t2n(hp.st.n_pages)[:R], ref["n_pages"])
    np.testing.assert_array_equal(t2n(hp.st.n_sel_hi)[:R], ref["n_sel_hi"])
    np.testing.assert_array_equal(t2n(hp.st.b_fix)[:R], ref["b"])
    # 700 tokens hold 41 selectable pages (< 64), 260 tokens 14 (< 256); the
    # last request falls back to ceil(0.1 * 116)
    assert ref["b"].tolist() == [32, 41, 128, 14, 12]
    np.testing.assert_array_equal(t2n(hp.st.page_cnt)[:R], ref["page_cnt"])
    nsh = ref["n_sel_hi"]
    tab, tab_ref = t2n(hp.st.page_table), ref["page_table"]
    for r in range(R):
        for kh in range(shape.n_kv):
            n = ref["page_cnt"][r, kh]
            a, b = set(tab[r, kh, :n].tolist()), set(tab_ref[r, kh, :n].tolist())
            if a != b:             # only pages tied with the threshold (1e-3)
                sel = [p for p in b if 1 <= p < nsh[r]]
                tau = min(ref["score"][r, kh, p] for p in sel)
                assert all(abs(ref["score"][r, kh, p] - tau) <= 1e-3 * abs(tau)
                           for p in a ^ b)
    ref64, _ = orc.attention_over_pages(
        f(cpu.q[0]), f(cpu.kv_caches[0][:, 0]), f(cpu.kv_caches[0][:, 1]),
        cpu.block_table.numpy(), tab, t2n(hp.st.page_cnt), cpu.seq_lens.numpy(),
        cpu.scale, shape.n_kv, shape.G)
    np.testing.assert_allclose(out[:R], ref64, atol=2e-2, rtol=1e-2)
