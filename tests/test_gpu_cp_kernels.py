"""Context-parallel glue kernels on ONE GPU: the ranks of a 4-way page split are
played one after the other (nothing waits on anything), and the union of their
final page tables must equal the single-sequence selector's / the oracle's."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import locks_oracle as orc
from conftest import t2n

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.mark.parametrize("kind", ["fine", "coarse", "equal"])
def test_pack_gather_select_equals_global_topb(kind):
    from locks import _cabi
    from locks.parallel import partition_pages
    from locks.selection import Rki4State, topb_select
    world, n_kv, page = 4, 2, 16
    seq_len = 9000 * page - 5
    sink, window, budget = 2, 6, 300
    npg = -(-seq_len // page)
    nsh = npg - window
    b = min(budget, nsh - sink)
    rng = np.random.default_rng(3)
    if kind == "fine":
        score = rng.standard_normal((n_kv, npg)).astype(np.float32)
    elif kind == "coarse":
        score = (np.round(rng.random((n_kv, npg)) * 32) / 32).astype(np.float32)
    else:
        score = np.full((n_kv, npg), 1.5, np.float32)
    # the answer: the single-sequence rule on the whole row
    tab_o, cnt_o = orc.topb_select(score[None], np.array([npg], np.int32),
                                   np.array([nsh], np.int32),
                                   np.array([b], np.int32), sink)
    parts = partition_pages(npg, world)
    cap = b + sink + window + 1
    cand_len = (2 * n_kv * cap + 3) // 4 * 4
    cand = torch.zeros(world, cand_len, device=DEV, dtype=torch.float32)
    states = []
    for r, (p0, p1) in enumerate(parts):
        n_loc = p1 - p0
        sink_loc = min(max(sink - p0, 0), n_loc)
        nsh_loc = min(max(nsh - p0, 0), n_loc)
        st = Rki4State(DEV, num_layers=1, num_blocks=4, n_kv=n_kv, G=1,
                       head_dim=128, page=page, max_reqs=1, max_pages=n_loc,
                       budget_pages=b, sink_pages=sink_loc, window_pages=window,
                       combine="nrm")
        st.n_pages.fill_(n_loc)
        st.n_sel_hi.fill_(nsh_loc)
        st.b_fix.fill_(b)
        st.score[0].copy_(torch.from_numpy(score[:, p0:p1]).to(DEV))
        topb_select(st, 1)                       # local top-b with the global b
        c = min(cap, n_loc)
        assert c == cap, "test sized so that every rank can hold cap entries"
        _cabi.call("locks_cp_pack", _cabi.ptr(st.page_table), _cabi.ptr(st.score),
                   _cabi.ptr(cand[r]), n_kv, n_loc, cap, sink_loc, nsh_loc, p0,
                   _cabi.stream())
        states.append((st, p0, n_loc, sink_loc, nsh_loc))
    got = [[] for _ in range(n_kv)]
    for r, (st, p0, n_loc, sink_loc, nsh_loc) in enumerate(states):
        _cabi.call("locks_cp_select", _cabi.ptr(cand), cand_len,
                   _cabi.ptr(st.page_table), _cabi.ptr(st.page_cnt), world, r,
                   n_kv, cap, n_loc, b, sink_loc, nsh_loc, _cabi.stream())
        torch.cuda.synchronize()
        cnt = t2n(st.page_cnt)[0]
        tab = t2n(st.page_table)[0]
        for kh in range(n_kv):
            mine = tab[kh, :cnt[kh]]
            assert (np.diff(mine) > 0).all()             # ascending, no repeats
            assert (tab[kh, cnt[kh]:cap] == -1).all()
            got[kh] += (mine + p0).tolist()
    for kh in range(n_kv):
        want = tab_o[0, kh, :cnt_o[0, kh]].tolist()
        assert got[kh] == want


def test_merge_gathered_equals_merge_of_all_partials():
    """locks_merge_gathered over 3 partial sets = the log-sum-exp merge of all
    their splits; empty splits (l = 0) carry garbage m / acc and are ignored."""
    from locks import _cabi
    n_groups, n_kv, G, split, d = 3, 2, 16, 4, 128
    g = torch.Generator().manual_seed(8)
    n_ml = n_kv * split * G
    pack_len = (n_ml * (2 + d) + 3) // 4 * 4
    packs = torch.zeros(n_groups, pack_len)
    m = torch.randn(n_groups, n_kv, split, G, generator=g) * 3
    l = torch.rand(n_groups, n_kv, split, G, generator=g) + 0.1
    acc = torch.randn(n_groups, n_kv, split, G, d, generator=g)
    l[0, :, 1] = 0.0                                   # empty splits
    l[2, 1, :, 3] = 0.0
    m[0, :, 1] = float("nan")
    acc[0, :, 1] = float("inf")
    for k in range(n_groups):
        packs[k, :n_ml] = m[k].reshape(-1)
        packs[k, n_ml:2 * n_ml] = l[k].reshape(-1)
        packs[k, 2 * n_ml:2 * n_ml + n_ml * d] = acc[k].reshape(-1)
    out = torch.zeros(1, n_kv * G, d, dtype=torch.bfloat16, device=DEV)
    dp = packs.to(DEV)
    _cabi.call("locks_merge_gathered", _cabi.ptr(dp), pack_len, n_groups,
               _cabi.ptr(out), out.stride(0), 1, n_kv, G, d, split, _cabi.stream())
    torch.cuda.synchronize()
    mm = m.permute(1, 3, 0, 2).reshape(n_kv, G, -1).double()
    ll = l.permute(1, 3, 0, 2).reshape(n_kv, G, -1).double()
    aa = acc.permute(1, 3, 0, 2, 4).reshape(n_kv, G, -1, d).double()
    live = ll > 0
    mm = torch.where(live, mm, torch.full_like(mm, -1e30))
    aa = torch.where(live[..., None], aa, torch.zeros_like(aa))
    M = mm.max(-1, keepdim=True).values
    w = torch.where(live, torch.exp(mm - M), torch.zeros_like(mm))
    want = (w[..., None] * aa).sum(2) / (w * ll).sum(-1, keepdim=True)
    np.testing.assert_allclose(out[0].float().cpu().numpy().reshape(n_kv, G, d),
                               want.float().numpy(), atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("mode", [0, 2])
def test_exchange_wait_runs_out_and_reports(mode):
    """A peer that never shows up: the exchange kernel gives up after its time
    limit, raises the status word and returns -- nothing hangs and the context
    stays usable.  (Rank 1 is a second region on the same GPU that no kernel
    ever writes flags into.)"""
    import ctypes
    from locks import _cabi
    slot = 4096
    nb = ctypes.c_int64()
    _cabi.call("locks_cp_region_bytes", slot, ctypes.byref(nb))
    r0, r1 = ctypes.c_void_p(), ctypes.c_void_p()
    _cabi.call("locks_cp_alloc", int(nb.value), ctypes.byref(r0))
    _cabi.call("locks_cp_alloc", int(nb.value), ctypes.byref(r1))
    peers = (ctypes.c_void_p * 8)()
    peers[0], peers[1] = r0.value, r1.value
    payload = torch.arange(64, device=DEV, dtype=torch.int32)
    out = torch.zeros(2, 64, device=DEV, dtype=torch.int32)
    status = torch.zeros(1, device=DEV, dtype=torch.int32)
    try:
        _cabi.call("locks_cp_exchange", peers, 2, 0, _cabi.ptr(payload), 256, slot,
                   _cabi.ptr(out), mode, _cabi.ptr(status), _cabi.stream())
        torch.cuda.synchronize()                     # returns after ~2 s
        assert int(status.item()) == 1               # LOCKS_ST_WAIT_TIMEOUT
        # the context is alive: a normal single-rank exchange works afterwards
        status.zero_()
        peers1 = (ctypes.c_void_p * 8)()
        peers1[0] = r0.value
        out1 = torch.zeros(1, 64, device=DEV, dtype=torch.int32)
        _cabi.call("locks_cp_exchange", peers1, 1, 0, _cabi.ptr(payload), 256, slot,
                   _cabi.ptr(out1), mode, _cabi.ptr(status), _cabi.stream())
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(out1[0], payload)
    finally:
        _cabi.call("locks_cp_free", r0)
        _cabi.call("locks_cp_free", r1)


def _single_rank_pair(seq_len, seed=11, n_layers=3):
    """The same seeded sequence through the single-GPU driver and through the
    context-parallel driver with ONE rank (the in-kernel exchanges then run
    against the rank's own link region: same code path, no peer)."""
    import math
    from locks import LocksConfig, synth
    from locks.cp_hotpath import ContextParallelHotPath
    from locks.hotpath import HotPath
    shape = synth.GqaShape(n_layers=n_layers, n_kv=2, G=16, d=128, page=16,
                           budget_pages=64, sink_pages=1, window_pages=8,
                           n_needles=6, n_outlier=4)
    cfg = LocksConfig(budget_pages=shape.budget_pages, sink_pages=shape.sink_pages,
                      window_pages=shape.window_pages)
    scale = 1.0 / math.sqrt(shape.d)
    npg = -(-seq_len // shape.page)
    caches, q, bt = synth.make_gqa_shard(seed, shape, seq_len, 0, npg, device=DEV)
    sl = torch.tensor([seq_len], dtype=torch.int32, device=DEV)
    hp = HotPath(caches, bt, sl, n_kv=shape.n_kv, G=shape.G, scale=scale, cfg=cfg)
    hp.build_all(); hp.derive(); hp.q.copy_(q)
    cp = ContextParallelHotPath(caches, bt, seq_len=seq_len, p0=0, p1=npg,
                                n_kv=shape.n_kv, G=shape.G, scale=scale, cfg=cfg,
                                transport="fused", loopback=True)
    cp.st.pp_rec.copy_(hp.st.pp_rec)
    cp.q.copy_(q)
    return hp, cp, shape


@pytest.mark.parametrize("seq_len", [4099, 40005, 300])
def test_fused_context_parallel_single_rank_equals_hot_path(seq_len):
    """Selector with the maxima exchange and the global cut inside, decode with
    the partial exchange and merge inside, against the plain kernels: the same
    page tables bit for bit and the same outputs; replayed as a graph several
    times (every replay is a new step with new exchange epochs)."""
    hp, cp, shape = _single_rank_pair(seq_len)
    ref = hp.step_eager().clone()
    torch.cuda.synchronize()
    tab_ref, cnt_ref = hp.st.page_table.clone(), hp.st.page_cnt.clone()
    got = cp.step_eager().clone()
    torch.cuda.synchronize()
    cp.st.check_status()
    assert torch.equal(cp.st.page_cnt, cnt_ref)
    assert torch.equal(cp.st.page_table, tab_ref)
    np.testing.assert_allclose(t2n(got), t2n(ref), atol=2e-2, rtol=1e-2)
    for _ in range(3):
        out = cp.step().clone()
    torch.cuda.synchronize()
    cp.st.check_status()
    assert torch.equal(out, got)
    assert torch.equal(cp.st.page_table, tab_ref)


def test_fused_context_parallel_wait_runs_out_and_reports():
    """A peer that never shows up, for the in-kernel exchanges: the link claims
    two ranks, rank 1's region is a second allocation on this GPU that nothing
    writes.  Selector and decode give up after their time limit, raise the
    status word and return; after ``resync`` a normal step works again."""
    import ctypes
    from locks import _cabi
    hp, cp, shape = _single_rank_pair(4099, n_layers=1)
    want = cp.step_eager().clone()
    torch.cuda.synchronize()
    cp.st.check_status()
    ghost = ctypes.c_void_p()
    _cabi.call("locks_cp_alloc", cp.link.nbytes, ctypes.byref(ghost))
    try:
        for d in cp._links:
            d.world = 2
            d.regions[1] = ghost.value
        cp.step_eager()
        torch.cuda.synchronize()                     # returns after a few seconds
        assert int(cp.st.status.item()) == 1         # LOCKS_ST_WAIT_TIMEOUT
        for d in cp._links:
            d.world = 1
            d.regions[1] = None
        cp.resync()
        got = cp.step_eager().clone()
        torch.cuda.synchronize()
        cp.st.check_status()
        assert torch.equal(got, want)
    finally:
        _cabi.call("locks_cp_free", ghost)
