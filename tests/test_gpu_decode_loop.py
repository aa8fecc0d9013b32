"""The append-and-attend step (``HotPath.append_step``): forty tokens are
appended to two ragged requests inside one replayed CUDA graph -- slot and
position update, page parameters, per layer KV write + score + select + decode,
summary build of completed pages on a forked branch -- and the state it leaves
is the state a fresh build over the final caches gives:

* the appended K (rotated) and V sit in the cache as the oracle's restatement
  of the write kernel says, bit for bit;
* every page completed on the way carries the summary a bulk build of the final
  cache produces, bit for bit, in every layer;
* the last step's selections and outputs equal those of a fresh driver that
  bulk-builds from the final caches and runs one step.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

import locks_oracle as orc
from conftest import t2n

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(extra, window_pages=2):
    from locks import synth
    shape = synth.GqaShape(n_layers=2, n_kv=2, G=4, budget_pages=6,
                           sink_pages=1, window_pages=window_pages, n_needles=2)
    lens = [100, 333]
    page = shape.page
    npg = [-(-s // page) for s in lens]
    NB = sum(npg) + extra * len(lens) + 2
    MP = max(npg) + extra
    cpu = synth.make_gqa_case(31, shape, lens, num_blocks=NB, max_pages=MP)
    bt = cpu.block_table.clone()
    used = set()
    for r, n in enumerate(npg):
        used |= set(bt[r, :n].tolist())
    free = [b for b in range(NB) if b not in used]
    for r, n in enumerate(npg):
        bt[r, n:n + extra] = torch.tensor(free[r * extra:(r + 1) * extra],
                                          dtype=torch.int32)
    return cpu, shape, bt, lens


@pytest.mark.parametrize("fuse_write,window_pages",
                         [(True, 2), (False, 2), (True, 1)])
def test_append_loop_leaves_the_state_of_a_fresh_build(fuse_write, window_pages):
    from locks.config import LocksConfig
    from locks.hotpath import HotPath
    steps, extra = 40, 3
    cpu, sh, bt_cpu, lens = _case(extra, window_pages)
    page, L, R = sh.page, sh.n_layers, len(lens)
    caches = [k.to(DEV) for k in cpu.kv_caches]
    bt = bt_cpu.to(DEV)
    sl = cpu.seq_lens.to(DEV).clone()
    cfg = LocksConfig(budget_pages=sh.budget_pages, sink_pages=sh.sink_pages,
                      window_pages=sh.window_pages)
    hp = HotPath(caches, bt, sl, n_kv=sh.n_kv, G=sh.G, scale=cpu.scale, cfg=cfg)
    hp.build_all()
    hp.derive()
    for l in range(L):
        hp.q[l, :R].copy_(cpu.q[l])
    g = torch.Generator().manual_seed(8)
    P = max(lens) + steps + 1
    ang = torch.rand(P, sh.d // 2, generator=g) * 6.28
    cs = torch.cat([ang.cos(), ang.sin()], 1).to(torch.bfloat16)
    hp.enable_append(cs.to(DEV), neox=True, fuse_write=fuse_write)
    new_k = torch.randn(steps, L, R, sh.n_kv, sh.d, generator=g).to(torch.bfloat16)
    new_v = torch.randn(steps, L, R, sh.n_kv, sh.d, generator=g).to(torch.bfloat16)
    n_checked = 0
    for s in range(steps):
        hp.new_k.copy_(new_k[s])
        hp.new_v.copy_(new_v[s])
        hp.append_step()
        # a one-page window scores the page the PREVIOUS step completed in this
        # very step: its summary must be in place before the first scorer.
        # Compare such steps with a fresh driver built from the caches as they are.
        if window_pages == 1 and s >= 1 and any(
                (n + s - 1) % page == page - 1 for n in lens):
            torch.cuda.synchronize()
            chk = HotPath(caches, bt, hp.seq_lens.clone(), n_kv=sh.n_kv, G=sh.G,
                          scale=cpu.scale, cfg=cfg)
            chk.build_all()
            chk.derive()
            for l in range(L):
                chk.q[l, :R].copy_(hp.q[l, :R])
            chk.step_eager()
            torch.cuda.synchronize()
            assert torch.equal(hp.st.page_cnt, chk.st.page_cnt), s
            assert torch.equal(hp.st.page_table, chk.st.page_table), s
            np.testing.assert_allclose(t2n(hp.out[:, :R]), t2n(chk.out[:, :R]),
                                       atol=2e-2, rtol=1e-2)
            n_checked += 1
    torch.cuda.synchronize()
    hp.st.check_status()
    assert window_pages != 1 or n_checked >= 2
    assert t2n(hp.seq_lens).tolist() == [n + steps for n in lens]
    out_loop = hp.out[:, :R].clone()
    tab_loop, cnt_loop = hp.st.page_table.clone(), hp.st.page_cnt.clone()

    # ---- (1) the appended tokens, against the oracle's write -----------------
    for l in range(L):
        for r in range(R):
            for s in (0, 7, steps - 1):
                tok = lens[r] + s
                blk = int(bt_cpu[r, tok // page])
                wk = np.zeros((blk + 1, page, sh.n_kv, sh.d), np.float32)
                wv = np.zeros_like(wk)
                orc.rope_and_cache(
                    new_k[s, l, r:r + 1].float().numpy(),
                    new_v[s, l, r:r + 1].float().numpy(), wk, wv,
                    np.array([blk * page + tok % page]), np.array([tok]),
                    cs.float().numpy(), sh.d, True, page)
                got = t2n(caches[l][blk, :, tok % page].float())
                assert np.array_equal(got[0], wk[blk, tok % page])
                assert np.array_equal(got[1], wv[blk, tok % page])

    # ---- (2) summaries of the pages completed on the way ---------------------
    hp.flush_builds()
    fresh = HotPath(caches, bt, hp.seq_lens.clone(), n_kv=sh.n_kv, G=sh.G,
                    scale=cpu.scale, cfg=cfg)
    fresh.build_all()
    fresh.derive()
    torch.cuda.synchronize()
    n_done = 0
    for r in range(R):
        final = lens[r] + steps
        for pg in range((final - 1) // page):
            blk = int(bt_cpu[r, pg])
            assert torch.equal(hp.st.pp_rec[:, blk], fresh.st.pp_rec[:, blk]), (r, pg)
            assert torch.equal(hp.st.pp_tag[:, blk].view(torch.int16),
                               fresh.st.pp_tag[:, blk].view(torch.int16)), (r, pg)
            n_done += pg >= lens[r] // page
    assert n_done >= 2 * (steps // page)

    # ---- (3) the last step, against a fresh driver on the final caches -------
    for l in range(L):
        fresh.q[l, :R].copy_(hp.q[l, :R])
    fresh.step_eager()
    torch.cuda.synchronize()
    fresh.st.check_status()
    assert torch.equal(cnt_loop, fresh.st.page_cnt)
    for r in range(R):
        for kh in range(sh.n_kv):
            n = int(cnt_loop[r, kh])
            assert sorted(tab_loop[r, kh, :n].tolist()) == \
                sorted(fresh.st.page_table[r, kh, :n].tolist())
    a, b = t2n(out_loop), t2n(fresh.out[:, :R])
    assert np.isfinite(a).all()
    # same kernels over the same bytes; the decode tolerance (2e-2 abs, 1e-2 rel)
    np.testing.assert_allclose(a, b, atol=2e-2, rtol=1e-2)


def test_step_host_equals_step():
    """``HotPath.step_host`` (host buffers in and out, copies inside the graph)
    returns what ``step`` leaves on the device, also after the host inputs
    change between replays."""
    from locks.config import LocksConfig
    from locks.hotpath import HotPath
    cpu, sh, bt_cpu, lens = _case(2)
    L, R = sh.n_layers, len(lens)
    caches = [k.to(DEV) for k in cpu.kv_caches]
    cfg = LocksConfig(budget_pages=sh.budget_pages, sink_pages=sh.sink_pages,
                      window_pages=sh.window_pages)
    hp = HotPath(caches, bt_cpu.to(DEV), cpu.seq_lens.to(DEV).clone(),
                 n_kv=sh.n_kv, G=sh.G, scale=cpu.scale, cfg=cfg)
    hp.build_all()
    hp.enable_host_io()
    hp.host_block_table.copy_(bt_cpu)
    g = torch.Generator().manual_seed(3)
    for trial, shorten in enumerate((0, 0, 33)):
        q = torch.randn(L, R, sh.n_kv * sh.G, sh.d, generator=g).to(torch.bfloat16)
        sl = cpu.seq_lens.clone()
        sl[1] -= shorten                     # the lengths travel with the step too
        hp.host_q.copy_(q)
        hp.host_seq_lens.copy_(sl)
        got = hp.step_host().clone()
        hp.st.check_status()
        # the same step through the device-side API
        hp.q[:, :R].copy_(q.to(DEV))
        hp.seq_lens.copy_(sl.to(DEV))
        hp.derive()
        want = hp.step_eager()[:, :R].cpu()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want), trial
