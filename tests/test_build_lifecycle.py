"""Which blocks get (re)built, and when: the scripted summary life cycle of
``tests/golden/lifecycle_script.py`` -- first decode, a request arriving, a
block reused with new content, steady tail steps, a preempted-and-resumed row,
a finished request's blocks handed to a new one, single-layer refresh, a padded
row with block ids outside the pool -- played through

* the oracle's block rules (CPU), which pins ``tail_blocks`` / ``delta_blocks``
  / ``refresh_blocks`` / ``bulk_blocks`` to the reference, and
* this library's ``rki4_build_{bulk,tail,delta,refresh}`` and the
  ``locks_rki4_tag_scan`` kernel (GPU, through the C ABI),

each compared event by event with ``tests/golden/gqa_lifecycle.npz``, the record
of the same script played through the reference's own functions.
"""
from __future__ import annotations

import importlib.util
import os

import numpy as np
import pytest
import torch

import locks_oracle as orc
from conftest import GOLDEN, load_golden, t2n


def _script():
    spec = importlib.util.spec_from_file_location(
        "lifecycle_script", os.path.join(GOLDEN, "lifecycle_script.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _check_events(ev, g):
    assert [e[0] for e in ev] == g["kind"].tolist()
    for i, (kind, ret, stale) in enumerate(ev):
        if stale is not None:
            # same blocks in the same (request-major, page-ascending) order
            assert list(stale) == g[f"stale{i}"].tolist(), (i, kind)
        if kind != "bulk_oob":
            assert ret == int(g["ret"][i]), (i, kind, ret)


def _check_codes(ref, new):
    """<= 0.1 % of codes differ, each by <= 1 LSB, after sign alignment; scales
    within one bf16 ulp."""
    Vr, Vn, Cr, Cn = orc.align_signs(ref, new)
    dv, dc = np.abs(Vr - Vn), np.abs(Cr - Cn)
    assert dv.max() <= 1 and (dv > 0).mean() <= 1e-3
    assert dc.max() <= 1 and (dc > 0).mean() <= 1e-3
    dm = np.abs(ref["mu8"].astype(np.int16) - new["mu8"].astype(np.int16))
    assert dm.max() <= 1 and (dm > 0).mean() <= 1e-3
    for k in ("vs", "cs", "mus"):
        rel = np.abs(ref[k] - new[k]) / np.maximum(np.abs(ref[k]), 1e-12)
        assert rel.max() <= 2 ** -7, k


def _golden_slabs(g):
    return {k: g["slab_" + k] for k in ("v4", "vs", "c8", "cs", "mu8", "mus")}


class _OracleApi:
    """The oracle's block rules driving its own page builder over numpy
    copies of the K planes (shared storage with the torch tensors the script
    mutates)."""

    def __init__(self, ls, K):
        self.ls, self.K = ls, K
        self.tags = np.full((ls.L, ls.NB, ls.N_KV, 8), np.nan, np.float32)
        self.slabs = [dict() for _ in range(ls.L)]     # block -> per-block slabs

    def _Kn(self, l):
        return self.K[l].float().numpy()

    def _build(self, layers, blocks):
        blocks = orc.mask_blocks(blocks, self.ls.NB, self.ls.NB)
        for l in layers:
            uniq = np.unique(blocks)
            if uniq.size == 0:
                continue
            out = orc.rki4_build_pages(self._Kn(l)[uniq])
            self.tags[l][uniq] = out["tag"]
            for i, b in enumerate(uniq):
                self.slabs[l][int(b)] = {k: v[i] for k, v in out.items()}
        return len(layers) * int(blocks.shape[0])

    def bulk(self, bt, sl, n, mf):
        return self._build(range(self.ls.L),
                           orc.bulk_blocks(t2n(bt)[:n], t2n(sl)[:n],
                                           self.ls.PAGE, mf))

    def stale(self, bt, sl, n, mf):
        return orc.delta_blocks(self.tags, [self._Kn(l) for l in range(self.ls.L)],
                                t2n(bt)[:n], t2n(sl)[:n], self.ls.PAGE,
                                mf).tolist()

    def delta(self, bt, sl, n, mf):
        return self._build(range(self.ls.L), np.array(self.stale(bt, sl, n, mf),
                                                      np.int64))

    def tail(self, bt, sl, n, rows):
        r = None if rows is None else t2n(rows)
        blocks = orc.tail_blocks(t2n(bt)[:n], t2n(sl)[:n], self.ls.PAGE, r)
        return self._build(range(self.ls.L), blocks)

    def refresh(self, layer, bt, sl, n, force):
        blocks = orc.refresh_blocks(self.tags[layer], self._Kn(layer),
                                    t2n(bt)[:n], t2n(sl)[:n], self.ls.PAGE, force)
        self._build([layer], blocks)
        return int(blocks.shape[0])


def test_oracle_block_rules_match_reference():
    ls = _script()
    g = load_golden("gqa_lifecycle")
    K, blocks, gen = ls.make_world()
    api = _OracleApi(ls, K)
    ev, rows, lens = ls.run(api, K, blocks, gen)
    _check_events(ev, g)
    np.testing.assert_array_equal(api.tags, g["tags"])           # NaN == NaN here
    keep = g["keep"].tolist()
    new = {k: np.stack([np.stack([api.slabs[l][b][k] for b in keep])
                        for l in range(ls.L)])
           for k in ("v4", "vs", "c8", "cs", "mu8", "mus")}
    _check_codes(_golden_slabs(g), new)


@pytest.mark.gpu
def test_gpu_build_lifecycle_matches_reference_and_oracle():
    from locks.selection import (Rki4State, rki4_build_bulk, rki4_build_delta,
                                 rki4_build_refresh, rki4_build_tail)
    from locks.selection.rki4_build import _delta_select
    DEV = "cuda"
    ls = _script()
    g = load_golden("gqa_lifecycle")
    K_cpu, blocks, gen = ls.make_world()
    K = [k.to(DEV) for k in K_cpu]
    st = Rki4State(DEV, num_layers=ls.L, num_blocks=ls.NB, n_kv=ls.N_KV, G=ls.G,
                   head_dim=ls.D, page=ls.PAGE, max_reqs=4, max_pages=ls.WIDTH,
                   budget_pages=4, sink_pages=1, window_pages=1)

    class Api:
        def bulk(self, bt, sl, n, mf):
            return rki4_build_bulk(st, K, bt, sl, n, mf)

        def stale(self, bt, sl, n, mf):
            return _delta_select(st, K, bt, sl, n, mf).tolist()

        def delta(self, bt, sl, n, mf):
            return rki4_build_delta(st, K, bt, sl, n, mf)

        def tail(self, bt, sl, n, rows):
            return rki4_build_tail(st, K, bt, sl, n, rows)

        def refresh(self, layer, bt, sl, n, force):
            return rki4_build_refresh(st, layer, K[layer], bt, sl, n, force=force)

    ev, rows, lens = ls.run(Api(), K, blocks, gen, to_dev=lambda t: t.to(DEV))
    torch.cuda.synchronize()
    _check_events(ev, g)
    # every tag, bit for bit (never-built blocks stay NaN), against the reference
    np.testing.assert_array_equal(t2n(st.pp_tag), g["tags"])
    # records of the blocks the events touched, against the reference
    keep = torch.tensor(g["keep"].tolist(), device=DEV)
    new = {"v4": t2n(st.pp_v4[:, keep]), "vs": t2n(st.pp_vs[:, keep]),
           "c8": t2n(st.pp_c8[:, keep]), "cs": t2n(st.pp_cs[:, keep]),
           "mu8": t2n(st.pp_mu8[:, keep]), "mus": t2n(st.pp_mus[:, keep])}
    _check_codes(_golden_slabs(g), new)
    # every block that carries a tag holds the oracle's summary of the FINAL
    # cache contents (a stale summary would show here), in both layers
    # (blocks finalized for the requests alive at the end; a block that lost its
    # request, like the third block of the finished request, keeps an old tag)
    live = sorted({blocks[n][pg] for n in rows for pg in range(lens[n] // ls.PAGE)})
    for l in range(ls.L):
        assert not np.isnan(g["tags"][l][live]).any()
        built = np.array(live)
        ref = orc.rki4_build_pages(t2n(K[l])[built])
        b = torch.tensor(built.tolist(), device=DEV)
        got = {"v4": t2n(st.pp_v4[l, b]), "vs": t2n(st.pp_vs[l, b]),
               "c8": t2n(st.pp_c8[l, b]), "cs": t2n(st.pp_cs[l, b]),
               "mu8": t2n(st.pp_mu8[l, b]), "mus": t2n(st.pp_mus[l, b])}
        _check_codes(ref, got)
    # the padded row's out-of-pool ids built nothing: block 0 of the table's
    # zero padding aside, no block outside the requests' own carries a tag
    owned = set(sum((blocks[n] for n in ("a", "b", "c")), [])) | {0}
    for l in range(ls.L):
        tagged = set(np.nonzero(~np.isnan(t2n(st.pp_tag[l])).any((-1, -2)))[0].tolist())
        assert tagged <= owned
