"""Generate the golden vectors under tests/golden/ by running the REFERENCE.

Run once, in a container that has the reference checkout, as

    LOCKS_REFERENCE_SRC=<reference>/src python tests/golden/make_golden.py

It imports the reference package ``locks`` (CPU torch path; its Triton kernels
through ``TRITON_INTERPRET=1``), feeds it the seeded synthetic inputs of
``locks-kv_b200/locks/synth.py`` and stores the reference's outputs as small
``.npz`` files.  Inputs are NOT stored: the tests regenerate them from the
seed with the same generator.  The test-suite never imports the reference.

The reference's decode kernels are interpreted with fp16 tensors because the
Triton interpreter does not read bf16 correctly; every bf16 value used here is
exactly representable in fp16 except below 2^-24, which does not matter at the
decode tolerance.
"""
from __future__ import annotations

import importlib.util
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("LOCKS_REFERENCE_SRC")
if not REF:
    raise SystemExit("set LOCKS_REFERENCE_SRC to the reference checkout's src/ "
                     "directory (the package `locks` v0.1.3 is imported from it)")
sys.path.insert(0, REF)

import numpy as np  # noqa: E402
import torch  # noqa: E402

spec = importlib.util.spec_from_file_location(
    "b200_synth", os.path.join(ROOT, "locks-kv_b200", "locks", "synth.py"))
synth = importlib.util.module_from_spec(spec)
sys.modules["b200_synth"] = synth
spec.loader.exec_module(synth)

from locks.attention.decode import (ResidentVSource,  # noqa: E402
                                    ensure_stage_b_buffers,
                                    sparse_paged_decode_batched)
from locks.selection import rki4_build as rb  # noqa: E402
from locks.selection.mla_score_torch import (mla_page_score_ref,  # noqa: E402
                                             topb_middle)
from locks.selection.mla_select import build_page_factors  # noqa: E402
from locks.selection.rki4_score_torch import rki4_score_torch  # noqa: E402
from locks.selection.rki4_state import Rki4State  # noqa: E402
from locks.selection.select import (_topb_select_kernel,  # noqa: E402
                                    _topb_select_torch, derive_page_params)
import triton  # noqa: E402


def f32(t):
    return t.detach().float().cpu().numpy()


def run_gqa(name, seed, shape, seq_lens, *, max_reqs=None, keep_blocks=48,
            combine="nrm", budget=None):
    case = synth.make_gqa_case(seed, shape, seq_lens, device="cpu")
    R = case.n_req
    MR = max_reqs or R
    page = shape.page
    st = Rki4State("cpu", num_layers=shape.n_layers, num_blocks=case.num_blocks,
                   n_kv=shape.n_kv, G=shape.G, head_dim=shape.d, page=page,
                   max_reqs=MR, max_pages=case.max_pages,
                   budget=(budget or 0.1),
                   budget_pages=(None if budget else shape.budget_pages),
                   sink_pages=shape.sink_pages,
                   window_pages=shape.window_pages, combine=combine)
    K_layers = [c[:, 0] for c in case.kv_caches]
    settled = case.seq_lens - 1
    max_fin = int((settled // page).max())
    n_built = rb.rki4_build_bulk(st, K_layers, case.block_table, settled, R,
                                 max_fin)
    derive_page_params(st, case.seq_lens, R)
    out = {"n_built": np.int64(n_built),
           "n_pages": st.n_pages[:R].numpy(), "n_sel_hi": st.n_sel_hi[:R].numpy(),
           "b_fix": st.b_fix[:R].numpy()}
    # slabs of the first keep_blocks logical pages of request 0 (layer 0)
    nb = min(keep_blocks, int(settled[0]) // page)
    blk = case.block_table[0, :nb].long()
    out.update({
        "slab_v4": st.pp_v4[0][blk].numpy(), "slab_vs": f32(st.pp_vs[0][blk]),
        "slab_c8": st.pp_c8[0][blk].numpy(), "slab_cs": f32(st.pp_cs[0][blk]),
        "slab_mu8": st.pp_mu8[0][blk].numpy(),
        "slab_mus": f32(st.pp_mus[0][blk]), "slab_tag": f32(st.pp_tag[0][blk]),
    })
    st.D, st.scale = shape.d, case.scale     # stamped by the builder upstream
    ensure_stage_b_buffers(st, "cpu", 128)
    hi_max = int(st.n_sel_hi[:R].max())
    cnt_max = 0
    per_layer = []
    for l in range(shape.n_layers):
        qpad = torch.zeros(MR, shape.n_kv * shape.G, shape.d,
                           dtype=torch.bfloat16)
        qpad[:R] = case.q[l]
        rki4_score_torch(st, l, qpad, case.block_table, case.seq_lens, R,
                         case.scale)
        if combine == "nrm":
            st.score.zero_()
            for r in range(R):
                hi = int(st.n_sel_hi[r])
                if hi > 0:
                    hm = st.score_h[r, :, :, :hi].amax(-1, keepdim=True)
                    acc = torch.zeros(shape.n_kv, hi)
                    for g in range(shape.G):       # g ascending, as the kernel
                        acc = acc + torch.exp(st.score_h[r, :, g, :hi] - hm[:, g])
                    st.score[r, :, :hi] = acc
        else:
            torch.amax(st.score_h, dim=2, out=st.score)
        _topb_select_torch(st, R)
        tab_torch = st.page_table.clone()
        cnt_torch = st.page_cnt.clone()
        # the reference's golden Triton selector must agree with its torch twin
        MP = case.max_pages
        P_PAD = triton.next_power_of_2(MP)
        S_PAD = triton.next_power_of_2(max(MP - st.window_pages - st.sink_pages, 2))
        _topb_select_kernel[(R, shape.n_kv)](
            st.score, st.n_pages, st.n_sel_hi, st.b_fix, st.page_table,
            st.page_cnt, st.sink_pages, st.score.stride(0), st.score.stride(1),
            MP, st.page_table.stride(0), st.page_table.stride(1),
            st.page_cnt.stride(0), P_PAD=P_PAD, S_PAD=S_PAD, num_warps=4)
        assert torch.equal(tab_torch[:R], st.page_table[:R]), "triton != torch"
        assert torch.equal(cnt_torch[:R], st.page_cnt[:R])
        # decode through the reference kernels (interpreter, fp16 storage)
        kv16 = case.kv_caches[l].to(torch.float16)
        q16 = qpad[:R].to(torch.float16)
        out16 = torch.zeros(R, shape.n_kv * shape.G, shape.d,
                            dtype=torch.float16)
        sparse_paged_decode_batched(q16, kv16, case.block_table, case.seq_lens,
                                    st, out16, ResidentVSource(kv16),
                                    scale=case.scale)
        cnt_max = max(cnt_max, int(st.page_cnt[:R].max()))
        per_layer.append((st.score_h[:R, :, :, :hi_max].clone(),
                          st.score[:R, :, :hi_max].clone(),
                          st.page_table[:R].clone(), st.page_cnt[:R].clone(),
                          out16.float()))
    out["score_h"] = np.stack([f32(p[0]) for p in per_layer])
    out["score"] = np.stack([f32(p[1]) for p in per_layer])
    out["page_table"] = np.stack([p[2][:, :, :cnt_max].numpy()
                                  for p in per_layer])
    out["page_cnt"] = np.stack([p[3].numpy() for p in per_layer])
    out["out"] = np.stack([f32(p[4]) for p in per_layer])
    out["split"] = np.int64(st.split)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, "built", n_built, "split", st.split, "cnt",
          st.page_cnt[:R].tolist())


def run_topb_kat():
    """Adversarial top-b cases: ties at the threshold, all-equal scores,
    underflow to +0, short rows (keep-all), b >= selectable."""
    rng = np.random.default_rng(7)
    MP, n_kv = 96, 3
    rows = []
    # (n_tok, scores builder)
    base = rng.random((n_kv, MP)).astype(np.float32)
    tie = base.copy(); tie[:, 10:40] = 0.5                       # tie band at tau
    alleq = np.full((n_kv, MP), 1.0, np.float32)
    zeros = np.zeros((n_kv, MP), np.float32); zeros[:, 5] = 1.0  # tau = +0
    coarse = np.round(base * 4) / 4                              # many collisions
    specs = [(96 * 16 - 3, base), (96 * 16, tie), (90 * 16, alleq),
             (80 * 16 + 1, zeros), (70 * 16, coarse), (3 * 16, base),
             (5 * 16 + 2, base), (20 * 16, tie), (1, base)]
    R = len(specs)
    st = Rki4State("cpu", num_layers=1, num_blocks=4, n_kv=n_kv, G=2,
                   head_dim=128, page=16, max_reqs=R, max_pages=MP,
                   budget_pages=12, sink_pages=2, window_pages=3)
    sl = torch.tensor([s[0] for s in specs], dtype=torch.int32)
    derive_page_params(st, sl, R)
    for r, (_, sc) in enumerate(specs):
        st.score[r] = torch.from_numpy(sc)
    _topb_select_torch(st, R)
    tab, cnt = st.page_table.clone(), st.page_cnt.clone()
    P_PAD = triton.next_power_of_2(MP)
    S_PAD = triton.next_power_of_2(max(MP - 3 - 2, 2))
    _topb_select_kernel[(R, n_kv)](
        st.score, st.n_pages, st.n_sel_hi, st.b_fix, st.page_table,
        st.page_cnt, st.sink_pages, st.score.stride(0), st.score.stride(1), MP,
        st.page_table.stride(0), st.page_table.stride(1),
        st.page_cnt.stride(0), P_PAD=P_PAD, S_PAD=S_PAD, num_warps=4)
    assert torch.equal(tab, st.page_table) and torch.equal(cnt, st.page_cnt)
    # fractional-budget derive on the same lengths
    st2 = Rki4State("cpu", num_layers=1, num_blocks=4, n_kv=n_kv, G=2,
                    head_dim=128, page=16, max_reqs=R, max_pages=MP,
                    budget=0.07, sink_pages=2, window_pages=3)
    derive_page_params(st2, sl, R)
    np.savez_compressed(
        os.path.join(HERE, "topb_kat.npz"), seq_lens=sl.numpy(),
        score=st.score.numpy(), n_pages=st.n_pages.numpy(),
        n_sel_hi=st.n_sel_hi.numpy(), b_fix=st.b_fix.numpy(),
        page_table=tab.numpy(), page_cnt=cnt.numpy(),
        frac_n_pages=st2.n_pages.numpy(), frac_n_sel_hi=st2.n_sel_hi.numpy(),
        frac_b_fix=st2.b_fix.numpy())
    print("topb_kat cnt", cnt.tolist())


def _load_lifecycle():
    spec = importlib.util.spec_from_file_location(
        "lifecycle_script", os.path.join(HERE, "lifecycle_script.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def run_lifecycle():
    """The scripted summary life cycle (tests/golden/lifecycle_script.py) played
    through the reference's rki4_build_{bulk,delta,tail,refresh} and
    _delta_select: per event the return value and the stale block list, at the
    end every tag and the records of the blocks the events touched."""
    from locks.selection.build import _delta_select
    ls = _load_lifecycle()
    K, blocks, g = ls.make_world()
    st = Rki4State("cpu", num_layers=ls.L, num_blocks=ls.NB, n_kv=ls.N_KV,
                   G=ls.G, head_dim=ls.D, page=ls.PAGE, max_reqs=4,
                   max_pages=ls.WIDTH, budget_pages=4, sink_pages=1,
                   window_pages=1)

    class Api:
        def bulk(self, bt, sl, n, mf):
            return rb.rki4_build_bulk(st, K, bt, sl, n, mf)

        def delta(self, bt, sl, n, mf):
            return rb.rki4_build_delta(st, K, bt, sl, n, mf)

        def stale(self, bt, sl, n, mf):
            return _delta_select(st.pp_tag, K, bt, sl, n, st.page, mf,
                                 st.tagw).tolist()

        def tail(self, bt, sl, n, rows):
            return rb.rki4_build_tail(st, K, bt, sl, n, rows)

        def refresh(self, layer, bt, sl, n, force):
            return rb.rki4_build_refresh(st, layer, K[layer], bt, sl, n,
                                         force=force)

    ev, rows, lens = ls.run(Api(), K, blocks, g)
    keep = [blocks["b"][3]] + blocks["c"][:3] + [blocks["a"][6], blocks["a"][2],
                                                 blocks["a"][0], blocks["b"][19]]
    kb = torch.tensor(keep)
    out = {"ret": np.array([e[1] for e in ev], np.int64),
           "kind": np.array([e[0] for e in ev]),
           "tags": f32(st.pp_tag), "keep": np.array(keep, np.int64),
           "slab_v4": st.pp_v4[:, kb].numpy(), "slab_vs": f32(st.pp_vs[:, kb]),
           "slab_c8": st.pp_c8[:, kb].numpy(), "slab_cs": f32(st.pp_cs[:, kb]),
           "slab_mu8": st.pp_mu8[:, kb].numpy(),
           "slab_mus": f32(st.pp_mus[:, kb])}
    for i, e in enumerate(ev):
        if e[2] is not None:
            out[f"stale{i}"] = np.array(e[2], np.int64)
    np.savez_compressed(os.path.join(HERE, "gqa_lifecycle.npz"), **out)
    print("gqa_lifecycle", [(e[0], e[1], e[2]) for e in ev])


def run_mla(name, seed, shape, seq_lens, rank=8):
    """MLA: the reference's factor build, torch scorer, keep rule and the
    attention block of its backend (``LocksMLAImpl.forward_mqa`` itself needs a
    CUDA device for its Triton scorer, so its CPU-runnable parts are called
    one by one in the order that method calls them)."""
    case = synth.make_mla_case(seed, shape, seq_lens, device="cpu", n_layers=1)
    Lkv, page = shape.kv_lora_rank, shape.page
    cache = case.caches[0]
    q = case.q[0].float()
    res = {}
    for bi, L in enumerate(seq_lens):
        n_pages = (L + page - 1) // page
        n_cache = L // page
        blks = case.block_table[bi, :n_pages].long()
        kvb = cache.index_select(0, blks).reshape(-1, shape.width)[:L]
        kv_c = kvb[:n_cache * page, :Lkv].float()
        Lf, Rf = build_page_factors(kv_c, n_cache, page, rank)
        k_rope = kvb[:n_cache * page, Lkv:].float().view(n_cache, page, -1)
        C8 = Lf @ Rf
        valid = torch.full((n_cache,), page, dtype=torch.long)
        ps = torch.full((n_pages,), float("-inf"))
        ps[:n_cache] = mla_page_score_ref(q[bi, :, :Lkv], q[bi, :, Lkv:], C8,
                                          k_rope, valid, case.scale)
        keep = topb_middle(ps, shape.budget_pages, shape.sink_pages,
                           shape.window_pages)
        idx = keep.nonzero().flatten()
        sel = cache.index_select(0, case.block_table[bi].long()[idx]) \
            .reshape(-1, shape.width).float()
        pos = (idx[:, None] * page + torch.arange(page)[None]).reshape(-1)
        sc = (q[bi] @ sel.T) * case.scale
        sc = sc.masked_fill(~(pos < L)[None], float("-inf"))
        attn = torch.softmax(sc, -1)
        res[f"score{bi}"] = ps.numpy()
        res[f"keep{bi}"] = idx.numpy()
        res[f"o{bi}"] = (attn @ sel[:, :Lkv]).numpy()
        res[f"lse{bi}"] = torch.logsumexp(sc, -1).numpy()
        if bi == 0:
            res["Lf0"] = Lf[:24].numpy()
            res["Rf0"] = Rf[:24].numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **res)
    print(name, "kept", [int(res[f"keep{b}"].shape[0])
                         for b in range(len(seq_lens))])


if __name__ == "__main__":
    torch.set_num_threads(8)
    run_gqa("gqa_c0", 1234, synth.CONFIG0, [4097])
    run_gqa("gqa_ragged", 99,
            synth.GqaShape(n_layers=2, n_kv=2, G=8, budget_pages=8,
                           sink_pages=1, window_pages=2, n_needles=2),
            [37, 530, 1203, 16 * 40], max_reqs=6, keep_blocks=20)
    run_gqa("gqa_maxfrac", 5,
            synth.GqaShape(n_layers=1, n_kv=4, G=2, budget_pages=0,
                           sink_pages=2, window_pages=1, n_needles=2),
            [911, 64], keep_blocks=8, combine="max", budget=0.15)
    run_topb_kat()
    run_lifecycle()
    run_mla("mla_small", 21,
            synth.MlaShape(n_layers=1, budget_pages=24, sink_pages=1,
                           window_pages=4), [777, 2048 + 5, 300])
