"""CPU oracle for the LOCKS decode hot path -- TEST INFRASTRUCTURE ONLY.

A numpy restatement of the reference algorithm (Js-Hwang1/locks-kv v0.1.3,
package ``locks``), one function per stage, each citing the reference file and
lines it follows (paths are relative to the reference's ``src/locks``).  It is
the checker the CUDA kernels are compared against and the timed CPU baseline of
the benchmark; nothing on the product path imports it.

Parity status: PINNED.  ``tests/golden/*.npz`` hold outputs of the reference's
own Python/torch code run on CPU (script ``tests/golden/make_golden.py``); the
CPU test-suite checks every function here against them.  The one third-party
piece is the symmetric eigensolver: the reference calls ``torch.linalg.eigh``
(LAPACK ``ssyevd``; torch>=2.4 per its pyproject), this file calls
``numpy.linalg.eigh`` (also ``ssyevd``).  Eigenvectors carry a free sign, so
summary codes are compared after per-column sign alignment
(:func:`align_signs`); everything downstream of the codes is sign-invariant.
One function is NOT pinned: :func:`rope_and_cache` restates a CUDA-only kernel
of the reference (no CPU twin exists to generate vectors from); its arithmetic
is a handful of fp32 products and sums read directly off the source.

All "bf16" arrays are float32 arrays holding bf16-representable values.
"""
from __future__ import annotations

import math

import numpy as np

RNK = 8          # summary rank                      selection/rki4_state.py:62
TAGW = 8         # content-tag width (bf16 channels) selection/rki4_state.py:51
QMAX, QMIN = 7, -8   # int4 range of the V basis     selection/rki4_state.py:76-77
NEG_INF = float("-inf")


# --------------------------------------------------------------------------- #
# bf16 / fp16 helpers                                                          #
# --------------------------------------------------------------------------- #
def bf16_round(x):
    """Round float32 -> nearest-even bf16, returned as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    nan = np.isnan(x)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) \
        & np.uint32(0xFFFF0000)
    out = r.view(np.float32).copy()
    out[nan] = np.nan
    return out


def fp16_round(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


# --------------------------------------------------------------------------- #
# Stage A.0 -- rki4 summary build                                              #
# --------------------------------------------------------------------------- #
def pack_int4(Vc):
    """(…, RNK, d) int8 codes -> (…, RNK, d/2) uint8, low nibble = even d row.
    selection/rki4_build.py:161-175 (``_pack_ibit`` at IBITS=4)."""
    lo = (Vc[..., 0::2].astype(np.int16) & 15).astype(np.uint8)
    hi = (Vc[..., 1::2].astype(np.int16) & 15).astype(np.uint8)
    return (lo | (hi << 4)).astype(np.uint8)


def unpack_int4(v4):
    """Inverse of :func:`pack_int4`: two's-complement nibbles ((n ^ 8) - 8).
    selection/rki4_score_torch.py:41-55."""
    v = v4.astype(np.int16)
    lo = ((v & 15) ^ 8) - 8
    hi = (((v >> 4) & 15) ^ 8) - 8
    out = np.empty(v4.shape[:-1] + (v4.shape[-1] * 2,), dtype=np.int8)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return out


def rki4_build_pages(Kp):
    """Summarise finalized key pages.

    Kp: (N, page, n_kv, d) float32 holding bf16 values (the engine K half
    gathered at N physical blocks).  Returns a dict with the seven summary
    components for each (block, kv-head):

      v4 (N,n_kv,8,d/2) u8 | vs (N,n_kv,8) bf16 | c8 (N,n_kv,page,8) i8 |
      cs (N,n_kv,page) bf16 | mu8 (N,n_kv,d) i8 | mus (N,n_kv) bf16 |
      tag (N,n_kv,8) bf16

    Follows selection/rki4_build.py:147-158 (``_write_pre``), :93-129
    (``_eigh_chunked``, default LAPACK path) and :178-225 (``_write_post``).
    Quantisation uses the fp32 scale; the stored scale is its bf16 rounding.
    """
    Kp = np.asarray(Kp, dtype=np.float32)
    N, page, n_kv, d = Kp.shape
    tag = Kp[:, page - 1, :, :TAGW].copy()
    K = np.ascontiguousarray(Kp.transpose(0, 2, 1, 3))          # (N,n_kv,page,d)
    mu = (K.sum(2, dtype=np.float32) / np.float32(page)).astype(np.float32)
    dc = K - mu[:, :, None, :]
    Gm = np.matmul(dc, dc.transpose(0, 1, 3, 2))                # (N,n_kv,page,page)
    S2, U = np.linalg.eigh(Gm.reshape(-1, page, page))          # ascending
    S2 = S2.reshape(N, n_kv, page).astype(np.float32)
    U = U.reshape(N, n_kv, page, page).astype(np.float32)
    S8 = np.sqrt(np.maximum(S2[..., -RNK:], np.float32(1e-10)))
    U8 = U[..., -RNK:]
    C = U8 * S8[..., None, :]                                   # (N,n_kv,page,8)
    V = np.matmul(dc.transpose(0, 1, 3, 2), U8) / S8[..., None, :]   # (N,n_kv,d,8)
    vsc = np.maximum(np.abs(V).max(2) / np.float32(QMAX), np.float32(1e-8))
    Vq = np.clip(np.rint(V / vsc[:, :, None, :]), QMIN, QMAX)
    Vc = np.ascontiguousarray(Vq.transpose(0, 1, 3, 2)).astype(np.int8)
    csc = np.maximum(np.abs(C).max(-1) / np.float32(127.0), np.float32(1e-8))
    Cq = np.clip(np.rint(C / csc[..., None]), -127, 127)
    msc = np.maximum(np.abs(mu).max(-1) / np.float32(127.0), np.float32(1e-8))
    muq = np.clip(np.rint(mu / msc[..., None]), -127, 127)
    return {
        "v4": pack_int4(Vc), "vs": bf16_round(vsc),
        "c8": Cq.astype(np.int8), "cs": bf16_round(csc),
        "mu8": muq.astype(np.int8), "mus": bf16_round(msc),
        "tag": tag,
    }


def align_signs(ref, new):
    """Per-(block, head, column) sign that maps ``new``'s eigen-gauge onto
    ``ref``'s: s = sign(sum_t C_ref[t,r] * C_new[t,r]) (0 -> +1).  Returns
    (V_ref, V_new_aligned, C_ref, C_new_aligned) as int16 arrays.
    The eigenvector sign freedom is stated by the reference itself at
    selection/jacobi_dual.py:10-17 and selection/rki4_build.py:65-72."""
    Vr = unpack_int4(ref["v4"]).astype(np.int16)               # (N,n_kv,8,d)
    Vn = unpack_int4(new["v4"]).astype(np.int16)
    Cr = ref["c8"].astype(np.int16)                             # (N,n_kv,page,8)
    Cn = new["c8"].astype(np.int16)
    s = np.sign((Cr.astype(np.int32) * Cn.astype(np.int32)).sum(-2))
    s[s == 0] = 1
    s = s.astype(np.int16)                                      # (N,n_kv,8)
    return Vr, Vn * s[..., None], Cr, Cn * s[..., None, :]


def bulk_blocks(block_table, settled_lens, page, max_fin):
    """All finalized (request, page) physical blocks, invalid slots -> 0.
    selection/build.py:414-426 (``_bulk_blocks``)."""
    bt = np.asarray(block_table)[:, :max_fin].astype(np.int64).copy()
    n_fin = np.asarray(settled_lens).astype(np.int64) // page
    valid = np.arange(max_fin)[None, :] < n_fin[:, None]
    bt[~valid] = 0
    return bt.reshape(-1)


def tail_blocks(block_table, settled_lens, page, rows=None):
    """Physical block of each request's last finalized page (clamped to 0).
    selection/build.py:372-385 (``_tail_blocks``)."""
    bt = np.asarray(block_table).astype(np.int64)
    sl = np.asarray(settled_lens).astype(np.int64)
    if rows is not None:
        bt, sl = bt[rows], sl[rows]
    fin1 = np.maximum(sl // page - 1, 0)
    return bt[np.arange(bt.shape[0]), fin1]


def delta_blocks(tag_slab, K_layers, block_table, settled_lens, page, max_fin):
    """Blocks whose stored content tag differs from the live K in any layer
    (NaN tags never compare equal).  selection/build.py:475-488."""
    bt = np.asarray(block_table)[:, :max_fin].astype(np.int64).copy()
    fin = np.asarray(settled_lens).astype(np.int64) // page
    valid = np.arange(max_fin)[None, :] < fin[:, None]
    bt[~valid] = 0
    blk = bt.reshape(-1)
    stale = np.zeros(blk.shape[0], dtype=bool)
    for l, K in enumerate(K_layers):
        cur = K[blk, page - 1, :, :TAGW]
        with np.errstate(invalid="ignore"):
            stale |= (cur != tag_slab[l][blk]).any(-1).any(-1)
    return blk[stale & valid.reshape(-1)]


def mask_blocks(blocks, nb_state, nb_cache):
    """Drop block ids outside the summary slab or the K tensor (the engine's
    memory-profile pass hands out placeholder tables).
    selection/rki4_build.py:133-144 (``_mask_blocks``)."""
    blocks = np.asarray(blocks, dtype=np.int64)
    nb = min(int(nb_state), int(nb_cache))
    return blocks[(blocks >= 0) & (blocks < nb)]


def refresh_blocks(tag_layer, K, block_table, settled_lens, page, force=False):
    """Single-layer refresh: the unique finalized blocks of the batch whose
    stored tag differs from the live K of THIS layer (all of them when
    ``force``).  selection/rki4_build.py:320-364 (``rki4_build_refresh``)."""
    sl = np.asarray(settled_lens).astype(np.int64)
    n_fin = sl // page
    max_fin = int(n_fin.max()) if n_fin.size else 0
    if max_fin == 0:
        return np.zeros(0, np.int64)
    bt = np.asarray(block_table)[:, :max_fin].astype(np.int64)
    fin = np.arange(max_fin)[None, :] < n_fin[:, None]
    blk = mask_blocks(bt[fin], tag_layer.shape[0], K.shape[0])
    if blk.size == 0:
        return blk
    if force:
        stale = np.ones(blk.shape[0], dtype=bool)
    else:
        cur = K[blk, page - 1, :, :TAGW]
        with np.errstate(invalid="ignore"):
            stale = (cur != tag_layer[blk]).any(-1).any(-1)
    return np.unique(blk[stale])


# --------------------------------------------------------------------------- #
# Stage A.1 -- per-step page parameters                                        #
# --------------------------------------------------------------------------- #
def derive_page_params(seq_lens, page, window, sink, budget_pages=0,
                       budget=0.1):
    """(n_pages, n_sel_hi, b) per request.  selection/select.py:36-45."""
    sl = np.asarray(seq_lens).astype(np.int64)
    npg = (sl + (page - 1)) // page
    nsh = npg - window
    s = nsh - sink
    bp = np.broadcast_to(np.asarray(budget_pages if budget_pages is not None
                                    else 0, dtype=np.int64), s.shape)
    b_abs = np.maximum(np.minimum(bp, np.maximum(s, 1)), 1)
    bf = np.ceil(s.astype(np.float64) * np.float64(budget))
    b_frac = np.minimum(np.maximum(bf.astype(np.int64), 1), np.maximum(s, 1))
    # budget_pages may be one number (the reference's engine-wide BUDGET_ABS)
    # or one entry per request (> 0: pages, <= 0: the fraction)
    b = np.where(bp > 0, b_abs, b_frac)
    return npg.astype(np.int32), nsh.astype(np.int32), b.astype(np.int32)


# --------------------------------------------------------------------------- #
# Stage A.2 -- page score                                                      #
# --------------------------------------------------------------------------- #
def quantize_query(q, n_kv, G):
    """Per-(kv-head, group-member) int8 round trip of q.
    Returns (q8 int8 (R,n_kv,G,d), qs float32 (R,n_kv,G,1)).
    selection/rki4_score_torch.py:121-123."""
    q = np.asarray(q, dtype=np.float32)
    R = q.shape[0]
    qv = q.reshape(R, n_kv, G, -1)
    qs = np.maximum(np.abs(qv).max(-1, keepdims=True), np.float32(1e-8)) \
        / np.float32(127.0)
    q8 = np.rint(qv / qs)
    return q8.astype(np.int8), qs.astype(np.float32)


def rki4_score(slabs, q, block_table, n_sel_hi, scale, n_kv, G, max_pages,
               chunk=2048):
    """Per-head page log-sum-exp estimate ``score_h (R, n_kv, G, MP)`` for
    pages [0, n_sel_hi[r]); everything else is 0.

    ``slabs``: dict of per-block arrays for one layer (keys as returned by
    :func:`rki4_build_pages`, indexed by physical block).
    Follows selection/rki4_score_torch.py:111-160.
    """
    q8, qs = quantize_query(q, n_kv, G)
    qref = q8.astype(np.float32) * qs                          # (R,n_kv,G,d)
    R = qref.shape[0]
    d = qref.shape[-1]
    NB = slabs["v4"].shape[0]
    out = np.zeros((R, n_kv, G, max_pages), dtype=np.float32)
    s = np.float32(scale)
    for r in range(R):
        hi = int(n_sel_hi[r])
        for c0 in range(0, max(hi, 0), chunk):
            c1 = min(c0 + chunk, hi)
            blk = np.clip(np.asarray(block_table[r, c0:c1]).astype(np.int64),
                          0, NB - 1)
            Vq = unpack_int4(slabs["v4"][blk]).astype(np.float32)   # (P,n_kv,8,d)
            Vref = Vq * slabs["vs"][blk][..., None]
            Cref = slabs["c8"][blk].astype(np.float32) \
                * slabs["cs"][blk][..., None]                       # (P,n_kv,page,8)
            muref = slabs["mu8"][blk].astype(np.float32) \
                * slabs["mus"][blk][..., None]                      # (P,n_kv,d)
            qt = np.einsum("pknd,kgd->pkgn", Vref, qref[r], optimize=True)
            tok = np.einsum("pktn,pkgn->pkgt", Cref, qt, optimize=True)
            mud = np.einsum("pkd,kgd->pkg", muref, qref[r], optimize=True)
            x = (tok + mud[..., None]) * s
            m = x.max(-1, keepdims=True)
            S = (m[..., 0] + np.log(np.exp(x - m).sum(-1))).astype(np.float32)
            out[r, :, :, c0:c1] = S.transpose(1, 2, 0)
    return out


def nrm_combine(score_h, n_sel_hi):
    """GQA combine: score[p] = sum_g exp(S[g,p] - max_{p' < n_sel_hi} S[g,p'])
    for p < n_sel_hi, summed in ascending g.  Pages >= n_sel_hi are left 0
    (never consumed).  selection/select_cuda.py:547-658."""
    R, n_kv, G, MP = score_h.shape
    score = np.zeros((R, n_kv, MP), dtype=np.float32)
    for r in range(R):
        hi = int(n_sel_hi[r])
        if hi <= 0:
            continue
        S = score_h[r, :, :, :hi]
        hm = S.max(-1, keepdims=True)
        acc = np.zeros((n_kv, hi), dtype=np.float32)
        for g in range(G):
            acc = acc + np.exp((S[:, g] - hm[:, g]).astype(np.float32))
        score[r, :, :hi] = acc
    return score


def max_combine(score_h):
    """Plain GQA group max (the ``quad_combine="max"`` ablation arm).
    selection/rki4_score_cuda.py:3497."""
    return score_h.max(2)


# --------------------------------------------------------------------------- #
# Stage A.3 -- exact top-b page selection                                      #
# --------------------------------------------------------------------------- #
def topb_select(score, n_pages, n_sel_hi, b_fix, sink, max_pages=None):
    """Ascending page table (-1 padded) + count per (request, kv-head).

    tau = b-th largest score over [sink, n_sel_hi); keep {> tau}, then pages
    == tau in ascending page order until exactly b selectable pages are kept;
    always keep [0, sink) and [n_sel_hi, n_pages); keep everything when the
    selectable range has <= 1 page.  selection/select.py:123-180 (torch twin)
    and :65-117 (golden kernel).
    """
    R, n_kv, MP = score.shape
    table = np.full((R, n_kv, MP), -1, dtype=np.int32)
    cnt = np.zeros((R, n_kv), dtype=np.int32)
    for r in range(R):
        npg, nsh, b = int(n_pages[r]), int(n_sel_hi[r]), int(b_fix[r])
        lo = min(sink, max(npg, 0))
        hi = max(min(nsh, npg), lo)
        L = hi - lo
        for kh in range(n_kv):
            keep = np.zeros(MP, dtype=bool)
            if L <= 1:
                keep[:max(npg, 0)] = True
            else:
                keep[:lo] = True
                keep[hi:npg] = True
                sel = score[r, kh, lo:hi]
                if b >= L:
                    keep[lo:hi] = True
                else:
                    tau = np.sort(sel)[::-1][b - 1]
                    gt = sel > tau
                    quota = max(b - int(gt.sum()), 0)
                    eq = sel == tau
                    eqrank = np.cumsum(eq.astype(np.int32))
                    keep[lo:hi] = gt | (eq & (eqrank <= quota))
            keep[max(npg, 0):] = False
            idx = np.nonzero(keep)[0].astype(np.int32)
            cnt[r, kh] = idx.shape[0]
            table[r, kh, :idx.shape[0]] = idx
    return table, cnt


# --------------------------------------------------------------------------- #
# Stage B -- split-K sparse paged decode + merge                               #
# --------------------------------------------------------------------------- #
def pps_min_default(n_req, n_kv=8):
    """Minimum pages per split program.  attention/decode.py:162-203
    (sm_90 table; the sm_120 and env rows are not part of the path)."""
    if n_kv == 1 and 4 < n_req <= 16:
        return 4
    if n_req == 1:
        return 2
    return 8 if n_req < 16 else 16


def sparse_decode_split(q, Kc, Vc, block_table, page_table, page_cnt, seq_lens,
                        scale, n_kv, G, split, pps_min):
    """Split-K partials (m, l, acc) over the selected pages.

    q (R, n_kv*G, d) bf16-valued; Kc/Vc (NB, page, n_kv, d) bf16-valued.
    Returns m, l (R,n_kv,split,G) and acc (R,n_kv,split,G,d); inactive splits
    keep m=-inf, l=0, acc=0 (the reference does not store them at all).
    QK is a bf16 dot with fp32 accumulation, P and V are rounded to fp16 for
    the PV product.  attention/decode.py:226-322.
    """
    q = np.asarray(q, dtype=np.float32)
    R = q.shape[0]
    d = q.shape[-1]
    page = Kc.shape[1]
    m_part = np.full((R, n_kv, split, G), NEG_INF, dtype=np.float32)
    l_part = np.zeros((R, n_kv, split, G), dtype=np.float32)
    acc_part = np.zeros((R, n_kv, split, G, d), dtype=np.float32)
    offs_t = np.arange(page)
    for r in range(R):
        sl = int(seq_lens[r])
        for kh in range(n_kv):
            cnt = int(page_cnt[r, kh])
            pps = max(-(-cnt // split), pps_min)
            qg = q[r, kh * G:(kh + 1) * G]                      # (G,d)
            for sp in range(split):
                j0 = sp * pps
                if j0 >= cnt:
                    break
                j1 = min(j0 + pps, cnt)
                m_i = np.full(G, NEG_INF, dtype=np.float32)
                l_i = np.zeros(G, dtype=np.float32)
                acc = np.zeros((G, d), dtype=np.float32)
                for j in range(j0, j1):
                    pt = int(page_table[r, kh, j])
                    blk = int(block_table[r, pt])
                    tmask = (pt * page + offs_t) < sl
                    k = np.where(tmask[:, None], Kc[blk, :, kh], 0.0)
                    v = np.where(tmask[:, None], Vc[blk, :, kh], 0.0)
                    s = (qg @ k.T).astype(np.float32) * np.float32(scale)
                    s = np.where(tmask[None, :], s, NEG_INF)
                    m_new = np.maximum(m_i, s.max(1))
                    with np.errstate(invalid="ignore"):
                        alpha = np.exp(m_i - m_new)
                        p = np.exp(s - m_new[:, None])
                    alpha = np.where(np.isnan(alpha), 0.0, alpha)
                    p = np.where(np.isnan(p), 0.0, p).astype(np.float32)
                    l_i = l_i * alpha + p.sum(1)
                    acc = acc * alpha[:, None] \
                        + fp16_round(p) @ fp16_round(v)
                    m_i = m_new
                m_part[r, kh, sp] = m_i
                l_part[r, kh, sp] = l_i
                acc_part[r, kh, sp] = acc
    return m_part, l_part, acc_part


def merge_splits(m_part, l_part, acc_part, page_cnt, split, pps_min):
    """Recombine the active split partials.  attention/merge.py:113-152.
    Returns out (R, n_kv*G, d) float32 (the reference stores it in q's dtype);
    rows with no attended page are 0, never NaN."""
    R, n_kv, _, G = m_part.shape
    d = acc_part.shape[-1]
    out = np.zeros((R, n_kv * G, d), dtype=np.float32)
    for r in range(R):
        for kh in range(n_kv):
            cnt = int(page_cnt[r, kh])
            pps = max(-(-cnt // split), pps_min)
            n_act = -(-cnt // pps)
            for g in range(G):
                m = m_part[r, kh, :n_act, g]
                l = l_part[r, kh, :n_act, g]
                a = acc_part[r, kh, :n_act, g]
                if n_act == 0:
                    continue
                m_max = m.max()
                with np.errstate(invalid="ignore"):
                    w = np.where(l > 0, np.exp(m - m_max), 0.0).astype(np.float32)
                l_tot = np.float32((l * w).sum(dtype=np.float32))
                o = (a * w[:, None]).sum(0, dtype=np.float32)
                out[r, kh * G + g] = o / l_tot if l_tot > 0 else 0.0
    return out


def attention_over_pages(q, Kc, Vc, block_table, page_table, page_cnt,
                         seq_lens, scale, n_kv, G):
    """fp64 softmax attention over exactly the selected pages (accuracy
    reference for the decode, independent of the split structure)."""
    q = np.asarray(q, dtype=np.float64)
    R, _, d = q.shape
    page = Kc.shape[1]
    out = np.zeros((R, n_kv * G, d), dtype=np.float64)
    lse = np.full((R, n_kv * G), NEG_INF, dtype=np.float64)
    for r in range(R):
        sl = int(seq_lens[r])
        for kh in range(n_kv):
            cnt = int(page_cnt[r, kh])
            if cnt == 0:
                continue
            pts = np.asarray(page_table[r, kh, :cnt]).astype(np.int64)
            blks = np.asarray(block_table[r])[pts].astype(np.int64)
            pos = (pts[:, None] * page + np.arange(page)[None, :]).reshape(-1)
            ok = pos < sl
            k = Kc[blks, :, kh].reshape(-1, d).astype(np.float64)[ok]
            v = Vc[blks, :, kh].reshape(-1, d).astype(np.float64)[ok]
            s = q[r, kh * G:(kh + 1) * G] @ k.T * float(scale)
            mx = s.max(-1, keepdims=True)
            p = np.exp(s - mx)
            den = p.sum(-1, keepdims=True)
            out[r, kh * G:(kh + 1) * G] = (p / den) @ v
            lse[r, kh * G:(kh + 1) * G] = (mx + np.log(den))[:, 0]
    return out, lse


def dense_decode(q, Kc, Vc, block_table, seq_lens, scale, n_kv, G):
    """Full-KV paged decode (every page of every request)."""
    R = np.asarray(q).shape[0]
    page = Kc.shape[1]
    MP = np.asarray(block_table).shape[1]
    table = np.full((R, n_kv, MP), -1, dtype=np.int32)
    cnt = np.zeros((R, n_kv), dtype=np.int32)
    for r in range(R):
        npg = -(-int(seq_lens[r]) // page)
        table[r, :, :npg] = np.arange(npg, dtype=np.int32)[None]
        cnt[r, :] = npg
    return attention_over_pages(q, Kc, Vc, block_table, table, cnt, seq_lens,
                                scale, n_kv, G)


# --------------------------------------------------------------------------- #
# End-to-end GQA step                                                          #
# --------------------------------------------------------------------------- #
def gqa_decode_step(slabs, q, Kc, Vc, block_table, seq_lens, scale, *, n_kv, G,
                    page, window, sink, budget_pages=0, budget=0.1,
                    combine="nrm", split=16, pps_min=None):
    """derive -> score -> combine -> top-b -> split decode -> merge for one
    layer; returns a dict of every intermediate.  Call order follows
    backend/attn.py:232-386 and backend/_runtime.py:661-723."""
    R = np.asarray(q).shape[0]
    MP = np.asarray(block_table).shape[1]
    npg, nsh, b = derive_page_params(seq_lens, page, window, sink,
                                     budget_pages, budget)
    score_h = rki4_score(slabs, q, block_table, nsh, scale, n_kv, G, MP)
    score = nrm_combine(score_h, nsh) if combine == "nrm" \
        else max_combine(score_h)
    table, cnt = topb_select(score, npg, nsh, b, sink)
    if pps_min is None:
        pps_min = pps_min_default(R, n_kv)
    m, l, acc = sparse_decode_split(q, Kc, Vc, block_table, table, cnt,
                                    seq_lens, scale, n_kv, G, split, pps_min)
    out = merge_splits(m, l, acc, cnt, split, pps_min)
    return {"n_pages": npg, "n_sel_hi": nsh, "b": b, "score_h": score_h,
            "score": score, "page_table": table, "page_cnt": cnt,
            "m_part": m, "l_part": l, "acc_part": acc, "out": out}


# --------------------------------------------------------------------------- #
# KV-write neighbour (parity unpinned: the reference kernel is CUDA-only)       #
# --------------------------------------------------------------------------- #
def rope_and_cache(key, val, k_cache, v_cache, slot_mapping, positions, cos_sin,
                   rot_dim, neox, page=16):
    """Rotate the new tokens' K and scatter K, V into the paged cache, in place.

    tier/k5_cuda.py:55-77 (``locks_rope_elem``) and :660-687
    (``rope_and_cache_fixc_kernel``).  key, val: (n_tok, n_kv, d) bf16-valued
    float32; caches (NB, page, n_kv, d); cos_sin (P, rot_dim) = cos half | sin
    half, bf16-valued.  Channels below rot_dim: fp32 products rounded
    separately, then one rounded sum / difference, then bf16; half-split
    pairing (lo, lo + rot/2) when ``neox`` else interleaved (dd, dd ^ 1).
    slot < 0 skips the row."""
    key = np.asarray(key, np.float32)
    val = np.asarray(val, np.float32)
    half = rot_dim // 2
    for r in range(key.shape[0]):
        s = int(slot_mapping[r])
        if s < 0:
            continue
        blk, t = s // page, s % page
        v_cache[blk, t] = val[r]
        out = key[r].copy()
        if cos_sin is not None:
            c = np.asarray(cos_sin[int(positions[r]), :half], np.float32)
            sn = np.asarray(cos_sin[int(positions[r]), half:rot_dim], np.float32)
            x = key[r]
            if neox:
                e, o = x[:, :half], x[:, half:rot_dim]
                lo = (e * c).astype(np.float32) - (o * sn).astype(np.float32)
                hi = (o * c).astype(np.float32) + (e * sn).astype(np.float32)
                out[:, :half], out[:, half:rot_dim] = lo, hi
            else:
                ev, od = x[:, 0:rot_dim:2], x[:, 1:rot_dim:2]
                out[:, 0:rot_dim:2] = (ev * c).astype(np.float32) - \
                    (od * sn).astype(np.float32)
                out[:, 1:rot_dim:2] = (od * c).astype(np.float32) + \
                    (ev * sn).astype(np.float32)
            out[:, :rot_dim] = bf16_round(out[:, :rot_dim])
        k_cache[blk, t] = out


# --------------------------------------------------------------------------- #
# MLA (latent KV) path                                                         #
# --------------------------------------------------------------------------- #
def mla_page_basis(blk, r):
    """Top-r left singular basis of each latent page from its page x page
    Gram; modes under sigma_1*sqrt(eps) are zeroed.
    selection/mla_select.py:26-51."""
    blk = np.asarray(blk, dtype=np.float32)
    Gm = np.matmul(blk, blk.transpose(0, 2, 1))
    lam, W = np.linalg.eigh(Gm)
    lam = lam[:, -r:][:, ::-1].astype(np.float32)
    W = W[:, :, -r:][:, :, ::-1].astype(np.float32)
    sig = np.sqrt(np.maximum(lam, 0))
    tol = sig[:, :1] * np.float32(math.sqrt(np.finfo(np.float32).eps))
    return W, np.where(sig > tol, sig, np.float32(0))


def mla_build_page_factors(kv_c, n_cache, page, rank, rpad=16):
    """Rank-``rank`` factors Lf (n_cache,page,rpad), Rf (n_cache,rpad,Lkv) of
    each full prompt page of the latent.  selection/mla_select.py:69-108."""
    kv_c = np.asarray(kv_c, dtype=np.float32)
    Lkv = kv_c.shape[1]
    Lf = np.zeros((max(n_cache, 0), page, rpad), dtype=np.float32)
    Rf = np.zeros((max(n_cache, 0), rpad, Lkv), dtype=np.float32)
    if n_cache <= 0:
        return Lf, Rf
    blk = kv_c[:n_cache * page].reshape(n_cache, page, Lkv)
    r = min(rank, page, Lkv, rpad)
    W, sig = mla_page_basis(blk, r)
    Lf[:, :, :r] = W * sig[:, None, :]
    inv = np.where(sig > 0, 1.0 / np.maximum(sig, np.finfo(np.float32).tiny),
                   0.0).astype(np.float32)
    Rf[:, :r, :] = np.matmul(W.transpose(0, 2, 1), blk) * inv[:, :, None]
    return Lf, Rf


def mla_page_score(q_c, q_rope, Lf, Rf, k_rope, valid, scale):
    """score[p] = max_h max_{t<valid[p]} ((q_c[h].Rf^T).Lf^T + q_rope[h].k_rope^T)[t]*scale
    selection/mla_score_torch.py:27-48 with C8 = Lf @ Rf
    (selection/mla_score_triton.py:98-151 evaluates the same factored form)."""
    q_c = np.asarray(q_c, dtype=np.float32)
    q_rope = np.asarray(q_rope, dtype=np.float32)
    a = np.einsum("hD,prD->phr", q_c, Rf, optimize=True)         # (P,H,rpad)
    s_nope = np.einsum("phr,ptr->hpt", a, Lf, optimize=True)
    s_rope = np.einsum("hd,ptd->hpt", q_rope, k_rope, optimize=True)
    approx = (s_nope + s_rope) * np.float32(scale)
    page = Lf.shape[1]
    vmask = np.arange(page)[None, :] < np.asarray(valid)[:, None]
    approx = np.where(vmask[None], approx, np.float32(-1e30))
    return approx.max(2).max(0).astype(np.float32)


def mla_topb_middle(page_score, budget_pages, n_sink, n_recent):
    """Keep mask: all pages if P <= budget; else sink + recent forced and the
    top-scored middle pages fill the rest of the budget.
    selection/mla_score_torch.py:51-73."""
    P = page_score.shape[0]
    keep = np.zeros(P, dtype=bool)
    if P <= budget_pages:
        keep[:] = True
        return keep
    forced = set(range(min(n_sink, P))) | set(range(max(0, P - n_recent), P))
    for p in forced:
        keep[p] = True
    n_mid = budget_pages - len(forced)
    if n_mid > 0:
        cand = np.ones(P, dtype=bool)
        for p in forced:
            cand[p] = False
        idx = np.nonzero(cand)[0]
        if idx.size:
            k = min(n_mid, idx.size)
            order = np.argsort(-page_score[idx], kind="stable")[:k]
            keep[idx[order]] = True
    return keep


def mla_decode_row(q, cache, bt_row, L, keep_idx, scale, Lkv):
    """Attention of one decode row over the kept pages of the latent cache.
    q (H, width), cache (NB, page, width).  Returns o (H, Lkv), lse (H,).
    backend/mla_attn.py:178-201."""
    page = cache.shape[1]
    q = np.asarray(q, dtype=np.float32)
    blks = np.asarray(bt_row)[keep_idx].astype(np.int64)
    sel = cache[blks].reshape(-1, cache.shape[2]).astype(np.float32)
    pos = (np.asarray(keep_idx)[:, None] * page
           + np.arange(page)[None, :]).reshape(-1)
    ok = pos < L
    scores = (q @ sel.T) * np.float32(scale)
    scores = np.where(ok[None, :], scores, np.float32(-1e30))
    mx = scores.max(-1, keepdims=True)
    p = np.exp(scores - mx)
    den = p.sum(-1, keepdims=True)
    o = (p / den) @ sel[:, :Lkv]
    return o.astype(np.float32), (mx + np.log(den))[:, 0].astype(np.float32)


def mla_decode_step(q, cache, block_table, seq_lens, scale, *, Lkv, rank,
                    budget_pages, sink, window):
    """Full MLA step for a batch: factors over the full prompt pages, factored
    score, top-b keep, attention.  backend/mla_attn.py:86-210."""
    q = np.asarray(q, dtype=np.float32)
    B, H, W = q.shape
    page = cache.shape[1]
    o = np.zeros((B, H, Lkv), dtype=np.float32)
    lse = np.zeros((B, H), dtype=np.float32)
    keeps, scores = [], []
    for bi in range(B):
        L = int(seq_lens[bi])
        if L <= 0:
            keeps.append(np.zeros(0, dtype=np.int64))
            scores.append(np.zeros(0, dtype=np.float32))
            continue
        n_pages = -(-L // page)
        if n_pages > budget_pages:
            n_cache = L // page
            blks = np.asarray(block_table[bi, :n_pages]).astype(np.int64)
            kvb = cache[blks].reshape(-1, W)[:L].astype(np.float32)
            Lf, Rf = mla_build_page_factors(kvb[:n_cache * page, :Lkv],
                                            n_cache, page, rank)
            kr = kvb[:n_cache * page, Lkv:].reshape(n_cache, page, -1)
            ps = np.full(n_pages, NEG_INF, dtype=np.float32)
            ps[:n_cache] = mla_page_score(
                q[bi, :, :Lkv], q[bi, :, Lkv:], Lf, Rf, kr,
                np.full(n_cache, page), scale)
            idx = np.nonzero(mla_topb_middle(ps, budget_pages, sink,
                                             window))[0]
            scores.append(ps)
        else:
            idx = np.arange(n_pages)
            scores.append(np.zeros(n_pages, dtype=np.float32))
        keeps.append(idx)
        o[bi], lse[bi] = mla_decode_row(q[bi], cache, block_table[bi], L, idx,
                                        scale, Lkv)
    return {"o": o, "lse": lse, "keep": keeps, "page_score": scores}
