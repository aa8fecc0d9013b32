"""Multi-GPU partitioning of the decode hot path (one process per GPU).

Two schemes, both new (the reference has no distributed code):

* **sequence sharding** -- ragged batches: requests are independent, so each
  rank owns whole sequences (:func:`shard_sequences`, greedy balance on the
  algorithmic bytes of a step); there is no data-path collective.

* **context parallel** -- one long sequence: rank k owns the contiguous page
  range :func:`partition_pages` gives it (its K/V pages and their summaries).
  Per layer three small exchanges make the result EQUAL to the single-GPU path:
    1. all-reduce(max) of the per-head score maxima -- the default GQA combine
       ``sum_g exp(S[g,p] - max_p S[g,p])`` needs the max over ALL pages;
    2. all-gather of each rank's best ``b`` (score, page) candidates; every rank
       then applies the same exact-b rule (``> tau``, then ``== tau`` by
       ascending page) to the union, so all ranks agree on the global set;
    3. all-gather of the split-K partials (m, l, acc) of the pages each rank
       attended, merged with the usual log-sum-exp weights.
  Collectives go through ``torch.distributed`` (NCCL on GPUs, gloo in the CPU
  tests); remote data always lands in local memory before a kernel reads it.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

REC_BYTES, PAGE_KV_BYTES = 818, 8192


def partition_pages(n_pages: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous, near-equal page ranges ``[(p0, p1), ...]`` per rank."""
    return [((n_pages * k) // world, (n_pages * (k + 1)) // world)
            for k in range(world)]


def step_bytes(seq_len: int, budget_pages: int, sink: int, window: int,
               page: int = 16) -> int:
    """Algorithmic bytes one (layer, kv-head) of a request costs per step."""
    npg = -(-seq_len // page)
    nsh = max(npg - window, 0)
    att = min(budget_pages, max(nsh - sink, 0)) + min(sink, npg) + min(window, npg)
    return nsh * REC_BYTES + att * PAGE_KV_BYTES


def shard_sequences(seq_lens: Sequence[int], budgets: Sequence[int], world: int,
                    sink: int = 1, window: int = 8) -> List[List[int]]:
    """Greedy longest-first balance of requests over ranks by step bytes."""
    cost = [step_bytes(s, b, sink, window) for s, b in zip(seq_lens, budgets)]
    order = sorted(range(len(cost)), key=lambda i: -cost[i])
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        k = min(range(world), key=lambda r: load[r])
        out[k].append(i)
        load[k] += cost[i]
    return [sorted(x) for x in out]


# --------------------------------------------------------------------------- #
# context parallel: the three exchanges                                        #
# --------------------------------------------------------------------------- #
def cp_allreduce_max(x: torch.Tensor, group=None) -> torch.Tensor:
    """Exchange 1: element-wise max over ranks (per-head score maxima)."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(x, op=dist.ReduceOp.MAX, group=group)
    return x


def local_candidates(score: torch.Tensor, p0: int, lo: int, hi: int, b: int):
    """Best ``b`` selectable pages of this rank's slice.

    score: (n_kv, n_local) combined scores of pages [p0, p0+n_local); only
    global pages in [lo, hi) are selectable.  Returns (scores (n_kv,b),
    pages (n_kv,b) int64 global ids), padded with (-inf, big id).  Ties are
    taken lowest page first, which is what the global rule needs."""
    n_kv, n_loc = score.shape
    ids = torch.arange(p0, p0 + n_loc, device=score.device)
    sel = (ids >= lo) & (ids < hi)
    s = torch.where(sel[None, :], score, torch.full_like(score, float("-inf")))
    k = min(b, n_loc)
    # stable descending sort keeps ascending page order among equal scores
    order = torch.sort(s, dim=1, descending=True, stable=True).indices[:, :k]
    cs = torch.gather(s, 1, order)
    cp = ids[order]
    if k < b:
        pad = b - k
        cs = torch.cat([cs, cs.new_full((n_kv, pad), float("-inf"))], 1)
        cp = torch.cat([cp, cp.new_full((n_kv, pad), 1 << 40)], 1)
    cp = torch.where(torch.isneginf(cs), torch.full_like(cp, 1 << 40), cp)
    return cs.contiguous(), cp.contiguous()


def global_select(cand_s: torch.Tensor, cand_p: torch.Tensor, b: int):
    """Exact-b rule on the union of all ranks' candidates.

    cand_s/cand_p: (n_kv, world*b).  Keeps the ``b`` best by (score desc, page
    asc) -- identical to "> tau, then == tau in ascending page order until b".
    Returns a bool mask over the candidates."""
    # order by page asc first, then a stable sort by score desc
    o1 = torch.sort(cand_p, dim=1, stable=True).indices
    s1 = torch.gather(cand_s, 1, o1)
    o2 = torch.sort(s1, dim=1, descending=True, stable=True).indices
    top = torch.gather(o1, 1, o2)[:, :b]
    keep = torch.zeros_like(cand_s, dtype=torch.bool)
    keep.scatter_(1, top, True)
    return keep & ~torch.isneginf(cand_s)


def cp_select(score: torch.Tensor, p0: int, n_pages: int, n_sel_hi: int, b: int,
              sink: int, group=None) -> List[torch.Tensor]:
    """Exchange 2.  Returns, per kv-head, the ascending GLOBAL ids of the pages
    of THIS rank's slice that the single-GPU selector would keep (selected
    pages, sink pages, recent-window pages)."""
    n_kv, n_loc = score.shape
    p1 = p0 + n_loc
    lo, hi = min(sink, n_pages), max(min(n_sel_hi, n_pages), min(sink, n_pages))
    ids = torch.arange(p0, p1, device=score.device)
    forced = (ids < lo) | ((ids >= hi) & (ids < n_pages))
    L = hi - lo
    if (n_sel_hi - sink) <= 1 or L <= 1 or b >= L:
        keep_loc = (forced | ((ids >= lo) & (ids < hi)))[None, :].expand(n_kv, -1)
    else:
        cs, cp = local_candidates(score, p0, lo, hi, b)
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if world > 1:
            gs = [torch.empty_like(cs) for _ in range(world)]
            gp = [torch.empty_like(cp) for _ in range(world)]
            dist.all_gather(gs, cs, group=group)
            dist.all_gather(gp, cp, group=group)
            all_s, all_p = torch.cat(gs, 1), torch.cat(gp, 1)
        else:
            all_s, all_p = cs, cp
        keep = global_select(all_s, all_p, b)
        keep_loc = forced[None, :].expand(n_kv, -1).clone()
        for kh in range(n_kv):
            pages = all_p[kh][keep[kh]]
            mine = pages[(pages >= p0) & (pages < p1)] - p0
            keep_loc[kh, mine] = True
    return [ids[keep_loc[kh]] for kh in range(n_kv)]


def merge_partials(m: torch.Tensor, l: torch.Tensor, acc: torch.Tensor):
    """Log-sum-exp merge over dim 0 (the partial index): m, l (S, ...),
    acc (S, ..., d) -> out (..., d).  Empty partials carry l == 0."""
    M = m.max(dim=0).values
    w = torch.where(l > 0, torch.exp(m - M), torch.zeros_like(m))
    den = (w * l).sum(0)
    num = (w[..., None] * acc).sum(0)
    return torch.where(den[..., None] > 0, num / den[..., None].clamp_min(1e-38),
                       torch.zeros_like(num))


def cp_merge(m: torch.Tensor, l: torch.Tensor, acc: torch.Tensor, group=None):
    """Exchange 3: all-gather every rank's partials (S, H), (S, H), (S, H, d)
    and merge them; every rank gets the full output (H, d)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world > 1:
        pack = torch.cat([m[..., None], l[..., None], acc], dim=-1).contiguous()
        bufs = [torch.empty_like(pack) for _ in range(world)]
        dist.all_gather(bufs, pack, group=group)
        pack = torch.cat(bufs, 0)
        m, l, acc = pack[..., 0], pack[..., 1], pack[..., 2:]
    return merge_partials(m, l, acc)
