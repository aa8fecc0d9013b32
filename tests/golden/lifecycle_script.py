"""A scripted life of the page summaries under continuous batching, shared by
the golden generator (which plays it through the REFERENCE's build functions)
and the GPU test (which plays it through this library's).  Plain torch, no
package imports: both sides load this file by path.

The script exercises every entry point that decides WHICH blocks are rebuilt
(reference ``selection/rki4_build.py:264-364``, ``selection/build.py:372-488``):

  bulk      first decode step of two requests (tags start as NaN)
  delta     a third request arrives + one block of a running request was reused
            with new content in ONE layer only (any-layer-stale rule)
  delta     nothing changed                               -> nothing rebuilt
  tail      one request crossed a page boundary (rows=[0])
  tail      every row (idempotent)
  delta     a row was preempted and came back, rows shuffled -> nothing rebuilt
  delta     a finished request's blocks were handed to a new request
  refresh   single-layer, tag-gated; then forced
  bulk      a padded row whose block ids lie outside the pool (the engine's
            memory-profile pass) builds nothing and faults nothing

``run(api, ...)`` drives an ``api`` object with the five build calls and returns
the list of per-event results (return value and, for delta events, the stale
block list) so that the two sides can be compared event by event.
"""
from __future__ import annotations

import torch

L, N_KV, G, D, PAGE = 2, 2, 4, 128, 16
NB, WIDTH = 64, 24                    # physical blocks, block-table columns
LENS = {"a": 100, "b": 333, "c": 50, "d": 40}


def make_world(seed: int = 4242):
    """K planes (L x (NB, PAGE, N_KV, D) bf16) filled with seeded noise, and a
    block assignment: request a -> 8 blocks, b -> 22, c -> 4 (d takes over
    c's blocks later)."""
    g = torch.Generator().manual_seed(seed)
    K = [torch.randn(NB, PAGE, N_KV, D, generator=g).to(torch.bfloat16)
         for _ in range(L)]
    perm = torch.randperm(NB, generator=g).tolist()
    blocks = {"a": perm[0:8], "b": perm[8:30], "c": perm[30:34]}
    blocks["d"] = list(blocks["c"])
    return K, blocks, g


def table(rows, blocks):
    """(len(rows), WIDTH) int32 block table; rows is a list of request names
    (None = padded row of zeros)."""
    bt = torch.zeros(len(rows), WIDTH, dtype=torch.int32)
    for r, name in enumerate(rows):
        if name is not None:
            b = blocks[name]
            bt[r, :len(b)] = torch.tensor(b, dtype=torch.int32)
    return bt


def lens_of(rows, lens):
    return torch.tensor([lens[n] if n is not None else 0 for n in rows],
                        dtype=torch.int32)


def run(api, K, blocks, g, to_dev=lambda t: t):
    """Play the script.  ``api`` has bulk / delta / tail / refresh with the
    reference's signatures minus the state (bound inside), plus
    ``stale(block_table, lens, n_req, max_fin)`` returning the delta's stale
    block list.  ``K`` tensors are mutated IN PLACE on their own device by
    ``mut(layer, block, rows_slice, values)``."""
    ev = []
    lens = dict(LENS)

    def mut(layer, blk, t0, t1):
        new = torch.randn(t1 - t0, N_KV, D, generator=g).to(torch.bfloat16)
        K[layer][blk, t0:t1] = to_dev(new)

    def max_fin(rows):
        return max(lens[n] // PAGE for n in rows if n is not None)

    # E0 bulk: first decode step of a and b
    rows = ["a", "b"]
    bt, sl = to_dev(table(rows, blocks)), to_dev(lens_of(rows, lens))
    ev.append(("bulk", api.bulk(bt, sl, 2, max_fin(rows)), None))

    # E1 delta: c arrives; block b[3] reused with new content in layer 0 only
    mut(0, blocks["b"][3], 0, PAGE)
    rows = ["a", "b", "c"]
    bt, sl = to_dev(table(rows, blocks)), to_dev(lens_of(rows, lens))
    st = api.stale(bt, sl, 3, max_fin(rows))
    ev.append(("delta", api.delta(bt, sl, 3, max_fin(rows)), st))

    # E2 delta: nothing changed
    st = api.stale(bt, sl, 3, max_fin(rows))
    ev.append(("delta", api.delta(bt, sl, 3, max_fin(rows)), st))

    # E3 tail: a decodes 13 tokens (100 -> 113 settled): page 6 (tokens 96..111)
    # is complete; the rows live in block a[6] (and a[7] for token 112)
    for l in range(L):
        mut(l, blocks["a"][6], 100 - 96, PAGE)
        mut(l, blocks["a"][7], 0, 1)
    lens["a"] = 113
    sl = to_dev(lens_of(rows, lens))
    ev.append(("tail", api.tail(bt, sl, 3, to_dev(torch.tensor([0]))), None))

    # E4 tail over every row: idempotent
    ev.append(("tail", api.tail(bt, sl, 3, None), None))

    # E5 delta: b was preempted and resumed with the same blocks, rows shuffled
    rows = ["a", "c", "b"]
    bt, sl = to_dev(table(rows, blocks)), to_dev(lens_of(rows, lens))
    st = api.stale(bt, sl, 3, max_fin(rows))
    ev.append(("delta", api.delta(bt, sl, 3, max_fin(rows)), st))

    # E6 delta: c finished, request d got c's blocks and prefilled 40 tokens
    for l in range(L):
        for pg in range(3):
            mut(l, blocks["d"][pg], 0, PAGE)
    rows = ["a", "d", "b"]
    bt, sl = to_dev(table(rows, blocks)), to_dev(lens_of(rows, lens))
    st = api.stale(bt, sl, 3, max_fin(rows))
    ev.append(("delta", api.delta(bt, sl, 3, max_fin(rows)), st))

    # E7 refresh: the last token of page a[2] changes in layer 1 only
    mut(1, blocks["a"][2], PAGE - 1, PAGE)
    ev.append(("refresh", api.refresh(1, bt, sl, 3, False), None))
    ev.append(("refresh", api.refresh(0, bt, sl, 3, False), None))
    one_bt, one_sl = bt[:1].contiguous(), sl[:1].contiguous()
    ev.append(("refresh", api.refresh(0, one_bt, one_sl, 1, True), None))

    # E8 bulk with a padded row that carries block ids outside the pool
    bt4 = table(rows + [None], blocks)
    bt4[3, :2] = torch.tensor([NB + 7, -3], dtype=torch.int32)
    sl4 = lens_of(rows + [None], lens)
    sl4[3] = 2 * PAGE
    ev.append(("bulk_oob", api.bulk(to_dev(bt4), to_dev(sl4), 4,
                                    max_fin(rows)), None))
    return ev, rows, lens
