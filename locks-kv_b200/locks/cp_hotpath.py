"""Context-parallel driver of the decode hot path: ONE long sequence whose pages
are spread over the ranks of a process group (one process per GPU).

Rank k holds the contiguous page range ``[p0, p1)`` -- its K/V pages and their
summaries -- and runs the same kernels as the single-GPU path on that slice.
Per layer three small exchanges make the result equal to the single-GPU one:

  1. all-reduce(max) of the per-head score maxima the scorer published (the
     default GQA combine normalises by the maximum over ALL pages);
  2. all-gather of every rank's best ``b`` (score, page) candidates -- the local
     selector run with the global budget -- after which every rank applies the
     same exact-b rule (score descending, page ascending) to the union and keeps
     its own members plus its sink / recent-window pages;
  3. all-gather of the split-K partials (m, l, acc) of the pages each rank
     attended, merged by ``locks_merge_gathered``.

The reference has no distributed code; the page rules are the reference's
(``selection/select.py:28-58``, ``:183-222``), applied to global page numbers.

Transports.  ``"fused"`` (default): the exchanges happen INSIDE the selector and
the decode kernel -- they store their words into every peer's link region over
NVLink and poll their own region (``locks_topb_select_cp``,
``locks_decode_fused_cp``), so a layer is three launches (score, select, decode)
at any number of GPUs, chained by programmatic dependent launch as on one GPU.
``"peer"``: one exchange kernel per exchange between the single-GPU kernels
(ten launches per layer); ``"nccl"``: library collectives -- both kept as the
baselines the fused path is measured against.  Remote data always lands in
local memory before a kernel of this library reads it.  The whole step has
fixed shapes and no host synchronisation, so it can be captured in a CUDA graph.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist

from . import _cabi
from .attention import ResidentVSource
from .attention.decode import _kv_args
from .config import LocksConfig
from .selection import Rki4State, rki4_build_bulk, rki4_score_only
from .selection.select import nrmtopb_select

_SIGN = -(1 << 31)          # int32 view of 0x80000000
_BIG_PAGE = (1 << 31) - 1


def global_page_params(seq_len: int, page: int, cfg: LocksConfig):
    """(n_pages, n_sel_hi, b) of the whole sequence, as ``derive_page_params``
    computes them for a request (reference ``selection/select.py:28-58``)."""
    npg = -(-int(seq_len) // page)
    nsh = npg - cfg.window_pages
    s = nsh - cfg.sink_pages
    if cfg.budget_pages:
        b = max(min(int(cfg.budget_pages), max(s, 1)), 1)
    else:
        frac = cfg.budget if cfg.budget is not None else 0.1
        b = min(max(int(math.ceil(s * frac)), 1), max(s, 1))
    return npg, nsh, b


class ContextParallelHotPath:
    """Decode steps of one sequence over the ranks of ``group``.

    kv_caches: per layer, this rank's paged cache ``(NB, 2, page, n_kv, d)``;
    block_table: ``(1, p1 - p0)`` int32, local page j -> local block.
    """

    def __init__(self, kv_caches: List[torch.Tensor], block_table: torch.Tensor,
                 *, seq_len: int, p0: int, p1: int, n_kv: int, G: int,
                 scale: float, cfg: LocksConfig, group=None,
                 split: Optional[int] = None, transport: str = "fused",
                 loopback: bool = False):
        """``loopback``: with ONE rank, still run the in-kernel exchanges, against
        the rank's own link region (tests, and timing the exchange code without a
        peer); by default a single rank has nothing to exchange and runs the
        plain single-GPU kernels."""
        dev = kv_caches[0].device
        self.device, self.cfg, self.group = dev, cfg, group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.kv_caches, self.block_table = kv_caches, block_table
        NB, _, page, _, d = kv_caches[0].shape
        self.page, self.d, self.n_kv, self.G = int(page), int(d), n_kv, G
        self.scale = float(scale)
        self.p0, self.p1 = int(p0), int(p1)
        n_loc = self.p1 - self.p0
        assert n_loc >= 1 and block_table.shape == (1, n_loc)
        npg, nsh, b = global_page_params(seq_len, self.page, cfg)
        assert self.p1 <= npg
        self.npg, self.nsh, self.b = npg, nsh, b
        # the slice seen as a sequence of its own: local page j = global p0 + j
        self.sink_loc = min(max(cfg.sink_pages - self.p0, 0), n_loc)
        self.nsh_loc = min(max(nsh - self.p0, 0), n_loc)
        tok_loc = min(int(seq_len) - self.p0 * self.page, n_loc * self.page)
        self.seq_lens = torch.tensor([tok_loc], dtype=torch.int32, device=dev)
        L = len(kv_caches)
        st = Rki4State(dev, num_layers=L, num_blocks=int(NB), n_kv=n_kv, G=G,
                       head_dim=int(d), page=int(page), max_reqs=1,
                       max_pages=n_loc, budget_pages=b,
                       sink_pages=self.sink_loc,
                       window_pages=max(cfg.window_pages, 1),
                       combine=cfg.quad_combine, zsplit=cfg.rki4_zsplit)
        assert st.combine == "nrm", "context parallel implements the nrm combine"
        st.scale = self.scale
        st.n_pages.fill_(n_loc)
        st.n_sel_hi.fill_(self.nsh_loc)
        st.b_fix.fill_(b)
        self.st = st
        self.K_layers = [c[:, 0] for c in kv_caches]
        self.vsources = [ResidentVSource(c) for c in kv_caches]
        H = n_kv * G
        self.q = torch.zeros(L, 1, H, d, device=dev, dtype=torch.bfloat16)
        self.out = torch.zeros(L, 1, H, d, device=dev, dtype=torch.bfloat16)
        # most pages a rank can end up attending: b selected + sink + window
        self.cap = min(n_loc, b + cfg.sink_pages + cfg.window_pages + 1)
        # split-K partials of all ranks: [world][m | l | acc], this rank writes
        # (and all-gathers in place) its own set
        # a rank attends about (b + sink + window) / world pages per kv head: one
        # CTA (8 warps) per head is enough from 4 ranks on, and every split less
        # halves the partial set that has to travel
        if split is None:
            split = 1 if self.world >= 4 else 2
        self.split = int(split)
        n_ml = n_kv * self.split * G
        self.n_ml = n_ml
        self.pack_len = (n_ml * (2 + d) + 3) // 4 * 4
        self.packs = torch.zeros(self.world, self.pack_len, device=dev,
                                 dtype=torch.float32)
        # (the peer transport gathers from a buffer of its own into `packs`)
        self.pack_mine = torch.zeros(self.pack_len, device=dev, dtype=torch.float32)
        mine = self.pack_mine if (transport == "peer" and self.world > 1) \
            else self.packs[self.rank]
        self.m_part = mine[:n_ml]
        self.l_part = mine[n_ml:2 * n_ml]
        self.acc_part = mine[2 * n_ml:2 * n_ml + n_ml * d]
        cand_len = (2 * n_kv * self.cap + 3) // 4 * 4     # 16-byte multiple
        self.cand_flat = torch.zeros(self.world, cand_len, device=dev,
                                     dtype=torch.float32)
        self.cand = self.cand_flat
        self.cand_mine = torch.zeros(cand_len, device=dev, dtype=torch.float32)
        self.cand_stride = cand_len
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        # transport of the three exchanges: "peer" = one fused kernel per rank
        # over NVLink peer memory (locks_cp_exchange), "nccl" = library
        # collectives (kept as the baseline the fused kernel is measured against)
        assert transport in ("fused", "peer", "nccl")
        self.transport = transport if (self.world > 1 or
                                       (transport == "fused" and loopback)) \
            else "none"
        self.hm_pad = None
        self.link = None
        if self.transport == "fused":
            from .peer import CpLinkRegion
            # candidate slots per rank: the same on every rank (the regions
            # share one layout), enough for the budget plus the forced pages
            cap_link = b + cfg.sink_pages + cfg.window_pages + 1
            self.link = CpLinkRegion(n_kv=n_kv, G=G, cap=cap_link, n_layers=L,
                                     group=group)
            self._links = [self.link.link(l, p0=self.p0, b_global=b,
                                          sink_loc=self.sink_loc,
                                          nsh_loc=self.nsh_loc)
                           for l in range(L)]
        if self.transport == "peer":
            from .peer import PeerExchange
            # keys and candidates (a few KB): flag-in-packet transport; partial
            # sets: the same up to 20 KB (measured cross-over), fenced bulk
            # transport beyond; one region per payload family
            self.px = PeerExchange(self.pack_len * 4, group,
                                   packets=self.pack_len * 4 <= 20 * 1024)
            self.px_small = PeerExchange(max(self.cand[0].numel() * 4, 64 * 4),
                                         group, packets=True)
            # the keys padded to a multiple of 16 bytes
            n_hm = (st.hmax.numel() + 3) // 4 * 4
            self.hm_pad = torch.zeros(n_hm, device=dev, dtype=torch.int32)

    # ---- summaries ---------------------------------------------------------
    def build_all(self) -> int:
        settled = self.seq_lens - 1 if self.p1 == self.npg else self.seq_lens
        max_fin = int(settled.max().item()) // self.page
        return rki4_build_bulk(self.st, self.K_layers, self.block_table, settled,
                               1, max_fin)

    # ---- the three exchanges -------------------------------------------------
    def _exchange_hmax(self) -> None:
        """Keys are order-preserving as UNSIGNED ints; flipping the top bit
        makes the int32 maximum agree.  0 ("no page scored here") loses."""
        if self.world == 1:
            return
        hm = self.st.hmax
        if self.transport == "peer":
            n = hm.numel()
            if self.hm_pad.numel() == n:
                self.px_small.all_max_u32(hm.view(-1), self.st.status)
            else:
                self.hm_pad[:n].copy_(hm.view(-1))
                self.px_small.all_max_u32(self.hm_pad, self.st.status)
                hm.view(-1).copy_(self.hm_pad[:n])
            return
        hm.bitwise_xor_(_SIGN)
        dist.all_reduce(hm, op=dist.ReduceOp.MAX, group=self.group)
        hm.bitwise_xor_(_SIGN)

    def _exchange_candidates(self) -> None:
        """Local top-b list -> global exact-b cut -> this rank's final list."""
        st, cap = self.st, self.cap
        mine = self.cand_mine if self.transport == "peer" else self.cand[self.rank]
        _cabi.call("locks_cp_pack", _cabi.ptr(st.page_table), _cabi.ptr(st.score),
                   _cabi.ptr(mine), int(self.n_kv), int(st.max_pages), int(cap),
                   int(self.sink_loc), int(self.nsh_loc), int(self.p0),
                   _cabi.stream())
        if self.transport == "peer":
            self.px_small.all_gather(self.cand_mine, self.cand, self.st.status)
        elif self.world > 1:
            dist.all_gather_into_tensor(self.cand.view(-1), mine.reshape(-1),
                                        group=self.group)
        _cabi.call("locks_cp_select", _cabi.ptr(self.cand),
                   int(self.cand_stride), _cabi.ptr(st.page_table), _cabi.ptr(st.page_cnt),
                   int(self.world), int(self.rank), int(self.n_kv), int(cap),
                   int(st.max_pages), int(self.b), int(self.sink_loc),
                   int(self.nsh_loc), _cabi.stream())

    def _decode_and_merge(self, l: int) -> None:
        st = self.st
        q = self.q[l]
        k, v = _kv_args(self.kv_caches[l], self.vsources[l])
        self.l_part.zero_()                  # splits without pages must read l = 0
        _cabi.call("locks_decode_split", _cabi.ptr(q), q.stride(0), _cabi.ptr(k),
                   _cabi.ptr(v), k.stride(0), k.stride(1), k.stride(2),
                   _cabi.ptr(self.block_table), self.block_table.stride(0),
                   _cabi.ptr(st.page_table), _cabi.ptr(st.page_cnt),
                   _cabi.ptr(self.seq_lens), _cabi.ptr(self.m_part),
                   _cabi.ptr(self.l_part), _cabi.ptr(self.acc_part), 1,
                   int(self.n_kv), int(self.G), int(self.d), int(self.page),
                   int(st.max_pages), int(self.split), 1, float(self.scale),
                   _cabi.ptr(st.status), _cabi.stream())
        if self.transport == "peer":
            self.px.all_gather(self.pack_mine, self.packs, self.st.status)
        elif self.world > 1:
            dist.all_gather_into_tensor(self.packs.view(-1), self.packs[self.rank],
                                        group=self.group)
        out = self.out[l]
        _cabi.call("locks_merge_gathered", _cabi.ptr(self.packs),
                   int(self.pack_len), int(self.world), _cabi.ptr(out),
                   out.stride(0), 1, int(self.n_kv), int(self.G), int(self.d),
                   int(self.split), _cabi.stream())

    # ---- the fused path: exchanges inside the selector and the decode -------
    def _layers_fused(self) -> None:
        import ctypes
        st = self.st
        self.link.begin_step()
        for l in range(len(self.kv_caches)):
            q = self.q[l]
            link = ctypes.cast(ctypes.pointer(self._links[l]), ctypes.c_void_p)
            rki4_score_only(st, l, q, self.block_table, self.seq_lens, 1,
                            self.scale)
            _cabi.call("locks_topb_select_cp", _cabi.ptr(st.score_h),
                       _cabi.ptr(st.score), _cabi.ptr(st.hmax),
                       _cabi.ptr(st.n_pages), _cabi.ptr(st.n_sel_hi),
                       _cabi.ptr(st.b_fix), _cabi.ptr(st.page_table),
                       _cabi.ptr(st.page_cnt), int(self.n_kv), int(self.G),
                       int(st.max_pages), int(st.sink_pages), link,
                       _cabi.ptr(st.status), _cabi.stream())
            k, v = _kv_args(self.kv_caches[l], self.vsources[l])
            out = self.out[l]
            _cabi.call("locks_decode_fused_cp", _cabi.ptr(q), q.stride(0),
                       _cabi.ptr(k), _cabi.ptr(v), k.stride(0), k.stride(1),
                       k.stride(2), _cabi.ptr(self.block_table),
                       self.block_table.stride(0), _cabi.ptr(st.page_table),
                       _cabi.ptr(st.page_cnt), _cabi.ptr(self.seq_lens),
                       _cabi.ptr(out), out.stride(0), int(self.n_kv), int(self.G),
                       int(self.d), int(self.page), int(st.max_pages),
                       float(self.scale), link, _cabi.ptr(st.status),
                       _cabi.stream())

    def resync(self) -> None:
        """After ``st.status`` reported a wait that ran out: bring the ranks'
        link regions and step counters back in line (collective, host-side)."""
        if self.link is not None:
            self.link.resync()
        self.st.status.zero_()

    # ---- one decode step ---------------------------------------------------
    def _layers(self) -> None:
        if self.transport == "fused":
            self._layers_fused()
            return
        st = self.st
        if self.world == 1:
            # one rank holds the whole sequence: the single-GPU kernels
            from .attention import sparse_paged_decode_fused
            for l in range(len(self.kv_caches)):
                rki4_score_only(st, l, self.q[l], self.block_table, self.seq_lens,
                                1, self.scale)
                nrmtopb_select(st, 1, has_hmax=True)
                sparse_paged_decode_fused(self.q[l], self.kv_caches[l],
                                          self.block_table, self.seq_lens, st,
                                          self.out[l], self.vsources[l],
                                          scale=self.scale)
            return
        for l in range(len(self.kv_caches)):
            rki4_score_only(st, l, self.q[l], self.block_table, self.seq_lens, 1,
                            self.scale)
            self._exchange_hmax()
            nrmtopb_select(st, 1, has_hmax=True)
            if self.nsh_loc == 0:
                st.hmax.zero_()      # nothing scored here: the selector did not re-arm it
            self._exchange_candidates()
            self._decode_and_merge(l)

    def step_eager(self) -> torch.Tensor:
        self._layers()
        return self.out

    def capture(self) -> None:
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._layers()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._layers()
        self.graph = g

    def step(self) -> torch.Tensor:
        if self.graph is None:
            self.capture()
        self.graph.replay()
        return self.out


def check_against_single_gpu(*, seq_len: int = 40005, n_layers: int = 3,
                             transport: str = "fused", group=None, seed: int = 11):
    """Self-check of a context-parallel set-up, run by ALL ranks of ``group``:
    one seeded sequence (2 KV heads x 16 query heads, budget 64 + 1 sink + 8
    recent pages) is decoded context-parallel -- eagerly and as a replayed graph
    -- and rank 0 compares it with the single-GPU hot path on the whole
    sequence: the union of the ranks' attended pages must EQUAL the single-GPU
    page table of the last layer, the outputs must agree within the decode
    tolerance (2e-2; bf16 outputs, different merge order), eager and graph
    outputs must be identical and no wait may have run out.
    Returns ``(ok, max_abs_err, messages)`` (the same on every rank)."""
    import math
    from . import synth
    from .hotpath import HotPath
    from .parallel import partition_pages
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    dev = torch.device("cuda", torch.cuda.current_device())
    shape = synth.GqaShape(n_layers=n_layers, n_kv=2, G=16, d=128, page=16,
                           budget_pages=64, sink_pages=1, window_pages=8,
                           n_needles=6, n_outlier=4)
    cfg = LocksConfig(budget_pages=shape.budget_pages, sink_pages=shape.sink_pages,
                      window_pages=shape.window_pages)
    scale = 1.0 / math.sqrt(shape.d)
    npg = -(-seq_len // shape.page)
    p0, p1 = partition_pages(npg, world)[rank]
    caches, q, bt = synth.make_gqa_shard(seed, shape, seq_len, p0, p1, device=dev)
    cp = ContextParallelHotPath(caches, bt, seq_len=seq_len, p0=p0, p1=p1,
                                n_kv=shape.n_kv, G=shape.G, scale=scale, cfg=cfg,
                                group=group, transport=transport)
    cp.build_all()
    cp.q.copy_(q)
    out_eager = cp.step_eager().clone()
    torch.cuda.synchronize()
    cnt = cp.st.page_cnt[0].tolist()
    mine = [(cp.st.page_table[0, kh, :cnt[kh]] + p0).tolist()
            for kh in range(shape.n_kv)]
    gathered = [mine]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, mine, group=group)
    out_graph = cp.step().clone()
    cp.step()
    torch.cuda.synchronize()
    msgs, ok, err = [], True, 0.0
    if not torch.equal(out_graph, cp.out):
        msgs.append(f"[rank {rank}] graph replay is not repeatable"); ok = False
    if (out_graph.float() - out_eager.float()).abs().max().item() > 0:
        msgs.append(f"[rank {rank}] graph and eager outputs differ"); ok = False
    status = int(cp.st.status.item())
    if status:
        msgs.append(f"[rank {rank}] kernel status word {status}"); ok = False
    if rank == 0:
        fc, fq, fbt = synth.make_gqa_shard(seed, shape, seq_len, 0, npg, device=dev)
        sl = torch.tensor([seq_len], dtype=torch.int32, device=dev)
        hp = HotPath(fc, fbt, sl, n_kv=shape.n_kv, G=shape.G, scale=scale, cfg=cfg)
        hp.build_all(); hp.derive(); hp.q.copy_(fq)
        ref = hp.step_eager().clone()
        torch.cuda.synchronize()
        rc = hp.st.page_cnt[0].tolist()
        for kh in range(shape.n_kv):
            want = hp.st.page_table[0, kh, :rc[kh]].tolist()
            got = sorted(p for r in range(world) for p in gathered[r][kh])
            if got != want:
                extra = sorted(set(got) - set(want))[:5]
                miss = sorted(set(want) - set(got))[:5]
                msgs.append(f"kv head {kh}: page sets differ ({len(got)} vs "
                            f"{len(want)}; extra {extra}, missing {miss})")
                ok = False
        err = (out_eager.float() - ref.float()).abs().max().item()
        if not err <= 2e-2:
            msgs.append(f"max |out - single GPU| = {err:.3e}"); ok = False
        del hp, fc
    res = [ok, err, msgs]
    if world > 1:
        flag = torch.tensor([0 if ok else 1], device=dev)
        dist.all_reduce(flag, group=group)
        res[0] = int(flag.item()) == 0
        box = [res if rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=group)
        res = [res[0], box[0][1], box[0][2] + ([] if rank == 0 else msgs)]
    if cp.link is not None:
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=group)       # nobody closes while a peer still stores
        cp.link.close()
    return tuple(res)
