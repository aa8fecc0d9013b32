"""V tier: V in pinned host memory, a bounded staging buffer in device memory.

The memory play of the reference's ``mem-v`` variant (``tier/pool.py:104-184``
pool, ``tier/dma.py:77-140`` copy engine, ``tier/decode_mem.py:168-180`` address
select in the decode, invariants ``tier/__init__.py:11-17``), laid out for one
GPU with a fast host link:

* the V of EVERY physical block lives in a pinned host pool (``PinnedHostVSource``:
  the K plane's strides, so the KV-write kernels store new V rows through the
  same pointer -- write-through, nothing in device memory is ever dirty);
* per layer a staging buffer of ``n_slots`` blocks in device memory and a device
  map ``v_map[block] -> slot | -1``.  ``locks_decode_fused_vtier`` reads a page
  from its slot when it has one and in place from the pool otherwise (same
  bytes, same output), marks the slots it read and lists the blocks of complete
  pages that missed;
* after a step the notes are read back on a side stream; before a later step
  the host -- without ever waiting for the GPU -- picks victims with a CLOCK
  hand that skips slots read since the last round and brings the missed blocks
  in with ONE ``cudaMemcpyAsync`` per run of contiguous blocks (runs land in
  contiguous slots) on that side stream, which is never captured -- the copy
  engine, no SM involved -- layer by layer, each layer's map update behind its
  copies.  The copies start behind everything already enqueued (no decode that
  could read a victim slot is in flight) and the next decode of layer l waits
  for layer l's event only, so the copies of later layers overlap the earlier
  layers' kernels.  With nothing to promote no stream waits for anything.  A
  miss therefore costs one or two steps of in-place reads (the reference's
  promote-at-graph-head protocol takes two, ``tier/k5.py:1-69``).

Invariants kept (and asserted by ``VTier.check()``): every block's V is in the
pool (I1); the host mirror, the device map and the slot owners agree (I2); no
two blocks share a slot (I3); a slot is overwritten only after the map stopped
naming it, in stream order (I4).  A block that is handed to another sequence
must be dropped with ``invalidate_blocks`` before its first page completes
(the KV-write path knows: the token lands on row 0 of the block).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch

from .. import _cabi
from .decode import PinnedHostVSource, _split_kv


class SlotClock:
    """Residency of one layer's staging buffer -- pure host logic.

    ``slot_of[block]`` / ``blk_of[slot]`` mirror the device map.  ``plan`` takes
    the blocks that missed and the slots that were read in the last step and
    returns copy runs ``(block0, slot0, n)`` -- n consecutive blocks into n
    consecutive slots -- plus the (block, slot | -1) map updates.  Victims come
    from a CLOCK hand: a slot read in the last step is passed over once."""

    def __init__(self, num_blocks: int, n_slots: int):
        self.slot_of = np.full(int(num_blocks), -1, dtype=np.int32)
        self.blk_of = np.full(int(n_slots), -1, dtype=np.int32)
        self.n_slots = int(n_slots)
        self.hand = 0

    def drop(self, blocks: Sequence[int]) -> List[Tuple[int, int]]:
        """Forget blocks (their content changed owner); map updates to apply."""
        upd = []
        for b in blocks:
            s = int(self.slot_of[b])
            if s >= 0:
                self.slot_of[b] = -1
                self.blk_of[s] = -1
                upd.append((int(b), -1))
        return upd

    def plan(self, missed: Sequence[int], ref: np.ndarray, max_blocks: int):
        ref = np.asarray(ref).astype(bool).copy()
        missed = sorted({int(b) for b in missed})[:max(0, int(max_blocks))]
        runs: List[List[int]] = []          # [block0, slot0, n]
        updates: List[Tuple[int, int]] = []
        taken = np.zeros(self.n_slots, dtype=bool)      # slots given out in this plan
        for b in missed:
            s_old = int(self.slot_of[b])
            if s_old >= 0:
                # the device reported a miss for a block the mirror holds: its map
                # entry was dropped on the device (block reuse); refill in place
                slot = s_old
            else:
                slot = -1
                for _ in range(2 * self.n_slots):
                    s = self.hand
                    self.hand = (self.hand + 1) % self.n_slots
                    if taken[s]:
                        continue
                    if ref[s]:
                        ref[s] = False                  # second chance
                        continue
                    slot = s
                    break
                if slot < 0:
                    break                               # everything is in use
                old = int(self.blk_of[slot])
                if old >= 0:
                    self.slot_of[old] = -1
                    updates.append((old, -1))
            taken[slot] = True
            self.blk_of[slot] = b
            self.slot_of[b] = slot
            updates.append((b, slot))
            if runs and runs[-1][0] + runs[-1][2] == b and \
                    runs[-1][1] + runs[-1][2] == slot:
                runs[-1][2] += 1
            else:
                runs.append([b, slot, 1])
        # a block evicted and re-admitted in one plan keeps only its last update
        last = {}
        for b, s in updates:
            last[b] = s
        return [tuple(r) for r in runs], sorted(last.items())

    def check(self) -> None:
        res = np.nonzero(self.slot_of >= 0)[0]
        slots = self.slot_of[res]
        assert len(set(slots.tolist())) == len(slots), "two blocks share a slot"
        assert (self.blk_of[slots] == res).all(), "slot owners disagree with the map"
        assert int((self.blk_of >= 0).sum()) == len(res), "orphan slot owner"


class TieredVSource:
    """V source of one layer for ``sparse_paged_decode_fused`` (tier variant)."""
    SRC_ID = 2

    def __init__(self, tier: "VTier", layer: int):
        self.tier, self.layer = tier, layer

    def args(self):
        v = self.tier.pool[self.layer].plane
        return v, v.stride(0), v.stride(1), v.stride(2)


class VTier:
    """All layers' pools, staging buffers, maps and the promotion machinery."""

    def __init__(self, kv_caches: Sequence[torch.Tensor], n_slots: int,
                 miss_cap: int = 4096, max_promote_blocks: int = 1 << 30):
        k0, v0 = _split_kv(kv_caches[0])
        dev = kv_caches[0].device
        self.device = dev
        self.L = len(kv_caches)
        self.NB = int(k0.shape[0])
        self.n_slots = int(n_slots)
        self.miss_cap = int(miss_cap)
        self.max_promote = int(max_promote_blocks)
        self.pool = [PinnedHostVSource(c) for c in kv_caches]
        page, n_kv, d = int(k0.shape[1]), int(k0.shape[2]), int(k0.shape[3])
        assert k0.stride(1) == n_kv * d and k0.stride(2) == d and k0.stride(3) == 1, \
            "the tier expects token rows of n_kv x d contiguous elements"
        self.block_elems = page * n_kv * d
        self.hot = [torch.zeros(self.n_slots, page, n_kv, d, device=dev,
                                dtype=v0.dtype) for _ in range(self.L)]
        self.v_map = torch.full((self.L, self.NB), -1, device=dev, dtype=torch.int32)
        self.ref = torch.zeros(self.L, self.n_slots, device=dev, dtype=torch.uint8)
        self.pending = torch.zeros(self.L, self.NB, device=dev, dtype=torch.int32)
        self.miss = torch.zeros(self.L, self.miss_cap, device=dev, dtype=torch.int32)
        self.miss_cnt = torch.zeros(self.L, device=dev, dtype=torch.int32)
        self.round = 1
        self.note_round = torch.full((1,), self.round, device=dev, dtype=torch.int32)
        self.last_missed = 0
        # pinned landing buffers of the read-back
        self.h_ref = torch.zeros(self.L, self.n_slots, dtype=torch.uint8,
                                 pin_memory=True)
        self.h_miss = torch.zeros(self.L, self.miss_cap, dtype=torch.int32,
                                  pin_memory=True)
        self.h_cnt = torch.zeros(self.L, dtype=torch.int32, pin_memory=True)
        self.clock = [SlotClock(self.NB, self.n_slots) for _ in range(self.L)]
        self.side = torch.cuda.Stream(device=dev)       # never captured
        self.ev_read = torch.cuda.Event()
        self.ev_layer = [torch.cuda.Event() for _ in range(self.L)]
        self._readback_pending = False
        self._layer_ready = [True] * self.L
        self.stats = {"steps": 0, "missed_blocks": 0, "promoted_blocks": 0,
                      "copy_runs": 0, "dropped_notes": 0}

    # ---- decode side -------------------------------------------------------------
    def vsource(self, layer: int) -> TieredVSource:
        return TieredVSource(self, layer)

    def wait_layer(self, layer: int) -> None:
        """Order the current stream behind the layer's promotion copies (the
        events live outside any graph: while a graph is being captured nothing
        is waited for -- call ``wait_all`` before replaying it)."""
        if not self._layer_ready[layer] and \
                not torch.cuda.is_current_stream_capturing():
            torch.cuda.current_stream(self.device).wait_event(self.ev_layer[layer])
            self._layer_ready[layer] = True

    def wait_all(self) -> None:
        for l in range(self.L):
            self.wait_layer(l)

    def decode(self, layer, q, kv_cache, block_table, seq_lens, st, out, scale):
        """Fused sparse decode of one layer with V through the tier."""
        self.wait_layer(layer)
        k, _ = _split_kv(kv_cache)
        vh = self.pool[layer].plane
        assert (k.stride(0), k.stride(1), k.stride(2)) == \
            (vh.stride(0), vh.stride(1), vh.stride(2))
        n_req = int(seq_lens.shape[0])
        _cabi.call("locks_decode_fused_vtier", _cabi.ptr(q), q.stride(0),
                   _cabi.ptr(k), _cabi.ptr(vh), k.stride(0), k.stride(1),
                   k.stride(2), _cabi.ptr(self.hot[layer]),
                   self.hot[layer].stride(0), _cabi.ptr(self.v_map[layer]),
                   _cabi.ptr(self.ref[layer]), _cabi.ptr(self.pending[layer]),
                   _cabi.ptr(self.miss[layer]), _cabi.ptr(self.miss_cnt[layer:]),
                   self.miss_cap, _cabi.ptr(self.note_round), _cabi.ptr(block_table),
                   block_table.stride(0),
                   _cabi.ptr(st.page_table), _cabi.ptr(st.page_cnt),
                   _cabi.ptr(seq_lens), _cabi.ptr(out), out.stride(0), n_req,
                   int(st.n_kv), int(st.G), int(st.d), int(st.page),
                   int(st.max_pages), float(scale), _cabi.ptr(st.status),
                   _cabi.stream())

    # ---- between steps -------------------------------------------------------------
    def end_step(self) -> None:
        """After a step's last decode was enqueued: start reading the residency
        notes back (side stream, behind the step) unless an earlier read-back
        is still waiting to be consumed -- the notes keep accumulating."""
        self.stats["steps"] += 1
        if self._readback_pending:
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.side):
            self.side.wait_event(ev)
            self.h_ref.copy_(self.ref, non_blocking=True)
            self.h_miss.copy_(self.miss, non_blocking=True)
            self.h_cnt.copy_(self.miss_cnt, non_blocking=True)
            self.ev_read.record(self.side)
        self._readback_pending = True

    def promote(self, block: bool = False) -> bool:
        """Before a step is enqueued: consume the last read-back and bring the
        listed blocks in.  Never waits for the GPU unless ``block``: when the
        read-back has not landed yet the step simply runs with what is staged
        (a miss is read in place) and the promotion happens one step later.
        True when a read-back was consumed."""
        if not self._readback_pending:
            return False
        if block:
            self.ev_read.synchronize()
        elif not self.ev_read.query():
            return False
        self._readback_pending = False
        cnt = self.h_cnt.numpy().copy()
        plans = []
        for l in range(self.L):
            n = int(cnt[l])
            listed = self.h_miss[l, :min(n, self.miss_cap)].numpy().copy()
            self.stats["missed_blocks"] += n
            self.stats["dropped_notes"] += max(0, n - self.miss_cap)
            runs, upd = self.clock[l].plan(listed, self.h_ref[l].numpy(),
                                           self.max_promote) if n else ([], [])
            plans.append((runs, upd))
        self.last_missed = int(cnt.sum())
        main = torch.cuda.current_stream(self.device)
        busy = any(upd for _, upd in plans)
        ev_main = None
        if busy:
            # a slot may be overwritten only when no decode that could still
            # read it is in flight: the copies start behind everything enqueued
            ev_main = torch.cuda.Event()
            ev_main.record(main)
        with torch.cuda.stream(self.side):
            # a new note round: blocks listed so far may be listed again; notes
            # written while these three run are lost and come back next round
            self.round += 1
            self.note_round.fill_(self.round)
            self.ref.zero_()
            self.miss_cnt.zero_()
            if busy:
                self.side.wait_event(ev_main)
                for l, (runs, upd) in enumerate(plans):
                    if upd:
                        self._apply(l, runs, upd)
                    self.ev_layer[l].record(self.side)
                    self._layer_ready[l] = False
        return True

    def _apply(self, l, runs, upd) -> None:
        """Side stream: unmap the victims, copy the runs, map the new blocks."""
        dev = self.device
        if upd:
            blk = torch.tensor([b for b, _ in upd], dtype=torch.int64)
            gone = torch.full((len(upd),), -1, dtype=torch.int32)
            # 1. no entry may name a slot that is about to be overwritten
            self.v_map[l].index_copy_(0, blk.to(dev, non_blocking=True),
                                      gone.to(dev, non_blocking=True))
        host, hot = self.pool[l].plane, self.hot[l]
        eb = host.element_size()
        for b0, s0, n in runs:
            # 2. one copy-engine transfer per run of contiguous blocks
            _cabi.call("locks_vtier_copy_run", _cabi.ptr(hot[s0]),
                       hot.stride(0) * eb, _cabi.ptr(host[b0]),
                       host.stride(0) * eb, self.block_elems * eb, int(n),
                       self.side.cuda_stream)
            self.stats["promoted_blocks"] += n
            self.stats["copy_runs"] += 1
        if upd:
            new = torch.tensor([s for _, s in upd], dtype=torch.int32)
            # 3. the new owners become visible behind their copies
            self.v_map[l].index_copy_(0, blk.to(dev, non_blocking=True),
                                      new.to(dev, non_blocking=True))

    def invalidate_blocks(self, blocks: Sequence[int]) -> None:
        """Blocks whose content now belongs to another sequence: forget them in
        every layer (current stream: ordered before the writes that follow)."""
        blocks = [int(b) for b in blocks]
        if not blocks:
            return
        idx = torch.tensor(blocks, dtype=torch.int64, device=self.device)
        for l in range(self.L):
            self.wait_layer(l)
            if self.clock[l].drop(blocks):
                self.v_map[l].index_fill_(0, idx, -1)

    # ---- checks ------------------------------------------------------------------
    def check(self) -> None:
        """Invariants: mirror == device map, no aliasing, staged bytes == pool."""
        torch.cuda.synchronize(self.device)
        vm = self.v_map.cpu().numpy()
        for l in range(self.L):
            c = self.clock[l]
            c.check()
            assert (vm[l] == c.slot_of).all(), "device map differs from the mirror"
            res = np.nonzero(c.slot_of >= 0)[0]
            if len(res):
                slots = torch.from_numpy(c.slot_of[res].astype(np.int64))
                staged = self.hot[l].index_select(0, slots.to(self.device)).cpu()
                want = self.pool[l].plane[torch.from_numpy(res)]
                assert torch.equal(staged.view(torch.int16), want.view(torch.int16)), \
                    "a staged block differs from the pool"

    def resident_blocks(self, layer: int) -> int:
        return int((self.clock[layer].slot_of >= 0).sum())
