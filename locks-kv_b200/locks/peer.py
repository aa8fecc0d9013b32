"""Peer-memory exchange between the ranks of one node (one process per GPU).

``PeerExchange`` owns one exchange region per rank (allocated by the library,
shared through CUDA IPC) and runs ``locks_cp_exchange``: an all-gather, or an
element-wise unsigned max, of a small payload as ONE kernel per rank over
NVLink peer stores -- no library collective on the data path.  Handles travel
through ``torch.distributed`` objects once, at set-up.  The reference has no
distributed code; this is the transport of the context-parallel decode.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from . import _cabi

MAX_RANKS = 8


class PeerExchange:
    def __init__(self, slot_bytes: int, group=None, packets: bool = False):
        """``packets``: small-payload transport -- every 32-bit word travels as an
        8-byte {word, epoch} packet and the receiver polls the packets themselves
        (no fence, no separate flag; needs 2 x the payload per slot).  A region
        uses one transport for its whole life."""
        assert dist.is_initialized(), "PeerExchange needs an initialised process group"
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        assert self.world <= MAX_RANKS, f"at most {MAX_RANKS} ranks"
        self.packets = bool(packets)
        self.slot_bytes = (int(slot_bytes) * (2 if packets else 1) + 15) // 16 * 16
        nb = ctypes.c_int64()
        _cabi.call("locks_cp_region_bytes", self.slot_bytes, ctypes.byref(nb))
        nbytes = int(nb.value)
        mine = ctypes.c_void_p()
        _cabi.call("locks_cp_alloc", nbytes, ctypes.byref(mine))
        self._mine = mine
        handle = (ctypes.c_ubyte * 64)()
        _cabi.call("locks_cp_ipc_export", mine, handle)
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self._peers = (ctypes.c_void_p * MAX_RANKS)()
        self._opened = []
        for r in range(self.world):
            if r == self.rank:
                self._peers[r] = mine.value
                continue
            h = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
            p = ctypes.c_void_p()
            _cabi.call("locks_cp_ipc_open", h, ctypes.byref(p))
            self._peers[r] = p.value
            self._opened.append(p)
        dist.barrier(group=group)          # every region is open everywhere

    def _run(self, payload: torch.Tensor, out: torch.Tensor, mode: int,
             status: Optional[torch.Tensor]) -> None:
        nbytes = payload.numel() * payload.element_size()
        assert payload.is_contiguous() and out.is_contiguous()
        need = nbytes * (2 if self.packets else 1)
        assert nbytes % 16 == 0 and need <= self.slot_bytes, \
            f"payload of {nbytes} B does not fit the {self.slot_bytes} B slot"
        mode += 2 if self.packets else 0
        _cabi.call("locks_cp_exchange", self._peers, int(self.world),
                   int(self.rank), _cabi.ptr(payload), int(nbytes),
                   int(self.slot_bytes), _cabi.ptr(out), int(mode),
                   _cabi.ptr(status), _cabi.stream())

    def all_gather(self, payload: torch.Tensor, out: torch.Tensor,
                   status: Optional[torch.Tensor] = None) -> None:
        """out (world, ...) <- every rank's payload (out[rank] included)."""
        assert out.numel() * out.element_size() == \
            self.world * payload.numel() * payload.element_size()
        self._run(payload, out, 0, status)

    def all_max_u32(self, keys: torch.Tensor,
                    status: Optional[torch.Tensor] = None) -> None:
        """In place: element-wise maximum over ranks of 32-bit words compared
        as UNSIGNED integers (the order-preserving score keys)."""
        assert keys.element_size() == 4
        self._run(keys, keys, 1, status)

    def close(self) -> None:
        for p in self._opened:
            _cabi.call("locks_cp_ipc_close", p)
        self._opened = []
        if self._mine is not None:
            _cabi.call("locks_cp_free", self._mine)
            self._mine = None


def _share_region(nbytes: int, group):
    """Allocate ``nbytes`` of zeroed device memory through the library and open
    every peer's allocation over CUDA IPC.  Returns (own pointer, ctypes array of
    the ranks' pointers as seen from this process, list of opened handles)."""
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    assert world <= MAX_RANKS, f"at most {MAX_RANKS} ranks"
    mine = ctypes.c_void_p()
    _cabi.call("locks_cp_alloc", int(nbytes), ctypes.byref(mine))
    peers = (ctypes.c_void_p * MAX_RANKS)()
    opened = []
    if world == 1:
        peers[0] = mine.value
        return mine, peers, opened
    handle = (ctypes.c_ubyte * 64)()
    _cabi.call("locks_cp_ipc_export", mine, handle)
    handles = [None] * world
    dist.all_gather_object(handles, bytes(handle), group=group)
    for r in range(world):
        if r == rank:
            peers[r] = mine.value
            continue
        h = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
        p = ctypes.c_void_p()
        _cabi.call("locks_cp_ipc_open", h, ctypes.byref(p))
        peers[r] = p.value
        opened.append(p)
    dist.barrier(group=group)              # every region is open everywhere
    return mine, peers, opened


class CpLinkRegion:
    """This rank's link region of the in-kernel context-parallel exchanges
    (``locks_topb_select_cp`` / ``locks_decode_fused_cp``) and the peers' regions
    opened over CUDA IPC.  ``link(layer, ...)`` gives the per-layer description
    the two entry points take.  With one rank the kernels exchange with
    themselves through the local region (same code path, no peer)."""

    def __init__(self, *, n_kv: int, G: int, cap: int, n_layers: int, group=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.n_kv, self.G, self.cap, self.n_layers = n_kv, G, int(cap), n_layers
        nb = ctypes.c_int64()
        _cabi.call("locks_cp_link_bytes", int(n_kv), int(G), int(cap), ctypes.byref(nb))
        self.nbytes = int(nb.value)
        self._mine, self._peers, self._opened = _share_region(self.nbytes, group)

    def link(self, layer: int, *, p0: int, b_global: int, sink_loc: int,
             nsh_loc: int) -> "_cabi.CpLinkDesc":
        d = _cabi.CpLinkDesc()
        for r in range(MAX_RANKS):
            d.regions[r] = self._peers[r]
        d.world, d.rank = self.world, self.rank
        d.layer, d.n_layers = int(layer), int(self.n_layers)
        d.p0, d.cap, d.b_global = int(p0), int(self.cap), int(b_global)
        d.sink_loc, d.nsh_loc = int(sink_loc), int(nsh_loc)
        return d

    def begin_step(self) -> None:
        """Advance the decode-step counter (once per step, before layer 0)."""
        _cabi.call("locks_cp_begin_step", self._mine, _cabi.stream())

    def resync(self) -> None:
        """After a wait ran out: every rank clears its region and all agree on
        a fresh step value.  Host-side barriers on both sides: no kernel of the
        old steps is in flight when the regions are cleared, none of the new
        ones starts before every region is clean."""
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        self._epoch_base = getattr(self, "_epoch_base", 0) + (1 << 20)
        _cabi.call("locks_cp_link_reset", self._mine, self.nbytes,
                   int(self._epoch_base) & 0x7FFFFFFF, _cabi.stream())
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)

    def close(self) -> None:
        for p in self._opened:
            _cabi.call("locks_cp_ipc_close", p)
        self._opened = []
        if self._mine is not None:
            _cabi.call("locks_cp_free", self._mine)
            self._mine = None
