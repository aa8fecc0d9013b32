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
