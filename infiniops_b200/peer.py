"""Peer buffers between the ranks of one machine (one process per GPU), for the GEMM epilogue that
stores its output slice straight into every other GPU's result matrix.

`PeerGroup` owns, per rank, one device arena that all ranks map: `flags` (one int per rank, written
by the peers' completion signals) followed by a data region from which result matrices are carved.
The device side is `libinfiniops_b200.so` (peer_alloc / peer_export / peer_open / peer_wait); this
module only moves the 64-byte handles between the processes with `torch.distributed` and hands the
arena out as torch tensors.  The reference has no counterpart (it has no communication layer).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import capi

_FLAG_BYTES = 256     # flag words of up to 32 ranks, padded so that the data region stays aligned
_CTRL_INTS = 8        # local control words: done counter, epoch, wait epoch, status[2]


class _DeviceArray:
    """Lets torch view raw device memory (`torch.as_tensor(obj, device=...)`)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerGroup:
    def __init__(self, data_bytes: int, device: torch.device, group=None):
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world - 1 > capi.MAX_PEERS:
            raise ValueError(f"at most {capi.MAX_PEERS + 1} ranks")
        lib = capi.lib()
        self.data_bytes = (data_bytes + 255) // 256 * 256
        total = _FLAG_BYTES + self.data_bytes
        base = ctypes.c_void_p()
        capi._check(lib.infiniops_b200_peer_alloc(total, ctypes.byref(base)))
        self.base = base.value
        handle = ctypes.create_string_buffer(64)
        capi._check(lib.infiniops_b200_peer_export(self.base, handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.peer_base: list[int] = []
        for r, raw in enumerate(handles):
            if r == self.rank:
                self.peer_base.append(self.base)
                continue
            mapped = ctypes.c_void_p()
            capi._check(lib.infiniops_b200_peer_open(raw, ctypes.byref(mapped)))
            self.peer_base.append(mapped.value)
        self._keep = _DeviceArray(self.base, total)
        self.arena = torch.as_tensor(self._keep, device=device)
        self.flags = self.arena[:_FLAG_BYTES].view(torch.int32)
        self.data = self.arena[_FLAG_BYTES:]
        self.ctrl = torch.zeros(_CTRL_INTS, dtype=torch.int32, device=device)   # local, never mapped by peers
        self._used = 0
        dist.barrier(group=group)

    # -- carving ---------------------------------------------------------------------------------
    def carve(self, nbytes: int) -> int:
        """Offset (in the data region, the same on every rank) of a fresh 256-byte aligned piece."""
        off = self._used
        self._used += (nbytes + 255) // 256 * 256
        if self._used > self.data_bytes:
            raise ValueError("peer arena exhausted")
        return off

    def local(self, off: int, shape, dtype) -> torch.Tensor:
        n = int(torch.tensor(shape).prod()) * torch.empty((), dtype=dtype).element_size()
        return self.data[off:off + n].view(dtype).view(*shape)

    def address(self, rank: int, off: int) -> int:
        return self.peer_base[rank] + _FLAG_BYTES + off

    def others(self) -> list[int]:
        return [r for r in range(self.world) if r != self.rank]

    # -- signalling ------------------------------------------------------------------------------
    def signal(self) -> capi.PeerSignal:
        """Completion signal for a launch: bumps this rank's epoch and publishes it to every peer."""
        s = capi.PeerSignal()
        s.done_counter = self.ctrl[0:].data_ptr()
        s.epoch = self.ctrl[1:].data_ptr()
        s.n_peers = self.world - 1
        for i, r in enumerate(self.others()):
            s.peer_flags[i] = self.peer_base[r]
        s.flag_slot = self.rank
        return s

    def wait(self, stream=None) -> None:
        """Enqueues the bounded wait for the next epoch of every peer."""
        capi._check(capi.lib().infiniops_b200_peer_wait(self.flags.data_ptr(), self.world, self.rank,
                                                        self.ctrl[2:].data_ptr(), self.ctrl[3:].data_ptr(),
                                                        capi._stream(stream)))

    def wait_status(self) -> tuple[int, int]:
        """(0, 0) unless a wait ran out: then (8, slot of the peer that never signalled)."""
        s = self.ctrl[3:5].tolist()
        return int(s[0]), int(s[1])

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        lib = capi.lib()
        for r, ptr in enumerate(self.peer_base):
            if r != self.rank:
                lib.infiniops_b200_peer_close(ptr)
        self.arena = self.flags = self.data = None
        dist.barrier(group=self.group)
        lib.infiniops_b200_peer_free(self.base)
