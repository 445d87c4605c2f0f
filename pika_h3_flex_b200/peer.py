"""Device buffers that the other ranks of a process group can store into, for the sequence-parallel reshard.

The reference runs one request on one GPU (reference ``README.md:115``); under sequence parallelism (BASELINE's
configuration 4) every rank prepares its token shard of all heads while each head is computed by one rank.  Instead
of staging blocks and exchanging them with a collective, the producing kernels store each row straight into the
memory of the rank that needs it: one ``cudaMalloc`` per rank, made visible to the other processes of the machine
through CUDA's inter-process handles (``h3a_peer_alloc`` / ``h3a_peer_open``) and reached over NVLink.  Peer memory
is only ever a STORE target here: every load, TMA tile and tensor map covers the rank's own memory.

A :class:`PeerArena` is that allocation plus the table of its address in every rank; sub-buffers are carved from it
at fixed offsets, identical on all ranks.  ``barrier()`` is the meeting point the protocol needs before the owner of
a buffer reads what the others stored: a one-element all-reduce on the group, ordered on the current stream (no host
synchronisation).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from ._lib import check


class _Raw:
    """Presents a raw device range to torch through ``__cuda_array_interface__`` (zero-copy)."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner  # keeps the arena alive while a tensor made from this object exists
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


class PeerArena:
    """``nbytes`` of device memory on this rank, opened by every rank of ``group`` (all ranks must construct it with
    the same size, in the same order).  ``addr(rank, offset)`` is the device address of byte ``offset`` of rank
    ``rank``'s arena as THIS process sees it; ``tensor(offset, shape, dtype)`` is a torch view of the local one."""

    ALIGN = 1024

    def __init__(self, nbytes: int, group=None, device=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > _lib.MAX_RANKS:
            raise ValueError(f"at most {_lib.MAX_RANKS} ranks share an arena")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.nbytes = int(nbytes)
        lib = _lib.load()
        self._lib = lib
        ptr = C.c_void_p(0)
        handle = C.create_string_buffer(_lib.PEER_HANDLE_BYTES)
        with torch.cuda.device(self.device):
            check(lib.h3a_peer_alloc(self.nbytes, C.byref(ptr), handle), "h3a_peer_alloc")
        self._own = int(ptr.value)
        self.ptrs: List[int] = [0] * self.world
        self.ptrs[self.rank] = self._own
        self._opened: List[int] = []
        if self.world > 1:
            handles: List[Optional[Tuple[bytes, int]]] = [None] * self.world
            dist.all_gather_object(handles, (handle.raw, self.nbytes), group=group)
            if any(h[1] != self.nbytes for h in handles):
                raise ValueError(f"ranks disagree on the arena size: {[h[1] for h in handles]}")
            with torch.cuda.device(self.device):
                for r, (raw, _) in enumerate(handles):
                    if r == self.rank:
                        continue
                    p = C.c_void_p(0)
                    check(lib.h3a_peer_open(raw, C.byref(p)), f"h3a_peer_open(rank {r})")
                    self.ptrs[r] = int(p.value)
                    self._opened.append(int(p.value))
        self._flag = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._raw = _Raw(self._own, self.nbytes, self)
        self._bytes = torch.as_tensor(self._raw, device=self.device)
        self._closed = False

    def addr(self, rank: int, offset: int = 0) -> int:
        return self.ptrs[rank] + int(offset)

    def tensor(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nb = n * torch.empty((), dtype=dtype).element_size()
        if offset % 16 or offset + nb > self.nbytes:
            raise ValueError("sub-buffer outside the arena or not 16-byte aligned")
        return self._bytes[offset : offset + nb].view(dtype).view(*shape)

    def barrier(self) -> None:
        """Every rank's work queued on its current stream before this call has completed before any rank's work
        queued after it starts.  Stream-ordered; the host does not wait."""
        if self.world > 1:
            dist.all_reduce(self._flag, group=self.group)

    def close(self) -> None:
        """Unmap the peers' arenas, meet, then free the own one (no rank may free while another still has it mapped)."""
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for p in self._opened:
                self._lib.h3a_peer_close(p)
            self._opened = []
            if self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)
            self._bytes = None
            self._lib.h3a_peer_free(self._own)


class Carver:
    """Hands out aligned offsets inside an arena; run the same sequence of ``take`` calls on every rank."""

    def __init__(self):
        self.size = 0

    def take(self, nbytes: int) -> int:
        off = self.size
        self.size = (off + int(nbytes) + PeerArena.ALIGN - 1) // PeerArena.ALIGN * PeerArena.ALIGN
        return off
