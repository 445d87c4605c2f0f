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


class PeerUnavailable(RuntimeError):
    """The ranks could not share device memory (allocation or inter-process mapping failed on some rank); raised on
    EVERY rank of the group, so that all of them can fall back to an exchange through the communication library."""


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
        # Set-up is collective and must FAIL collectively: a rank whose allocation or mapping fails still takes part in
        # every exchange below, and all ranks raise PeerUnavailable together instead of leaving the others blocked.
        self._own = 0
        self._opened: List[int] = []
        self.ptrs: List[int] = [0] * self.world
        problem = None
        ptr = C.c_void_p(0)
        handle = C.create_string_buffer(_lib.PEER_HANDLE_BYTES)
        with torch.cuda.device(self.device):
            rc = lib.h3a_peer_alloc(self.nbytes, C.byref(ptr), handle)
        if rc != _lib.H3A_OK:
            problem = f"rank {self.rank}: h3a_peer_alloc of {self.nbytes} bytes: {_lib.status_string(rc)}"
        else:
            self._own = int(ptr.value)
            self.ptrs[self.rank] = self._own
        if self.world > 1:
            handles: List[Optional[Tuple[Optional[bytes], int, Optional[str]]]] = [None] * self.world
            dist.all_gather_object(handles, (handle.raw if problem is None else None, self.nbytes, problem), group=group)
            problems = [h[2] for h in handles if h[2]]
            if not problems and any(h[1] != self.nbytes for h in handles):
                problems = [f"ranks disagree on the arena size: {[h[1] for h in handles]}"]
            if not problems:
                with torch.cuda.device(self.device):
                    for r, (raw, _, _) in enumerate(handles):
                        if r == self.rank:
                            continue
                        p = C.c_void_p(0)
                        rc = lib.h3a_peer_open(raw, C.byref(p))
                        if rc != _lib.H3A_OK:
                            problem = f"rank {self.rank}: h3a_peer_open(rank {r}): {_lib.status_string(rc)}"
                            break
                        self.ptrs[r] = int(p.value)
                        self._opened.append(int(p.value))
                verdicts: List[Optional[str]] = [None] * self.world
                dist.all_gather_object(verdicts, problem, group=group)
                problems = [v for v in verdicts if v]
            if problems:  # every rank is here with the same verdict
                self._release(meet=True)
                raise PeerUnavailable("; ".join(problems))
        elif problem is not None:
            raise PeerUnavailable(problem)
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

    def _release(self, meet: bool = False) -> None:
        with torch.cuda.device(self.device):
            for p in self._opened:
                self._lib.h3a_peer_close(p)
            self._opened = []
            if meet and self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)  # no rank frees while another still has it mapped
            self._bytes = None
            if self._own:
                self._lib.h3a_peer_free(self._own)
                self._own = 0

    def close(self) -> None:
        """Unmap the peers' arenas, meet, then free the own one (no rank may free while another still has it mapped)."""
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        self._release(meet=True)


class Carver:
    """Hands out aligned offsets inside an arena; run the same sequence of ``take`` calls on every rank."""

    def __init__(self):
        self.size = 0

    def take(self, nbytes: int) -> int:
        off = self.size
        self.size = (off + int(nbytes) + PeerArena.ALIGN - 1) // PeerArena.ALIGN * PeerArena.ALIGN
        return off
