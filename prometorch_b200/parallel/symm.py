"""Symmetric peer memory for the fused compute+collective kernels.

One process per GPU.  ``SymmGroup.alloc(nbytes)`` is a collective: every rank
allocates ``nbytes`` of device memory, the CUDA IPC handles are exchanged
through the process group (the only host-side traffic), and each rank maps all
peers' buffers.  The returned :class:`SymmBuffer` gives ``peer_ptr(r)`` — an
address valid on *this* GPU that refers to rank ``r``'s buffer — which the
kernels dereference with plain loads/stores over NVLink.

This is the data plane that replaces the reference's TCP star and /dev/shm
process groups (torch/distributed/ddp.cpp:287-422, 84-139).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from .. import _native as N


@N.register_decls
def _decls(L):
    vp = C.c_void_p
    L.ptb_symm_alloc.argtypes = [C.c_size_t, C.POINTER(vp), vp]
    L.ptb_symm_alloc.restype = C.c_int
    L.ptb_symm_open.argtypes = [vp, C.POINTER(vp)]
    L.ptb_symm_open.restype = C.c_int
    L.ptb_symm_close.argtypes = [vp]
    L.ptb_symm_close.restype = C.c_int
    L.ptb_symm_free.argtypes = [vp]
    L.ptb_symm_free.restype = C.c_int
    L.ptb_enable_peer_access.argtypes = [C.c_int, C.c_int]
    L.ptb_enable_peer_access.restype = C.c_int


GUARD = 256                      # bytes of canary words before and after every symmetric buffer
_CANARY = 0x5AFEC0DE


class SymmBuffer:
    """``nbytes`` of this rank's memory that every peer can address, between two guard regions filled with a known
    word.  Kernels of the peers write into it through raw pointers; :meth:`check_canaries` tells on the host whether
    anything wrote past either end."""

    def __init__(self, group: "SymmGroup", nbytes: int, local: int, peers: List[int]):
        # `local` / `peers` are the allocation bases; the usable region starts GUARD bytes in
        self.group, self.nbytes = group, nbytes
        self._base_local, self._base_peers = local, peers
        self.local, self._peers = local + GUARD, [p + GUARD if p else 0 for p in peers]
        self._guard_view(0).fill_(_CANARY)
        self._guard_view(1).fill_(_CANARY)

    def _guard_view(self, which: int) -> torch.Tensor:
        class _A:
            pass
        a = _A()
        addr = self._base_local if which == 0 else self._base_local + GUARD + self.nbytes
        a.__cuda_array_interface__ = {"shape": (GUARD // 4,), "typestr": "<i4", "data": (addr, False), "version": 3}
        return torch.as_tensor(a, device=self.group.device)

    def check_canaries(self):
        """Raise if a guard word changed (someone wrote outside the buffer)."""
        for which, name in ((0, "before"), (1, "after")):
            g = self._guard_view(which)
            bad = (g != _CANARY).nonzero()
            if bad.numel():
                raise RuntimeError(f"symmetric buffer of {self.nbytes} bytes: guard word {int(bad[0])} {name} the buffer was overwritten")

    def peer_ptr(self, rank: int) -> int:
        return self._peers[rank]

    def tensor(self, dtype=torch.float32, rank: Optional[int] = None) -> torch.Tensor:
        """A torch view of the local buffer (or of a peer's mapping)."""
        addr = self.local if rank is None else self._peers[rank]
        item = torch.empty(0, dtype=dtype).element_size()
        typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1", torch.bfloat16: "<u2",
                   torch.float16: "<f2", torch.uint32: "<u4"}[dtype]

        class _A:
            pass
        a = _A()
        a.__cuda_array_interface__ = {"shape": (self.nbytes // item,), "typestr": typestr, "data": (addr, False), "version": 3}
        t = torch.as_tensor(a, device=self.group.device)
        return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t

    def free(self):
        lib = N.lib()
        for r, p in enumerate(self._base_peers):
            if r != self.group.rank and p:
                lib.ptb_symm_close(p)
        if self._base_local:
            lib.ptb_symm_free(self._base_local)
        self.local, self._peers, self._base_local, self._base_peers = 0, [], 0, []


class SymmGroup:
    """Ranks of a ``torch.distributed`` process group that share peer-mapped buffers."""

    def __init__(self, pg=None, device=None):
        import torch.distributed as dist
        self.dist = dist
        self.pg = pg if pg is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.pg)
        self.world = dist.get_world_size(self.pg)
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self._bufs: List[SymmBuffer] = []

    def alloc(self, nbytes: int) -> SymmBuffer:
        lib = N.lib()
        torch.cuda.set_device(self.device)
        nbytes = (int(nbytes) + 255) // 256 * 256
        ptr = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        N.check(lib.ptb_symm_alloc(nbytes + 2 * GUARD, C.byref(ptr), handle), "symm alloc")
        handles: List[Optional[bytes]] = [None] * self.world
        self.dist.all_gather_object(handles, bytes(handle), group=self.pg)
        peers = []
        for r, h in enumerate(handles):
            if r == self.rank:
                peers.append(ptr.value)
                continue
            p = C.c_void_p()
            hb = (C.c_ubyte * 64).from_buffer_copy(h)
            N.check(lib.ptb_symm_open(hb, C.byref(p)), f"symm open (rank {r})")
            peers.append(p.value)
        buf = SymmBuffer(self, nbytes, ptr.value, peers)
        self._bufs.append(buf)
        self.barrier()
        return buf

    def barrier(self):
        torch.cuda.synchronize(self.device)
        self.dist.barrier(group=self.pg)

    def check_canaries(self):
        """Check the guard words of every buffer of this group (call between steps, e.g. from tests or a debug run)."""
        torch.cuda.synchronize(self.device)
        for b in self._bufs:
            if b.local:
                b.check_canaries()

    def close(self):
        self.barrier()
        for b in self._bufs:
            b.free()
        self._bufs = []
