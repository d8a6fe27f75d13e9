"""Peer-mapped output buffers for the row-sharded mul_mat that gathers over NVLink by itself.

One process per GPU.  Every rank allocates its buffers through the C ABI (``weft_b200_peer_alloc``: device
memory plus a 64-byte CUDA IPC handle), the handles travel once through ``torch.distributed``
(``all_gather_object``; any backend), and every rank opens every other rank's buffers
(``weft_b200_peer_open``).  The result is, per buffer, a table of ``world`` device pointers -- rank r's
buffer as mapped in this process -- in the form ``weft_b200_mul_mat_shard_gather`` takes.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Sequence

SYNC_INTS = 32      # the sync block of include/weft_b200.h: int[32], zero-filled by peer_alloc
STAGE_BYTES = 2 * 8 * 65536   # WEFT_B200_GATHER_STAGE_BYTES: the staging area of the flagged-value protocol, any call shape


def exchange_handles(mine: Sequence[bytes], world: int, group=None) -> list[list[bytes]]:
    """All ranks' handle lists, indexed [rank][buffer]."""
    import torch.distributed as dist

    everyone: list = [None] * world
    dist.all_gather_object(everyone, [bytes(h) for h in mine], group=group)
    if any(len(handles) != len(mine) for handles in everyone):
        raise RuntimeError("ranks exported different numbers of buffers")
    return everyone


def pointer_table(pointers: Sequence[int]):
    """ctypes array of device pointers, one per rank."""
    return (ctypes.c_void_p * len(pointers))(*pointers)


class PeerBuffers:
    """``sizes[i]`` bytes on every rank for buffer i, each mapped on all ranks.

    ``tables[i]`` is the ctypes pointer table of buffer i (index = rank); ``local[i]`` is this rank's own
    device pointer.  ``close()`` unmaps the peers' buffers and frees the own ones; call it on every rank.
    """

    def __init__(self, lib, world: int, rank: int, sizes: Sequence[int], *, group=None,
                 exchange: Callable[[Sequence[bytes], int], list[list[bytes]]] | None = None) -> None:
        self._lib, self.world, self.rank = lib, world, rank
        lib.weft_b200_peer_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]
        lib.weft_b200_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
        lib.weft_b200_peer_close.argtypes = [ctypes.c_void_p]
        lib.weft_b200_peer_free.argtypes = [ctypes.c_void_p]
        self.local: list[int] = []
        handles: list[bytes] = []
        for size in sizes:
            pointer, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
            self._check(lib.weft_b200_peer_alloc(size, ctypes.byref(pointer), handle))
            self.local.append(pointer.value)
            handles.append(handle.raw)
        everyone = (exchange or (lambda mine, w: exchange_handles(mine, w, group)))(handles, world)
        self._opened: list[int] = []
        self.tables = []
        for index in range(len(sizes)):
            pointers = []
            for peer in range(world):
                if peer == rank:
                    pointers.append(self.local[index])
                    continue
                pointer = ctypes.c_void_p()
                self._check(lib.weft_b200_peer_open(everyone[peer][index], ctypes.byref(pointer)))
                self._opened.append(pointer.value)
                pointers.append(pointer.value)
            self.tables.append(pointer_table(pointers))

    def _check(self, status: int) -> None:
        if status:
            from .runtime.driver import last_error

            raise RuntimeError("weft_b200 peer memory: " + last_error(self._lib))

    def close(self, barrier: Callable[[], None] | None = None) -> None:
        """``barrier`` (e.g. ``torch.distributed.barrier``) runs between unmapping the peers' buffers and freeing the
        own ones, so that no rank frees memory another rank still has mapped."""
        for pointer in self._opened:
            self._lib.weft_b200_peer_close(ctypes.c_void_p(pointer))
        if barrier is not None:
            barrier()
        for pointer in self.local:
            self._lib.weft_b200_peer_free(ctypes.c_void_p(pointer))
        self._opened, self.local = [], []
