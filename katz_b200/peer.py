"""Peer-memory arena for the exchanges of the latent-row split (katz_peer_* in include/katz_b200.h).

One arena per rank, allocated by the library with cudaMalloc and mapped into the other processes of the group through
CUDA IPC handles (exchanged once with torch.distributed). `allgather` pushes a local block into the same slot of every
rank's arena and returns, in stream order, when every rank's block has arrived here: one small kernel instead of a NCCL
collective. The reference has no counterpart (its 2-GPU mode exchanges through torch.distributed,
sdxl_unet_server.py:199-215).
"""
import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib
from ._lib import KatzError


class _Raw:
    """Memory the library allocated, presented to torch through the CUDA array interface."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerArena:
    def __init__(self, rank, world, group=None, device=None, nbytes=None):
        if world < 2:
            raise KatzError("a peer arena needs at least two ranks")
        lib = _lib.load()
        self.rank, self.world, self.group = rank, world, group
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.nbytes = int(nbytes if nbytes is not None else os.environ.get("KATZ_PEER_ARENA_BYTES", 1 << 30))
        self.ctrl = lib.katz_peer_ctrl_bytes()
        # Every rank takes part in every collective below whatever happened locally, and all ranks reach the same verdict:
        # a rank that cannot allocate, export or map sends that fact along instead of leaving the others waiting.
        ptr = ctypes.c_void_p()
        self._ptr, self._opened = 0, []
        with torch.cuda.device(self.device):
            hb = lib.katz_peer_ipc_handle_bytes()
            handle = ctypes.create_string_buffer(hb)
            mine = None
            if lib.katz_peer_arena_alloc(self.nbytes, ctypes.byref(ptr)) == 0:
                self._ptr = ptr.value
                if lib.katz_peer_ipc_export(ptr, handle) == 0:
                    mine = bytes(handle.raw)
            handles = [None] * world
            dist.all_gather_object(handles, mine, group=group)
            bases, ok = [], all(h is not None for h in handles)
            if ok:
                for r in range(world):
                    if r == rank:
                        bases.append(self._ptr)
                        continue
                    p = ctypes.c_void_p()
                    if lib.katz_peer_ipc_open(ctypes.create_string_buffer(handles[r], hb), ctypes.byref(p)) != 0:
                        ok = False
                        break
                    self._opened.append(p.value)
                    bases.append(p.value)
            verdict = [None] * world
            dist.all_gather_object(verdict, bool(ok), group=group)
            if not all(verdict):
                self.close()
                raise KatzError("peer arenas could not be set up on every rank (allocation, IPC export or mapping failed)")
        self.bases = (ctypes.c_ulonglong * world)(*bases)
        self.local = torch.as_tensor(_Raw(self._ptr, self.nbytes), device=self.device)      # uint8 view of this rank's arena
        self._slots = []          # (offset, bytes) per call site of a step, in call order
        self._cursor = (self.ctrl + 255) // 256 * 256
        dist.barrier(group=group)     # every arena is mapped everywhere before anything is pushed

    def slot(self, index, nbytes):
        """Offset of the buffer of the index-th exchange of a step (assigned on first use, the same on every rank)."""
        if index < len(self._slots):
            off, size = self._slots[index]
            if size != nbytes:
                raise KatzError("exchange %d of the step changed size (%d -> %d bytes)" % (index, size, nbytes))
            return off
        if index != len(self._slots):
            raise KatzError("exchanges must be numbered consecutively")
        off = self._cursor
        if off + nbytes > self.nbytes:
            raise KatzError("peer arena of %d bytes is too small (KATZ_PEER_ARENA_BYTES)" % self.nbytes)
        self._cursor = (off + nbytes + 255) // 256 * 256
        self._slots.append((off, nbytes))
        return off

    def allgather(self, src, index, wait=True):
        """src: CUDA tensor, contiguous or a column slice [..., c0:c1] of a contiguous tensor, whose rows are multiples of
        16 bytes -> [world, *src.shape] view of the arena (packed). wait=False: push and raise the flags only; the consumer
        (ops.attention(peer=...)) waits for each peer's flag itself, so the transfer overlaps its work on the local block."""
        es = src.element_size()
        if src.is_contiguous():
            rows, row_bytes, pitch = 1, src.numel() * es, src.numel() * es
        else:
            # rows of src.shape[-1] elements at a constant pitch
            lead = src.reshape(-1, src.shape[-1]) if src.dim() > 1 else None
            ok = src.dim() >= 2 and src.stride(-1) == 1 and all(
                src.stride(i) == src.stride(i + 1) * src.shape[i + 1] for i in range(src.dim() - 2))
            if not ok or lead is None:
                raise KatzError("peer all-gather needs a contiguous block or a column slice of one")
            rows, row_bytes, pitch = src.numel() // src.shape[-1], src.shape[-1] * es, src.stride(-2) * es
        if row_bytes % 16 or pitch % 16 or src.data_ptr() % 16:
            raise KatzError("peer all-gather needs 16-byte aligned rows of a multiple of 16 bytes")
        nb = rows * row_bytes
        off = self.slot(index, self.world * nb)
        st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _lib.call("katz_peer_allgather" if wait else "katz_peer_push", ctypes.c_void_p(src.data_ptr()), rows, row_bytes, pitch,
                  off, self.bases, self.rank, self.world, st)
        return self.local[off:off + self.world * nb].view(src.dtype).view((self.world,) + tuple(src.shape))

    def ctrl_address(self):
        """Device address of this rank's control words (exchange counter, flags): what a consumer that waits itself reads."""
        return self._ptr

    def close(self):
        """Unmap the peers' arenas and free this rank's. Collective in effect: call it on every rank, after a
        synchronisation, when no kernel that uses the arena is in flight or captured in a live CUDA graph."""
        lib = _lib.load()
        for p in self._opened:
            lib.katz_peer_ipc_close(ctypes.c_void_p(p))
        self._opened = []
        if self._ptr:
            self.local = None
            torch.cuda.synchronize(self.device)
            lib.katz_peer_arena_free(ctypes.c_void_p(self._ptr))
            self._ptr = 0

    def clear_status(self):
        """Forget a time-out recorded so far (the ranks of a job are not in step while they warm up and capture)."""
        _lib.check(_lib.load().katz_peer_clear_status(ctypes.c_void_p(self._ptr)), "katz_peer_clear_status")

    def status(self):
        """0, or 100 + the rank whose block never arrived within the bounded wait. Synchronises the device."""
        return _lib.load().katz_peer_status(ctypes.c_void_p(self._ptr))
