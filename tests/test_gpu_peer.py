"""GPU: the peer-memory all-gather on ONE GPU. Two arenas in one process stand for two ranks; the other rank's flag is
either written by the host beforehand (the exchange completes) or never (the bounded wait runs out and the status word
says which rank was missing). No second process, no fault: the kernel returns in both cases."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _arena(lib, nbytes):
    from katz_b200 import _lib
    p = ctypes.c_void_p()
    _lib.check(lib.katz_peer_arena_alloc(nbytes, ctypes.byref(p)), "katz_peer_arena_alloc")
    return p.value


def _view(ptr, nbytes):
    from katz_b200.peer import _Raw
    return torch.as_tensor(_Raw(ptr, nbytes), device="cuda")


def test_peer_allgather_places_blocks_and_times_out_cleanly(cuda_device):
    from katz_b200 import _lib
    lib = _lib.load()
    nbytes = 1 << 20
    ctrl = lib.katz_peer_ctrl_bytes()
    a0, a1 = _arena(lib, nbytes), _arena(lib, nbytes)
    try:
        v0, v1 = _view(a0, nbytes), _view(a1, nbytes)
        bases = (ctypes.c_ulonglong * 2)(a0, a1)
        g = torch.Generator().manual_seed(5)
        wide = torch.randn(64, 96, generator=g).half().cuda()
        src = wide[:, 32:96]                       # a column slice: 64 rows of 128 bytes, 192 bytes apart
        off = ctrl
        # exchange 1 as rank 0, with rank 1's flag for epoch 1 already raised in rank 0's arena
        v0[256 + 4:256 + 8].copy_(torch.tensor([1, 0, 0, 0], dtype=torch.uint8))
        rc = lib.katz_peer_allgather(ctypes.c_void_p(src.data_ptr()), 64, 128, 192, off, bases, 0, 2, None)
        assert rc == 0
        torch.cuda.synchronize()
        assert lib.katz_peer_status(ctypes.c_void_p(a0)) == 0
        want = src.contiguous().view(torch.uint8).flatten()
        assert torch.equal(v0[off:off + 8192], want) and torch.equal(v1[off:off + 8192], want)      # slot 0 on both ranks
        assert int(v1[256:260].view(torch.int32)[0]) == 1                                           # rank 0's flag at rank 1
        # exchange 2: nobody raises rank 1's flag -> the wait runs out, the status names rank 1, the context stays usable
        rc = lib.katz_peer_allgather(ctypes.c_void_p(src.data_ptr()), 64, 128, 192, off + 16384, bases, 0, 2, None)
        assert rc == 0
        torch.cuda.synchronize()
        assert lib.katz_peer_status(ctypes.c_void_p(a0)) == 101
        assert float(torch.ones(4, device="cuda").sum()) == 4.0
        # argument errors come back before anything is launched
        assert lib.katz_peer_allgather(ctypes.c_void_p(src.data_ptr()), 64, 120, 192, off, bases, 0, 2, None) == -3
        assert lib.katz_peer_allgather(ctypes.c_void_p(src.data_ptr()), 64, 128, 192, 0, bases, 0, 2, None) == -3
    finally:
        torch.cuda.synchronize()
        lib.katz_peer_arena_free(ctypes.c_void_p(a0))
        lib.katz_peer_arena_free(ctypes.c_void_p(a1))
