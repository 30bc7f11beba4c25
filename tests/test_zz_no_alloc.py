"""GroupNorm entry point for callers that cannot allocate device memory: a serving process that has handed all device
memory to another allocator, or a plugin in a runtime that forbids allocations after start-up, has no scratch buffer to
pass. `katz_group_norm_nhwc_f16_noalloc` keeps its partial sums in a fixed array inside the library instead.

Called here straight through the C ABI (ctypes, raw pointers) and compared with the scratch-taking entry point on two
calls in a row with different inputs and shapes, so a stale partial left by the first call would show in the second.
This file is collected last on purpose: a run that stops at the first failure has then run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_no_alloc_group_norm_matches_scratch_entry_point(cuda_device):
    from katz_b200 import _lib
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    limit = lib.katz_group_norm_static_scratch_bytes()
    assert limit == 512 * 1024
    g = torch.Generator().manual_seed(0)
    # two calls in a row: different shapes, slab counts and statistics
    for B, HW, C, act, shift in [(2, 4096, 320, 1, 2.0), (1, 1024, 1280, 0, -1.0)]:
        x = (torch.randn(B, HW, C, generator=g) + shift).half().cuda()
        gamma = (1 + 0.1 * torch.randn(C, generator=g)).half().cuda()
        beta = (0.1 * torch.randn(C, generator=g)).half().cuda()
        need = lib.katz_group_norm_scratch_bytes(B, HW, C, 32)
        assert 0 < need <= limit
        scratch = torch.zeros(need, dtype=torch.uint8, device="cuda")      # zero-filled once, as the header asks
        y_ref = torch.empty_like(x)
        rc = lib.katz_group_norm_nhwc_f16(_ptr(x), _ptr(y_ref), _ptr(gamma), _ptr(beta), B, HW, C, 32, 1e-5, act, _ptr(scratch),
                                          need, stream)
        assert rc == 0
        y = torch.full_like(x, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = lib.katz_group_norm_nhwc_f16_noalloc(_ptr(x), _ptr(y), _ptr(gamma), _ptr(beta), B, HW, C, 32, 1e-5, act, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before          # torch's allocator was not touched
        # same kernels in the same order with fixed-order reductions: the same bits
        assert torch.isfinite(y.float()).all()
        assert torch.equal(y, y_ref)
    # the reset of the ticket counters allocates nothing and leaves the next call correct
    y2 = torch.empty_like(x)
    before = torch.cuda.memory_allocated()
    assert lib.katz_group_norm_static_scratch_reset(stream) == 0
    assert lib.katz_group_norm_nhwc_f16_noalloc(_ptr(x), _ptr(y2), _ptr(gamma), _ptr(beta), B, HW, C, 32, 1e-5, act, stream) == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before and torch.equal(y2, y_ref)


def test_no_alloc_group_norm_rejects_sizes_beyond_its_array(cuda_device):
    from katz_b200 import _lib
    lib = _lib.load()
    B, HW, C, G = 4096, 64, 64, 32          # many batch elements -> more partial sums than the fixed array holds
    assert lib.katz_group_norm_scratch_bytes(B, HW, C, G) > lib.katz_group_norm_static_scratch_bytes()
    x = torch.zeros(8, dtype=torch.float16, device="cuda")
    rc = lib.katz_group_norm_nhwc_f16_noalloc(_ptr(x), _ptr(x), None, None, B, HW, C, G, 1e-5, 0, None)
    assert rc == -3                         # KATZ_E_SIZE, returned before anything is launched
    with pytest.raises(_lib.KatzError, match="shape outside"):
        _lib.check(rc, "katz_group_norm_nhwc_f16_noalloc")
