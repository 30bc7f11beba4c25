"""CPU: the shared-memory LoRA hand-off protocol (flags 0 / 1..9 / 10 / 100) between a loader process and a reader."""
import multiprocessing as mp
import os

import numpy as np
import pytest
import torch


def _info():
    return {"unet.a.lora.down.weight": {"shape": [8, 32], "nbytes": 8 * 32 * 2},
            "unet.a.lora.up.weight": {"shape": [16, 8], "nbytes": 16 * 8 * 2}}


def _tensors(code):
    rng = np.random.default_rng(code)
    return {k: rng.standard_normal(m["shape"]).astype(np.float16) for k, m in _info().items()}


def _loader(prefix, idle):
    from katz_b200.lora_shm import LoraShmLoader
    ld = LoraShmLoader(0, 1, _info(), _tensors, prefix=prefix)
    try:
        ld.serve(idle_timeout_s=idle)
    finally:
        ld.close()


def test_shm_protocol_round_trip():
    from katz_b200.lora_shm import LoraShmClient
    prefix = "katzt%d_" % os.getpid()
    ctx = mp.get_context("spawn")
    p = ctx.Process(target=_loader, args=(prefix, 60.0))
    p.start()
    cl = LoraShmClient([_info()], prefix=prefix, attach_timeout_s=60)
    try:
        assert cl.status() == 0 and not cl.ready()
        for code in (1, 2):
            cl.request([code])
            cl.wait(timeout_s=60)
            assert cl.status() == 10
            got = cl.gather(0, "cpu")
            for k, v in _tensors(code).items():
                assert torch.equal(got[k], torch.from_numpy(v))
            cl.clear()
            assert cl.status() == 0
        with pytest.raises(Exception):
            cl.request([0])
        cl.quit()
        p.join(timeout=30)
        assert p.exitcode == 0
    finally:
        cl.close()
        if p.is_alive():
            p.kill()


def test_reader_times_out_on_a_dead_loader():
    from katz_b200 import KatzError
    from katz_b200.lora_shm import LoraShmClient
    prefix = "katzu%d_" % os.getpid()
    with pytest.raises(KatzError):
        LoraShmClient([_info()], prefix=prefix, attach_timeout_s=0.3)
    # a loader that never gets a request gives up instead of spinning forever
    from katz_b200.lora_shm import LoraShmLoader
    ld = LoraShmLoader(0, 1, _info(), _tensors, prefix=prefix)
    try:
        with pytest.raises(KatzError):
            ld.serve(idle_timeout_s=0.2)
        cl = LoraShmClient([_info()], prefix=prefix, attach_timeout_s=5)
        cl.request([1])
        with pytest.raises(KatzError):
            cl.wait(timeout_s=0.2)          # nobody is serving
        cl.close()
    finally:
        ld.close()
