"""CPU: the C-ABI library builds, loads, and exports every symbol include/katz_b200.h declares; host-side checks that
need no device."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "katz_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(katz_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from katz_b200 import _lib, build
    build.build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), "declared in katz_b200.h but not exported: %s" % name
    assert set(declared) == set(_lib.SIGNATURES.keys()), set(declared) ^ set(_lib.SIGNATURES.keys())
    loaded = _lib.load()
    assert loaded.katz_abi_version() == 1
    assert loaded.katz_build_arch() == b"sm_100a"


def test_argument_errors_need_no_device():
    from katz_b200 import _lib
    lib = _lib.load()
    assert lib.katz_group_norm_scratch_bytes(2, 4096, 320, 32) > 0
    assert lib.katz_group_norm_scratch_bytes(0, 4096, 320, 32) == -1
    assert lib.katz_lora_tile_rows(_lib.KATZ_DTYPE_F16) == 128 and lib.katz_lora_tile_cols() == 128
    e = _lib.LoraLayer()
    assert lib.katz_lora_layer_check(ctypes.byref(e), 0) < 0           # null W
    assert lib.katz_linear_f16_mma(None, 0, None, None, 0, 1, 1, 8, None, None, 0, 0, None, 0, 0, 1.0, None) == -1
    assert lib.katz_group_norm_apply_nhwc_f16(None, None, None, 1, None, None, 1, 1, 8, 1, 1.0, 1e-5, 0, None) == -1
    assert lib.katz_attention_f16_mma(1, 1, 1, 1, 1, 1, 64, 64, 32, 64, 64, 64, 64, 0, 0, 0, 0, 0.125, 0, 0, None) == -3
    with pytest.raises(_lib.KatzError):
        _lib.check(-2, "x")


def test_ops_refuse_cpu_tensors():
    from katz_b200 import KatzError, ops
    from katz_b200.unet import KatzUNet
    from katz_b200.params import TINY_UNET_CONFIG
    with pytest.raises(KatzError):
        ops.linear(torch.zeros(8, 8, dtype=torch.float16), torch.zeros(8, 8, dtype=torch.float16))
    with pytest.raises(KatzError):
        KatzUNet(TINY_UNET_CONFIG, device="cpu")


def test_euler_schedule_host_mirror(golden_dir):
    import numpy as np
    from katz_b200.scheduler import EulerSchedule
    g = np.load(os.path.join(golden_dir, "euler_sdxl.npz"))
    s = EulerSchedule().set_timesteps(50)
    np.testing.assert_array_equal(s.timesteps.numpy(), g["timesteps"])
    np.testing.assert_array_equal(s.sigmas.numpy(), g["sigmas"])
    assert abs(s.init_noise_sigma - float(g["init_noise_sigma"])) < 1e-6
    with pytest.raises(NotImplementedError):
        EulerSchedule(beta_schedule="squaredcos_cap_v2")


def test_binding_arity_matches_the_header():
    """Every ctypes signature has as many arguments as the header's prototype (a drifted binding corrupts the call)."""
    from katz_b200 import _lib
    text = open(os.path.join(ROOT, "include", "katz_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = dict(re.findall(r"\b(katz_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S))
    assert set(protos) == set(_lib.SIGNATURES)
    for name, params in protos.items():
        params = params.strip()
        n = 0 if params in ("", "void") else len([p for p in params.split(",") if p.strip()])
        assert n == len(_lib.SIGNATURES[name][1]), "%s: header has %d parameters, binding %d" % (name, n, len(_lib.SIGNATURES[name][1]))
