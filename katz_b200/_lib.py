"""ctypes binding of libkatz_b200.so (the C ABI declared in include/katz_b200.h).

There is no CPU fallback: if the shared library is missing or an entry point fails, the caller gets an exception.
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_longlong, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkatz_b200.so")

KATZ_DTYPE_F16 = 0
KATZ_DTYPE_F32 = 1
ACT_NONE = 0
ACT_SILU = 1
LORA_MAX_ADAPTERS = 4

_ERRORS = {
    -1: "invalid argument (null pointer or bad enum)",
    -2: "pointer or stride not aligned as the kernel requires",
    -3: "shape outside what the kernel supports",
    -4: "driver entry point or device set-up missing",
    -5: "a bounded device-side wait gave up",
}


class KatzError(RuntimeError):
    pass


class LoraLayer(Structure):
    """Mirror of `struct katz_lora_layer`."""
    _fields_ = [
        ("W", c_void_p),
        ("W0", c_void_p),
        ("B", c_void_p * LORA_MAX_ADAPTERS),
        ("A", c_void_p * LORA_MAX_ADAPTERS),
        ("rank", c_int * LORA_MAX_ADAPTERS),
        ("scale", c_float * LORA_MAX_ADAPTERS),
        ("out_features", c_int),
        ("in_features", c_int),
        ("n_lora", c_int),
        ("reserved_", c_int),
    ]


_V, _I, _L, _F = c_void_p, c_int, c_longlong, c_float


class LinearExtras(Structure):
    """Mirror of `struct katz_linear_extras`."""
    _fields_ = [("ln_stats", c_void_p), ("ln_c12", c_void_p), ("ln_slots", c_int), ("ln_eps", c_float), ("stats_out", c_void_p)]


# name -> (restype, argtypes). Every symbol include/katz_b200.h declares must be listed here; a test checks it.
SIGNATURES = {
    "katz_abi_version": (_I, []),
    "katz_build_arch": (c_char_p, []),
    "katz_lora_tile_rows": (_I, [_I]),
    "katz_lora_tile_cols": (_I, []),
    "katz_lora_layer_check": (_I, [POINTER(LoraLayer), _I]),
    "katz_lora_table_check": (_I, [POINTER(LoraLayer), _I, _I, POINTER(c_int)]),
    "katz_lora_merge": (_I, [_V, _V, _I, _I, _I, _F, _I, _I, _V, _V]),
    "katz_lora_encode_tile_maps": (_I, [POINTER(LoraLayer), _I, _V]),
    "katz_lora_fast_tile_rows": (_I, [_I]),
    "katz_lora_fast_tile_cols": (_I, [_I]),
    "katz_lora_encode_tile_maps_dtype": (_I, [POINTER(LoraLayer), _I, _I, _V]),
    "katz_group_norm_scratch_bytes": (_L, [_I, _I, _I, _I]),
    "katz_group_norm_nhwc_f16": (_I, [_V, _V, _V, _V, _I, _I, _I, _I, _F, _I, _V, _L, _V]),
    "katz_group_norm_stats_nhwc_f16": (_I, [_V, _V, _I, _I, _I, _I, _V, _L, _V]),
    "katz_group_norm_apply_nhwc_f16": (_I, [_V, _V, _V, _I, _V, _V, _I, _I, _I, _I, ctypes.c_double, _F, _I, _V]),
    "katz_group_norm_static_scratch_bytes": (_L, []),
    "katz_group_norm_static_scratch_reset": (_I, [_V]),
    "katz_group_norm_nhwc_f16_noalloc": (_I, [_V, _V, _V, _V, _I, _I, _I, _I, _F, _I, _V]),
    "katz_group_norm_nchw_f16": (_I, [_V, _V, _V, _V, _I, _I, _I, _I, _F, _I, _V]),
    "katz_fast_gelu_mul_f16": (_I, [_V, _V, _V, _L, _V]),
    "katz_layer_norm_f16": (_I, [_V, _V, _V, _V, _I, _I, _F, _V]),
    "katz_geglu_erf_f16": (_I, [_V, _V, _L, _I, _I, _V]),
    "katz_linear_f16_mma": (_I, [_V, _I, _V, _V, _I, _I, _I, _I, _V, _V, _I, _I, _V, _I, _I, _F, _V]),
    "katz_linear_f16": (_I, [_V, _I, _V, _V, _I, _I, _I, _I, _V, _V, _I, _I, _V, _I, _I, _F, _V]),
    "katz_linear_geglu_f16": (_I, [_V, _I, _V, _V, _I, _I, _I, _I, _V, _V]),
    "katz_ln_fold_f16": (_I, [_V, _V, _V, _V, _V, _V, _I, _I, _V]),
    "katz_linear_ex_f16": (_I, [_V, _I, _V, _V, _I, _I, _I, _I, _V, _V, _I, _I, _V, _I, _I, _F, POINTER(LinearExtras), _V]),
    "katz_linear_geglu_ex_f16": (_I, [_V, _I, _V, _V, _I, _I, _I, _I, _V, POINTER(LinearExtras), _V]),
    "katz_conv3x3_nhwc_f16": (_I, [_V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _V, _V, _I, _V, _I, _F, _V]),
    "katz_tc05_status": (_I, []),
    "katz_tc05_clear_status": (_I, []),
    "katz_upsample_nearest2x_nhwc_f16": (_I, [_V, _V, _I, _I, _I, _I, _V]),
    "katz_conv2d_nhwc_f16_mma": (_I, [_V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _V, _V, _I, _V, _I, _F, _V]),
    "katz_attention_f16": (_I, [_V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _L, _L, _L, _L, _F, _I, _L, _V]),
    "katz_conv3x3_small_nhwc_f16": (_I, [_V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _V, _I, _V]),
    "katz_attention_split_scratch_bytes": (_L, []),
    "katz_attention_split_f16": (_I, [_V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _L, _L, _L, _L, _F, _I, _L, _V, _L, _V]),
    "katz_attention_peer_f16": (_I, [_V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _L, _L, _L, _L, _F, _I, _L, _V, _L, _V, _I, _V]),
    "katz_attention_f16_mma": (_I, [_V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _L, _L, _L, _L, _F, _I, _L, _V]),
    "katz_residual_intake_f16": (_I, [_V, _V, POINTER(c_void_p), POINTER(c_float), _I, _L, _V]),
    "katz_timestep_embedding_f16": (_I, [_V, _V, _I, _I, _I, _V]),
    "katz_silu_f16": (_I, [_V, _V, _L, _V]),
    "katz_softmax_rows_f16": (_I, [_V, _V, _I, _I, _L, _L, _V]),
    "katz_halo_assemble_f16": (_I, [_V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _V]),
    "katz_peer_ctrl_bytes": (_I, []),
    "katz_peer_arena_alloc": (_I, [_L, POINTER(c_void_p)]),
    "katz_peer_arena_free": (_I, [_V]),
    "katz_peer_ipc_handle_bytes": (_I, []),
    "katz_peer_ipc_export": (_I, [_V, _V]),
    "katz_peer_ipc_open": (_I, [_V, POINTER(c_void_p)]),
    "katz_peer_ipc_close": (_I, [_V]),
    "katz_peer_allgather": (_I, [_V, _L, _L, _L, _L, POINTER(ctypes.c_ulonglong), _I, _I, _V]),
    "katz_peer_push": (_I, [_V, _L, _L, _L, _L, POINTER(ctypes.c_ulonglong), _I, _I, _V]),
    "katz_peer_status": (_I, [_V]),
    "katz_peer_clear_status": (_I, [_V]),
    "katz_add_f16": (_I, [_V, _V, _V, _L, _V]),
    "katz_concat_channels_f16": (_I, [_V, _V, _V, _L, _I, _I, _V]),
    "katz_nchw_to_nhwc_f16": (_I, [_V, _V, _I, _I, _I, _I, _V]),
    "katz_nhwc_to_nchw_f16": (_I, [_V, _V, _I, _I, _I, _I, _V]),
    "katz_euler_scale_input": (_I, [_V, _V, _L, _F, _I, _I, _V]),
    "katz_euler_cfg_step": (_I, [_V, _V, _V, _L, _F, _F, _F, _I, _V]),
}

_lib = None


def load():
    """Load the shared library once. Raises KatzError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise KatzError(
            "libkatz_b200.so is not built (%s missing). Run `python -m katz_b200.build` or "
            "`python -c 'import __graft_entry__ as g; g.build()'`. There is no CPU fallback." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise KatzError("libkatz_b200.so does not export %s; rebuild it" % name) from e
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code, what):
    """Turn a non-zero return code of an entry point into an exception."""
    if code == 0:
        return
    if code < 0:
        raise KatzError("%s: %s (code %d)" % (what, _ERRORS.get(code, "argument error"), code))
    raise KatzError("%s: CUDA error %d" % (what, code))


# kernels launched per successful entry-point call (everything else launches one)
_KERNELS_PER_CALL = {"katz_group_norm_nhwc_f16": 2}
_launches = 0


def launch_count():
    """Kernels this process has launched through the library so far."""
    return _launches


def note_launches(n):
    global _launches
    _launches += n


def call(name, *args):
    global _launches
    lib = load()
    check(getattr(lib, name)(*args), name)
    _launches += _KERNELS_PER_CALL.get(name, 1)
