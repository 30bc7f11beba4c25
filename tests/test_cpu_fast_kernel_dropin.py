"""CPU: the drop-in `fast_kernel` package registers the two operators with the schemas torch infers from the reference's
C++ signatures (fast_kernel/csrc/group_norm.cuh:7-15, gelu.cuh:44, registered in bind.cu:13-14), and — where a checkout
of the reference is present (the REFERENCE_ROOT variable, or the default location below) — the reference fork's own
diffusers/models/normalization.py and activations.py import against THIS package and reach its operators
(normalization.py:23,91; activations.py:21,145). Nothing is computed: there is no GPU here, and the operators refuse CPU
tensors instead of falling back."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("REFERENCE_ROOT", "/root/reference")


def test_ops_are_registered_with_the_reference_schemas():
    import fast_kernel  # noqa: F401  (import side effect: registration)
    gn = torch.ops.fast_kernel.group_norm_fp16.default._schema
    ge = torch.ops.fast_kernel.fast_gelu_mul_fp16.default._schema
    assert str(gn) == ("fast_kernel::group_norm_fp16(Tensor x, Tensor y, float eps, int num_groups, str activation, "
                       "Tensor weight, Tensor bias, bool affine, bool channels_last) -> ()")
    assert str(ge) == "fast_kernel::fast_gelu_mul_fp16(Tensor x, Tensor m) -> Tensor"
    # one registration for every backend, as the reference's CompositeExplicitAutograd dispatch: a CPU tensor reaches the
    # katz_b200 implementation, which refuses it (no CPU path) instead of "no kernel for backend CPU"
    x = torch.zeros(1, 32, 2, 2, dtype=torch.float16).contiguous(memory_format=torch.channels_last)
    with pytest.raises(RuntimeError, match="CUDA fp16 tensor"):
        torch.ops.fast_kernel.group_norm_fp16(x, torch.empty_like(x), 1e-5, 32, "silu", torch.ones(32).half(),
                                              torch.zeros(32).half(), True, False)
    v = torch.zeros(4, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA fp16 tensor"):
        torch.ops.fast_kernel.fast_gelu_mul_fp16(v, v)
    with pytest.raises(RuntimeError, match="same shape"):
        torch.ops.fast_kernel.fast_gelu_mul_fp16(v, v[:, :1])


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "diffusers-hf", "src", "diffusers")),
                    reason="no checkout of the reference here")
def test_reference_fork_modules_import_and_call_this_fast_kernel():
    code = textwrap.dedent("""
        import os, sys
        sys.path.insert(0, %r)                       # this repository: provides `fast_kernel`
        sys.path.insert(1, os.path.join(%r, "diffusers-hf", "src"))
        os.environ["ENABLE_FUSED_NORM_SILU"] = "1"
        os.environ["ENABLE_FUSED_GEGLU"] = "1"
        import huggingface_hub
        if not hasattr(huggingface_hub, "cached_download"):
            huggingface_hub.cached_download = huggingface_hub.hf_hub_download
        import transformers.utils as tu
        if not hasattr(tu, "FLAX_WEIGHTS_NAME"):
            tu.FLAX_WEIGHTS_NAME = "flax_model.msgpack"
        import torch
        import fast_kernel
        assert fast_kernel.__file__.startswith(%r), fast_kernel.__file__
        from diffusers.models import normalization, activations
        assert normalization.fast_kernel is fast_kernel and activations.fast_kernel is fast_kernel
        norm, act = normalization.fused_norm_silu(64)       # the fork's fused GroupNorm + SiLU module
        assert isinstance(norm, normalization.GroupNorm)
        x = torch.randn(1, 64, 4, 4).half()
        try:
            norm.half()(x)
        except RuntimeError as e:
            assert "CUDA fp16 tensor" in str(e), e           # reached katz_b200's operator, which has no CPU path
        else:
            raise SystemExit("the fork's GroupNorm did not call fast_kernel.group_norm_fp16")
        g = activations.GEGLU(64, 128).half()
        try:
            g(torch.randn(2, 8, 64).half())
        except RuntimeError as e:
            assert "CUDA fp16 tensor" in str(e), e
        else:
            raise SystemExit("the fork's GEGLU did not call fast_kernel.fast_gelu_mul_fp16")
        print("dropin-ok")
    """) % (ROOT, REF, ROOT)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "dropin-ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
