"""Drop-in for the reference's `fast_kernel` package (diffusers-hf/src/fast_kernel/fast_kernel/__init__.py:1-6):
importing it registers `torch.ops.fast_kernel.group_norm_fp16` and `torch.ops.fast_kernel.fast_gelu_mul_fp16`, which
diffusers/models/normalization.py:91 and diffusers/models/activations.py:145 call. The ops run the sm_100a kernels of
libkatz_b200.so; there is no fallback."""
try:
    import torch  # noqa: F401
    from katz_b200 import fast_kernel_ops as _C  # noqa: F401
except ImportError:
    print("Failed to import fast_kernel._C")
    raise
