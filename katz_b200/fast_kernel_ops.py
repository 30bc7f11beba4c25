"""`TORCH_LIBRARY(fast_kernel)` equivalent: the two operators of the reference extension
(fast_kernel/csrc/main.cpp:10-12, bind.cu:12-15), same schemas, implemented over the C ABI.

  fast_kernel::group_norm_fp16(Tensor x, Tensor y, float eps, int num_groups, str activation, Tensor weight,
                               Tensor bias, bool affine, bool channels_last) -> ()
  fast_kernel::fast_gelu_mul_fp16(Tensor x, Tensor m) -> Tensor

As in the reference (group_norm.cu:264-273 -> :225-233,162) the ninth argument is forwarded as `channels_first`: the
fork calls it with False for NHWC-contiguous input (normalization.py:90-91).
"""
import torch

from . import ops
from .ops import ACT_NONE, ACT_SILU

# The schemas torch infers from the reference's C++ signatures (group_norm.cuh:7-15, gelu.cuh:44): plain `Tensor`
# arguments (weight and bias are NOT optional, `y` carries no alias annotation although it is written), registered for
# every backend at once under CompositeExplicitAutograd as bind.cu:13-14 does.
GROUP_NORM_SCHEMA = ("group_norm_fp16(Tensor x, Tensor y, float eps, int num_groups, str activation, Tensor weight, "
                     "Tensor bias, bool affine, bool channels_last) -> ()")
GELU_MUL_SCHEMA = "fast_gelu_mul_fp16(Tensor x, Tensor m) -> Tensor"
_lib = torch.library.Library("fast_kernel", "DEF")
_lib.define(GROUP_NORM_SCHEMA)
_lib.define(GELU_MUL_SCHEMA)


def _group_norm_fp16(x, y, eps, num_groups, activation, weight, bias, affine, channels_last):
    if activation == "none":
        act = ACT_NONE
    elif activation == "silu":
        act = ACT_SILU
    else:
        # the reference prints and returns without writing (group_norm.cu:219-221)
        print("Unsupported activation: %s" % activation)
        return
    channels_first = bool(channels_last)
    g = weight if affine else None
    b = bias if affine else None
    if x.dim() != 4:
        raise RuntimeError("group_norm_fp16 expects a 4-D tensor")
    if channels_first:
        ops.group_norm_nchw(x.contiguous(), g, b, num_groups, eps, act, out=y)
    else:
        # logical NCHW shape, NHWC memory
        B, C, H, W = x.shape
        xv = x.permute(0, 2, 3, 1)
        yv = y.permute(0, 2, 3, 1)
        if not xv.is_contiguous() or not yv.is_contiguous():
            raise RuntimeError("group_norm_fp16: x and y must be channels-last contiguous")
        ops.group_norm_nhwc(xv, g, b, num_groups, eps, act, out=yv)


def _fast_gelu_mul_fp16(x, m):
    if x.shape != m.shape:
        raise RuntimeError("Input tensors x and m must have the same shape.")
    if not x.is_contiguous():
        raise RuntimeError("Input tensor x must be contiguous.")
    if not m.is_contiguous():
        raise RuntimeError("Input tensor m must be contiguous.")
    return ops.fast_gelu_mul(x, m)


_lib.impl("group_norm_fp16", _group_norm_fp16, "CompositeExplicitAutograd")
_lib.impl("fast_gelu_mul_fp16", _fast_gelu_mul_fp16, "CompositeExplicitAutograd")
