"""TEST INFRASTRUCTURE — CPU oracle of the two `fast_kernel` operators and of the small per-step kernels.

fast_gelu_mul restates FusedFastGeluMulFunctor<Half> (fast_kernel/csrc/gelu.cuh:29-42): every operation is a half
operation except the tanh, taken in float. group_norm restates GroupNormFP16 (fast_kernel/csrc/group_norm.cu:155-274):
fp32 statistics over each (batch, group), affine, optional SiLU, fp16 output. No reference test covers these operators
(the reference ships none for its extension), so their parity is pinned only by the formulas — "parity unpinned" for
these two against reference-run outputs. Only tests/, smoke() and bench.py's CPU baseline import this file.
"""
import numpy as np
import torch


def fast_gelu_mul(x, m):
    """x, m: fp16 numpy arrays."""
    h = np.float16
    x = x.astype(h)
    alpha, beta = h(0.7978845608028654), h(0.044714998453855515)
    t = (beta * x).astype(h)
    t = (t * x).astype(h)
    t = (t * x).astype(h)
    t = (x + t).astype(h)
    t = (alpha * t).astype(h)
    th = np.tanh(t.astype(np.float32)).astype(h)
    r = (h(0.5) * x).astype(h)
    r = (r * (h(1.0) + th).astype(h)).astype(h)
    return (r * m.astype(h)).astype(h)


def group_norm(x_nchw, groups, weight, bias, eps, silu):
    """x: fp16 torch tensor [B,C,H,W]; statistics and affine in fp32; returns fp16."""
    y = torch.nn.functional.group_norm(x_nchw.float(), groups, None if weight is None else weight.float(),
                                       None if bias is None else bias.float(), eps)
    if silu:
        y = torch.nn.functional.silu(y)
    return y.half()


def geglu_erf(hg):
    """activations.py:146-149 on an fp16 tensor: chunk, gelu (rounded to half), multiply (rounded to half)."""
    h, g = hg.chunk(2, dim=-1)
    return (h.float() * torch.nn.functional.gelu(g.float()).half().float()).half()
