"""Tensor-level wrappers over the C ABI: each takes torch CUDA tensors, checks layout, and launches on the current
torch stream. No op here computes anything in torch; a missing library or a failing launch raises KatzError."""
import ctypes
import os

import torch

from . import _lib
from ._lib import ACT_NONE, ACT_SILU, KatzError, call  # noqa: F401


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _f16(t, name):
    if t.dtype != torch.float16 or not t.is_cuda:
        raise KatzError("%s must be a CUDA fp16 tensor (got %s on %s)" % (name, t.dtype, t.device))
    return t


def _use_tc05():
    return os.environ.get("KATZ_GEMM", "tc05") != "mma"


def _al16(t):
    return t is None or t.data_ptr() % 16 == 0


def _tc05_linear_ok(x, w, bias, residual, rowvec, out):
    """Shapes/alignments the tcgen05 GEMM takes; anything else goes to the mma.sync kernel."""
    M, K = x.shape
    N = w.shape[0]
    if K % 64 or N % 8 or x.stride(0) % 8 or out.stride(0) % 8:
        return False
    if not (_al16(x) and _al16(w) and _al16(out) and _al16(bias) and _al16(residual) and _al16(rowvec)):
        return False
    if residual is not None and residual.stride(0) % 8:
        return False
    if rowvec is not None and rowvec.stride(0) % 8:
        return False
    return True


def _tc05_rowvec_ok(rowvec, rows_per_batch):
    """The tcgen05 epilogue adds one row vector per 128-row tile."""
    return rowvec is None or (rows_per_batch > 0 and rows_per_batch % 128 == 0)


def gemm_kernel_name():
    """Which GEMM family `linear` dispatches large aligned shapes to."""
    return "tcgen05" if _use_tc05() else "mma.sync"


def tc05_status():
    """Status word of the tcgen05 kernels (0 = no bounded wait ever gave up). Synchronises the device."""
    return _lib.load().katz_tc05_status()


class LnFold:
    """A LayerNorm folded into the linear layer that consumes it: `wf` = W diag(gamma) (fp16), `c12` = per output column
    (sum_k W'[n,k], sum_k W[n,k] beta[k] + bias[n]) in fp32, `eps` the norm's epsilon. Built by `ln_fold`."""

    def __init__(self, wf, c12, eps):
        self.wf, self.c12, self.eps = wf, c12, float(eps)


def ln_fold(w, gamma, beta, bias=None, eps=1e-5, out=None):
    """(Re)compute the folded constants of LayerNorm(gamma, beta) followed by linear(w, bias). Pass `out` (an LnFold) to
    refresh it in place after `w` changed."""
    _f16(w, "w"), _f16(gamma, "gamma"), _f16(beta, "beta")
    if not w.is_contiguous() or w.dim() != 2 or gamma.numel() != w.shape[1] or beta.numel() != w.shape[1]:
        raise KatzError("ln_fold: w must be a contiguous [N, K] tensor and gamma/beta [K]")
    N, K = w.shape
    if out is None:
        out = LnFold(torch.empty_like(w), torch.empty((N, 2), dtype=torch.float32, device=w.device), eps)
    call("katz_ln_fold_f16", _p(w), _p(gamma), _p(beta), _p(bias), _p(out.wf), _p(out.c12), N, K, _stream())
    return out


def ln_fusable(M, K, N):
    """Whether `linear(layer_norm(x), w)` with x [M, K], w [N, K] can run as one folded GEMM on the tcgen05 path."""
    return _use_tc05() and K % 64 == 0 and N % 8 == 0


def _extras(x, ln, ln_stats, stats_out, M, K, N):
    from ._lib import LinearExtras
    ex = LinearExtras()
    keep = []
    if ln is not None:
        if ln_stats is None or ln_stats.dtype != torch.float32 or not ln_stats.is_contiguous() or ln_stats.dim() != 3 \
                or ln_stats.shape[1] != M or ln_stats.shape[2] != 2 or ln_stats.shape[0] != (K + 31) // 32:
            raise KatzError("folded LayerNorm needs the producer's statistics [ceil(K/32), M, 2] fp32")
        ex.ln_stats, ex.ln_c12, ex.ln_slots, ex.ln_eps = ln_stats.data_ptr(), ln.c12.data_ptr(), ln_stats.shape[0], ln.eps
    if stats_out is True:
        stats_out = torch.empty(((N + 31) // 32, M, 2), dtype=torch.float32, device=x.device)
    if stats_out is not None:
        if stats_out.dtype != torch.float32 or not stats_out.is_contiguous() or tuple(stats_out.shape) != ((N + 31) // 32, M, 2):
            raise KatzError("stats_out must be a contiguous fp32 [ceil(N/32), M, 2] tensor")
        ex.stats_out = stats_out.data_ptr()
    return ex, stats_out


def feed_forward_geglu(x, w, bias, out=None, ln=None, ln_stats=None):
    """GEGLU feed-forward projection: x[M,K], w[2F,K] (the unsplit `proj`), bias[2F] -> [M,F] = h * gelu(g).
    One fused tcgen05 GEMM when the shape allows, else GEMM + gating kernel. With `ln` (an LnFold whose `wf` replaces `w`;
    `bias` is already inside it) and `ln_stats` (the row statistics of x) x is the input of the LayerNorm."""
    _f16(x, "x")
    if ln is not None:
        w, bias = ln.wf, None
    _f16(w, "w")
    M, K = x.shape
    F = w.shape[0] // 2
    if out is None:
        out = torch.empty((M, F), dtype=torch.float16, device=x.device)
    fused_ok = (_use_tc05() and os.environ.get("KATZ_FUSED_GEGLU", "1") == "1" and K % 64 == 0 and F % 16 == 0
                and x.stride(1) == 1 and x.stride(0) % 8 == 0 and w.is_contiguous() and _al16(x) and _al16(w) and _al16(out)
                and _al16(bias) and out.stride(0) % 8 == 0)
    if ln is not None:
        if not fused_ok:
            raise KatzError("feed_forward_geglu: this shape cannot take a folded LayerNorm")
        ex, _ = _extras(x, ln, ln_stats, None, M, K, 2 * F)
        call("katz_linear_geglu_ex_f16", _p(x), x.stride(0), _p(w), _p(out), out.stride(0), M, F, K, None, ctypes.byref(ex), _stream())
        return out
    if fused_ok:
        call("katz_linear_geglu_f16", _p(x), x.stride(0), _p(w), _p(out), out.stride(0), M, F, K, _p(bias), _stream())
        return out
    return geglu_erf(linear(x, w, bias), out=out)


def upsample_nearest2x(x, out=None):
    _f16(x, "x")
    B, H, W, C = x.shape
    if out is None:
        out = torch.empty((B, 2 * H, 2 * W, C), dtype=torch.float16, device=x.device)
    call("katz_upsample_nearest2x_nhwc_f16", _p(x), _p(out), B, H, W, C, _stream())
    return out


def linear(x, w, bias=None, residual=None, act=ACT_NONE, rowvec=None, rows_per_batch=0, out=None, out_scale=1.0,
           ln=None, ln_stats=None, stats_out=None):
    """out[M,N] = x[M,K] @ w[N,K]^T (+bias) (+rowvec[m // rows_per_batch]) -> act -> (+residual) * out_scale.
    `x`, `residual`, `out` may be row-strided 2-D views (unit column stride).
    Folded LayerNorm: with `ln` (an LnFold; its `wf` replaces `w` and holds the bias) and `ln_stats` the call computes
    linear(layer_norm(x)); with `stats_out=True` (or a buffer) it also returns the row statistics of its own output for the
    next folded LayerNorm: `(out, stats)`."""
    _f16(x, "x")
    if ln is not None:
        w, bias = ln.wf, None
    _f16(w, "w")
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise KatzError("linear: shape mismatch x%s w%s" % (tuple(x.shape), tuple(w.shape)))
    if x.stride(1) != 1 or not w.is_contiguous():
        raise KatzError("linear: x must have unit column stride and w must be contiguous")
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=x.device)
    if out.stride(1) != 1 or out.shape != (M, N):
        raise KatzError("linear: bad out")
    if residual is not None and (residual.shape != (M, N) or residual.stride(1) != 1):
        raise KatzError("linear: bad residual")
    tc05 = _use_tc05() and _tc05_linear_ok(x, w, bias, residual, rowvec, out) and _tc05_rowvec_ok(rowvec, rows_per_batch)
    if ln is not None or stats_out is not None:
        if not tc05:
            raise KatzError("linear: this shape cannot take a folded LayerNorm / emit row statistics (tcgen05 path only)")
        ex, stats = _extras(x, ln, ln_stats, stats_out, M, K, N)
        call("katz_linear_ex_f16", _p(x), x.stride(0), _p(w), _p(out), out.stride(0), M, N, K, _p(bias), _p(rowvec),
             rowvec.stride(0) if rowvec is not None else 0, rows_per_batch, _p(residual),
             residual.stride(0) if residual is not None else 0, act, float(out_scale), ctypes.byref(ex), _stream())
        return (out, stats) if stats is not None else out
    name = "katz_linear_f16" if tc05 else "katz_linear_f16_mma"
    call(name, _p(x), x.stride(0), _p(w), _p(out), out.stride(0), M, N, K, _p(bias), _p(rowvec),
         rowvec.stride(0) if rowvec is not None else 0, rows_per_batch, _p(residual),
         residual.stride(0) if residual is not None else 0, act, float(out_scale), _stream())
    return out


def conv2d(x, w, bias=None, ksize=3, stride=1, pad=1, upsample=False, x2=None, rowvec=None, residual=None,
           act=ACT_NONE, out=None, out_scale=1.0, pad_h=None):
    """NHWC convolution. x: [B,Hs,Ws,C1] (+ optional x2 [B,Hs,Ws,C2] concatenated along channels); w: [Cout,k,k,C1+C2].
    With upsample=True the input is read through a nearest 2x upsample. rowvec: [B, >=Cout] row-strided view added per
    batch element; residual: [B,Hout,Wout,Cout]. `pad_h` overrides the vertical padding (0 for a row shard whose input
    already carries its halo rows)."""
    _f16(x, "x"), _f16(w, "w")
    if not x.is_contiguous() or not w.is_contiguous():
        raise KatzError("conv2d: x and w must be contiguous")
    B, Hs, Ws, C1 = x.shape
    C2 = 0
    if x2 is not None:
        if not x2.is_contiguous() or x2.shape[:3] != x.shape[:3]:
            raise KatzError("conv2d: bad x2")
        C2 = x2.shape[3]
    Cout = w.shape[0]
    if w.numel() != Cout * ksize * ksize * (C1 + C2):
        raise KatzError("conv2d: weight does not match [Cout,k,k,Cin]")
    ph = pad if pad_h is None else pad_h
    Hin, Win = (Hs * 2, Ws * 2) if upsample else (Hs, Ws)
    Hout = (Hin + 2 * ph - ksize) // stride + 1
    Wout = (Win + 2 * pad - ksize) // stride + 1
    if out is None:
        out = torch.empty((B, Hout, Wout, Cout), dtype=torch.float16, device=x.device)
    if residual is not None and (tuple(residual.shape) != (B, Hout, Wout, Cout) or not residual.is_contiguous()):
        raise KatzError("conv2d: bad residual")
    tw = min(Wout, 128)
    if (_use_tc05() and ksize == 3 and stride in (1, 2) and pad == 1 and ph in (0, 1) and x2 is None and C1 % 64 == 0
            and Cout % 8 == 0 and tw >= 8 and (tw & (tw - 1)) == 0 and Wout % tw == 0 and (stride == 1 or Win % 2 == 0)
            and _al16(x) and _al16(w) and _al16(out)
            and _al16(bias) and _al16(residual) and (rowvec is None or (_al16(rowvec) and rowvec.stride(0) % 8 == 0))):
        src = upsample_nearest2x(x) if upsample else x
        call("katz_conv3x3_nhwc_f16", _p(src), _p(w), _p(out), B, Hin, Win, C1, Cout, stride, ph, _p(bias), _p(rowvec),
             rowvec.stride(0) if rowvec is not None else 0, _p(residual), act, float(out_scale), _stream())
        return out
    if (ksize == 3 and stride in (1, 2) and pad == 1 and ph in (0, 1) and x2 is None and not upsample and rowvec is None
            and residual is None and out_scale == 1.0 and C1 in (8, 16, 32) and Cout % 8 == 0 and Cout <= 1024
            and _al16(x) and _al16(w) and _al16(out) and _al16(bias) and os.environ.get("KATZ_CONV_SMALL", "1") != "0"):
        # few input channels (the ControlNet conditioning embedding): direct convolution from a shared-memory patch
        call("katz_conv3x3_small_nhwc_f16", _p(x), _p(w), _p(out), B, Hin, Win, C1, Cout, stride, ph, _p(bias), act, _stream())
        return out
    call("katz_conv2d_nhwc_f16_mma", _p(x), _p(x2), _p(w), _p(out), B, Hin, Win, C1, C2, Cout, ksize, stride, ph, pad,
         1 if upsample else 0, _p(bias), _p(rowvec), rowvec.stride(0) if rowvec is not None else 0, _p(residual), act,
         float(out_scale), _stream())
    return out


_gn_scratch = {}


def _scratch(device, nbytes):
    # one buffer per (device, stream): launches that share a scratch buffer must be ordered, and two branches of a CUDA
    # graph (the two halves of a CFG batch on two streams) are not
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    buf = _gn_scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        # zero-filled: the head of the scratch holds the GroupNorm ticket counters, which the kernels return to zero
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _gn_scratch[key] = buf
    return buf


def group_norm_nhwc(x, gamma, beta, groups, eps, act=ACT_NONE, out=None):
    """GroupNorm (+SiLU) over an NHWC tensor [B,H,W,C] (or [B,HW,C])."""
    _f16(x, "x")
    if not x.is_contiguous():
        raise KatzError("group_norm: x must be contiguous")
    B, C = x.shape[0], x.shape[-1]
    HW = x.numel() // (B * C)
    if out is None:
        out = torch.empty_like(x)
    lib = _lib.load()
    need = lib.katz_group_norm_scratch_bytes(B, HW, C, groups)
    if need < 0:
        raise KatzError("group_norm: bad shape")
    # The scratch buffer is shared by every GroupNorm call on this device: calls are ordered on one stream.
    scratch = _scratch(x.device, need)
    call("katz_group_norm_nhwc_f16", _p(x), _p(out), _p(gamma), _p(beta), B, HW, C, groups, float(eps), act,
         _p(scratch), scratch.numel(), _stream())
    return out


def group_norm_stats(x, groups):
    """fp64 (sum, sum of squares) per (batch, group) of an NHWC shard: [B, G, 2]. First half of a GroupNorm whose
    statistics span several GPUs."""
    _f16(x, "x")
    if not x.is_contiguous():
        raise KatzError("group_norm: x must be contiguous")
    B, C = x.shape[0], x.shape[-1]
    HW = x.numel() // (B * C)
    lib = _lib.load()
    need = lib.katz_group_norm_scratch_bytes(B, HW, C, groups)
    if need < 0:
        raise KatzError("group_norm: bad shape")
    scratch = _scratch(x.device, need)
    sums = torch.empty((B, groups, 2), dtype=torch.float64, device=x.device)
    call("katz_group_norm_stats_nhwc_f16", _p(x), _p(sums), B, HW, C, groups, _p(scratch), scratch.numel(), _stream())
    return sums


def group_norm_apply(x, sums, gamma, beta, groups, n_total, eps, act=ACT_NONE, out=None):
    """Second half: normalise the shard with the statistics of the whole tensor; n_total = elements per (batch, group)
    over the WHOLE tensor. sums: fp64 [B, G, 2] (already summed over the shards) or [P, B, G, 2] (one entry per shard,
    added here in shard order)."""
    _f16(x, "x")
    B, C = x.shape[0], x.shape[-1]
    HW = x.numel() // (B * C)
    if sums.dtype != torch.float64 or not sums.is_contiguous() or tuple(sums.shape[-3:]) != (B, groups, 2) or sums.dim() not in (3, 4):
        raise KatzError("group_norm_apply: sums must be a contiguous fp64 [B, G, 2] or [P, B, G, 2] tensor")
    n_parts = sums.shape[0] if sums.dim() == 4 else 1
    if out is None:
        out = torch.empty_like(x)
    call("katz_group_norm_apply_nhwc_f16", _p(x), _p(out), _p(sums), n_parts, _p(gamma), _p(beta), B, HW, C, groups,
         float(n_total), float(eps), act, _stream())
    return out


def group_norm_nchw(x, gamma, beta, groups, eps, act=ACT_NONE, out=None):
    _f16(x, "x")
    if not x.is_contiguous():
        raise KatzError("group_norm: x must be contiguous")
    B, C = x.shape[0], x.shape[1]
    HW = x.numel() // (B * C)
    if out is None:
        out = torch.empty_like(x)
    call("katz_group_norm_nchw_f16", _p(x), _p(out), _p(gamma), _p(beta), B, HW, C, groups, float(eps), act, _stream())
    return out


def layer_norm(x, gamma, beta, eps=1e-5, out=None):
    _f16(x, "x")
    if not x.is_contiguous():
        raise KatzError("layer_norm: x must be contiguous")
    C = x.shape[-1]
    rows = x.numel() // C
    if out is None:
        out = torch.empty_like(x)
    call("katz_layer_norm_f16", _p(x), _p(out), _p(gamma), _p(beta), rows, C, float(eps), _stream())
    return out


def geglu_erf(hg, out=None):
    """hg: [M, 2F] contiguous -> [M, F] = hg[:, :F] * gelu(hg[:, F:])."""
    _f16(hg, "hg")
    M, F2 = hg.shape
    F = F2 // 2
    if out is None:
        out = torch.empty((M, F), dtype=torch.float16, device=hg.device)
    call("katz_geglu_erf_f16", _p(hg), _p(out), M, F, hg.stride(0), _stream())
    return out


def fast_gelu_mul(x, m, out=None):
    _f16(x, "x"), _f16(m, "m")
    if x.shape != m.shape:
        raise KatzError("Input tensors x and m must have the same shape.")
    if not x.is_contiguous():
        raise KatzError("Input tensor x must be contiguous.")
    if not m.is_contiguous():
        raise KatzError("Input tensor m must be contiguous.")
    if out is None:
        out = torch.empty_like(x)
    call("katz_fast_gelu_mul_f16", _p(x), _p(m), _p(out), x.numel(), _stream())
    return out


def softmax_rows(x, out=None):
    """Row softmax of a 2-D fp16 matrix of logits (fp32 arithmetic); `out` may be `x`. Rows may be strided."""
    _f16(x, "x")
    if x.dim() != 2 or x.stride(1) != 1:
        raise KatzError("softmax_rows: x must be 2-D with unit column stride")
    if out is None:
        out = torch.empty_like(x)
    if out.shape != x.shape or out.stride(1) != 1 or out.dtype != torch.float16:
        raise KatzError("softmax_rows: bad out")
    call("katz_softmax_rows_f16", _p(x), _p(out), x.shape[0], x.shape[1], x.stride(0), out.stride(0), _stream())
    return out


_attn_scratch = {}


def _attention_scratch(device):
    """Scratch of the attention kernel's cut query tiles: one zero-filled buffer per device, of the size that is enough
    for every shape, allocated once (a captured graph keeps pointing at it)."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)      # per stream, as the GroupNorm scratch
    buf = _attn_scratch.get(key)
    if buf is None:
        buf = torch.zeros(int(_lib.load().katz_attention_split_scratch_bytes()), dtype=torch.uint8, device=device)
        _attn_scratch[key] = buf
    return buf


def attention(q, k, v, heads, out=None, scale=None, kv_chunks=None, peer=None):
    """q: [B,Sq,>=H*64] view, k/v: [B,Sk,...] views (unit last stride, any row/batch stride); returns [B,Sq,H*64].
    kv_chunks=(n_chunks, chunk_rows, chunk_stride): k/v describe the FIRST chunk ([B, chunk_rows, ...]); chunk c of the
    keys/values starts `c * chunk_stride` elements later (the [P, B, s, C] result of an all-gather of row shards).
    peer=(address of this rank's arena control words, this rank's chunk): the chunks were pushed WITHOUT waiting
    (PeerArena.allgather(wait=False)) and the kernel waits for each peer's flag before it first touches that peer's chunk."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _f16(t, n)
        if t.dim() != 3 or t.stride(2) != 1:
            raise KatzError("attention: %s must be [B,S,C] with unit last stride" % n)
    B, Sq, _ = q.shape
    Sk = k.shape[1]
    chunk_rows, chunk_stride = 0, 0
    if kv_chunks is not None:
        n_chunks, chunk_rows, chunk_stride = kv_chunks
        Sk = n_chunks * chunk_rows
    D = 64
    if out is None:
        out = torch.empty((B, Sq, heads * D), dtype=torch.float16, device=q.device)
    if scale is None:
        scale = D ** -0.5
    args = (_p(q), _p(k), _p(v), _p(out), B, heads, Sq, Sk, D, q.stride(1), k.stride(1), v.stride(1), out.stride(1),
            q.stride(0), k.stride(0), v.stride(0), out.stride(0), float(scale), chunk_rows, chunk_stride, _stream())
    strides_ok = all(t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0 and _al16(t) for t in (q, k, v, out))
    # KATZ_ATTN: "tc05" / "mma" force a kernel; by default a single key tile (cross-attention over 77 text tokens) goes to
    # the mma.sync kernel, whose CTAs share an SM (measured 9.5 us against 13.5 us for 2x20 heads x 1024 queries)
    mode = os.environ.get("KATZ_ATTN", "auto")
    if (_use_tc05() and (mode == "tc05" or (mode == "auto" and Sk > 128)) and strides_ok
            and (chunk_rows == 0 or (chunk_rows % 128 == 0 and chunk_stride % 8 == 0))):
        if peer is not None:
            scratch = _attention_scratch(q.device)
            call("katz_attention_peer_f16", *args[:-1], _p(scratch), scratch.numel(), ctypes.c_void_p(int(peer[0])), int(peer[1]),
                 args[-1])
        elif os.environ.get("KATZ_ATTN_SPLIT", "1") != "0":
            scratch = _attention_scratch(q.device)
            call("katz_attention_split_f16", *args[:-1], _p(scratch), scratch.numel(), args[-1])
        else:
            call("katz_attention_f16", *args)
    else:
        if peer is not None:
            raise KatzError("attention: chunks that are still in flight need the tcgen05 kernel (128-row chunks, aligned strides)")
        call("katz_attention_f16_mma", *args)
    return out


def residual_intake(src, residuals, scales, out=None):
    """out = src + half(sum_i scales[i] * residuals[i])."""
    _f16(src, "src")
    n = len(residuals)
    if out is None:
        out = torch.empty_like(src)
    ptrs = (ctypes.c_void_p * n)(*[r.data_ptr() for r in residuals])
    for r in residuals:
        _f16(r, "residual")
        if r.numel() != src.numel() or not r.is_contiguous():
            raise KatzError("residual_intake: residual shape/layout mismatch")
    sc = (ctypes.c_float * n)(*[float(s) for s in scales])
    call("katz_residual_intake_f16", _p(src), _p(out), ptrs, sc, n, src.numel(), _stream())
    return out


def timestep_embedding(t, dim, out=None):
    """t: fp32 CUDA tensor [rows] -> fp16 [rows, dim]."""
    if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
        raise KatzError("timestep_embedding: t must be a contiguous CUDA fp32 tensor")
    rows = t.numel()
    if out is None:
        out = torch.empty((rows, dim), dtype=torch.float16, device=t.device)
    call("katz_timestep_embedding_f16", _p(t), _p(out), rows, dim, out.stride(0), _stream())
    return out


def silu(x, out=None):
    _f16(x, "x")
    if out is None:
        out = torch.empty_like(x)
    call("katz_silu_f16", _p(x), _p(out), x.numel(), _stream())
    return out


def add(a, b, out=None):
    _f16(a, "a"), _f16(b, "b")
    if out is None:
        out = torch.empty_like(a)
    call("katz_add_f16", _p(a), _p(b), _p(out), a.numel(), _stream())
    return out


def concat_channels(a, b, out=None):
    """[..., C1] ++ [..., C2] -> [..., C1+C2] (skip-connection concat of the up blocks)."""
    _f16(a, "a"), _f16(b, "b")
    C1, C2 = a.shape[-1], b.shape[-1]
    rows = a.numel() // C1
    if out is None:
        out = torch.empty(tuple(a.shape[:-1]) + (C1 + C2,), dtype=torch.float16, device=a.device)
    call("katz_concat_channels_f16", _p(a), _p(b), _p(out), rows, C1, C2, _stream())
    return out


def halo_assemble(x, edges, rank, world, top=True, bottom=True, upsample=False, out=None):
    """x [B,h,W,C] + gathered edge rows [P,2,B,W,C] (None when world == 1) -> the padded (optionally 2x upsampled) input
    of a row shard's 3x3 convolution."""
    _f16(x, "x")
    if not x.is_contiguous() or (edges is not None and not edges.is_contiguous()):
        raise KatzError("halo_assemble: x and edges must be contiguous")
    B, h, W, C = x.shape
    shape = (B, 2 * h + 2, 2 * W, C) if upsample else (B, h + int(top) + int(bottom), W, C)
    if out is None:
        out = torch.empty(shape, dtype=torch.float16, device=x.device)
    call("katz_halo_assemble_f16", _p(x), _p(edges), _p(out), B, h, W, C, int(top), int(bottom), 1 if upsample else 0, rank,
         world, _stream())
    return out


def nchw_to_nhwc(x, cpad=None, out=None):
    _f16(x, "x")
    B, C, H, W = x.shape
    cpad = cpad or C
    if out is None:
        out = torch.empty((B, H, W, cpad), dtype=torch.float16, device=x.device)
    call("katz_nchw_to_nhwc_f16", _p(x.contiguous()), _p(out), B, C, H * W, cpad, _stream())
    return out


def nhwc_to_nchw(x, c=None, out=None):
    _f16(x, "x")
    B, H, W, cpad = x.shape
    c = c or cpad
    if out is None:
        out = torch.empty((B, c, H, W), dtype=torch.float16, device=x.device)
    call("katz_nhwc_to_nchw_f16", _p(x), _p(out), B, c, H * W, cpad, _stream())
    return out


def euler_scale_input(x, sigma, copies=1, out=None, cpu_torch_rounding=False):
    """half(x / sqrt(sigma^2 + 1)), written `copies` times. See euler_cfg_step for `cpu_torch_rounding`."""
    _f16(x, "x")
    if out is None:
        out = torch.empty((copies * x.shape[0],) + tuple(x.shape[1:]), dtype=torch.float16, device=x.device)
    call("katz_euler_scale_input", _p(x), _p(out), x.numel(), float(sigma), copies, 1 if cpu_torch_rounding else 0, _stream())
    return out


def euler_cfg_step(x, eps_uncond, eps_cond, guidance, sigma, sigma_next, cpu_torch_rounding=False):
    """In-place Euler step on the fp16 latent x with classifier-free guidance. The default reproduces torch's CUDA
    kernels (division by a host scalar = multiplication by its reciprocal; fp32 sigma); `cpu_torch_rounding`
    reproduces torch's CPU kernels (true division; sigma rounded to fp16 before `sigma * eps`)."""
    _f16(x, "x"), _f16(eps_uncond, "eps_uncond")
    call("katz_euler_cfg_step", _p(x), _p(eps_uncond), _p(eps_cond), x.numel(), float(guidance), float(sigma),
         float(sigma_next), 1 if cpu_torch_rounding else 0, _stream())
    return x
