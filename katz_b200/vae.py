"""The VAE decode that follows the denoising loop, on the library's kernels.

`KatzVaeDecoder` computes what `AutoencoderKL.decode(z).sample` computes (diffusers/models/autoencoders/autoencoder_kl.py;
`Decoder.forward`, models/autoencoders/vae.py:285-347) for the reference pipeline's last step
(pipelines/controlnet/pipeline_controlnet_sd_xl_katz.py:1690-1706: `latents / scaling_factor`, then `vae.decode`), with
the reference's state-dict keys (the fork's `norm_silu1.0` spelling or upstream's `norm1`), in fp16 as the reference
runs its fp16-safe VAE (sdxl_pipeline.py:85).

Layout is NHWC throughout; NCHW exists at the two ends only. Every 3x3 convolution with 64-aligned input channels
runs on the tcgen05 implicit-GEMM kernel (M = pixels: up to a million rows per image), the 4-channel ends on the
mma.sync kernel. The mid-block attention has ONE head of `C` channels (512 for SDXL), which the 64-channel flash
kernels do not cover; it is three GEMMs and a row softmax: scores = (q k^T) / sqrt(C) from `katz_linear_f16` (scale in
the epilogue), `katz_softmax_rows_f16`, then probabilities x V^T. At 1024x1024 pixels that is a 16384 x 16384 score
matrix per image (512 MB in fp16), 5 % of the decode's FLOPs.
"""
from collections import OrderedDict

import torch

from . import ops
from ._lib import KatzError
from .ops import ACT_NONE, ACT_SILU
from .params import vae_decoder_param_shapes

_ALT = ((".norm1.", ".norm_silu1.0."), (".norm2.", ".norm_silu2.0."))


def _canonical(k):
    if ".resnets." in k:
        for a, b in _ALT:
            k = k.replace(a, b)
    return k


class KatzVaeDecoder:
    """decode(z): [B, latent_channels, h, w] fp16 CUDA -> [B, out_channels, h * 2^(levels-1), w * 2^(levels-1)] fp16."""

    def __init__(self, cfg, device="cuda", state_dict=None):
        self.cfg = dict(cfg)
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KatzError("KatzVaeDecoder needs a CUDA device (there is no CPU path)")
        self.shapes = vae_decoder_param_shapes(cfg)
        self.w = {}
        self.use_cuda_graph = False
        self._graphs = {}
        if state_dict is not None:
            self.load_state_dict(state_dict)

    # ---- weights: convolutions [Cout, ky, kx, Cin padded to 8], linears [N, K]. post_quant_conv gets 8 output rows (the
    # next convolution reads 8-channel pixels; rows 4..7 are zero), conv_out 4 (which keeps it on the narrow-N kernel).
    @staticmethod
    def _cout_pad(key, cout):
        return 8 if key.startswith("post_quant_conv.") else (cout + 3) // 4 * 4

    def load_state_dict(self, sd, strict=True):
        dev = self.device
        seen = set()
        for k, v in sd.items():
            ck = _canonical(k)
            if ck not in self.shapes:
                if strict and (k.startswith("decoder.") or k.startswith("post_quant_conv.")):
                    raise KatzError("unexpected key in state dict: %s" % k)
                continue                      # encoder-side keys of a whole AutoencoderKL state dict
            shp = self.shapes[ck]
            if tuple(v.shape) != tuple(shp):
                raise KatzError("shape mismatch for %s: %s vs %s" % (k, tuple(v.shape), tuple(shp)))
            src = v.to(device=dev, dtype=torch.float16)
            if len(shp) == 4:
                cout, cin = shp[0], shp[1]
                t = torch.zeros((self._cout_pad(ck, cout), shp[2], shp[3], (cin + 7) // 8 * 8), dtype=torch.float16, device=dev)
                t[:cout, :, :, :cin].copy_(src.permute(0, 2, 3, 1))
            elif ck.endswith(".bias") and (ck[:-5] + ".weight") in self.shapes and len(self.shapes[ck[:-5] + ".weight"]) == 4:
                t = torch.zeros((self._cout_pad(ck, shp[0]),), dtype=torch.float16, device=dev)
                t[:shp[0]].copy_(src)
            else:
                t = src.contiguous().clone()
            self.w[ck] = t
            seen.add(ck)
        missing = [k for k in self.shapes if k not in seen]
        if strict and missing:
            raise KatzError("missing keys in state dict: %s ..." % missing[:5])
        self._graphs.clear()
        return missing

    def state_dict(self):
        out = OrderedDict()
        for k, shp in self.shapes.items():
            t = self.w[k]
            if len(shp) == 4:
                out[k] = t[:shp[0], :, :, :shp[1]].permute(0, 3, 1, 2).contiguous()
            else:
                out[k] = t[:shp[0]].clone()
        return out

    # ---- blocks
    def _gn(self, x, p, act):
        return ops.group_norm_nhwc(x, self.w[p + ".weight"], self.w[p + ".bias"], self.cfg["norm_num_groups"], 1e-6, act)

    def _conv(self, x, p, **kw):
        return ops.conv2d(x, self.w[p + ".weight"], self.w[p + ".bias"], **kw)

    def _resnet(self, p, x):
        """ResnetBlock2D without a time embedding (models/resnet.py:352-415, eps 1e-6)."""
        B, H, W, cin = x.shape
        h = self._gn(x, p + ".norm_silu1.0", ACT_SILU)
        h = self._conv(h, p + ".conv1")
        h = self._gn(h, p + ".norm_silu2.0", ACT_SILU)
        sc = x
        if (p + ".conv_shortcut.weight") in self.w:
            wsc = self.w[p + ".conv_shortcut.weight"]
            cout = wsc.shape[0]
            sc = ops.linear(x.view(B * H * W, cin), wsc.view(cout, cin), self.w[p + ".conv_shortcut.bias"]).view(B, H, W, cout)
        return self._conv(h, p + ".conv2", residual=sc)

    def _attention(self, p, x):
        """One head over all pixels (unet_2d_blocks.py:681-694, AttnProcessor2_0): GroupNorm, q/k/v with bias,
        softmax(q k^T / sqrt(C)) v, output projection with bias, residual."""
        B, H, W, C = x.shape
        S = H * W
        h = self._gn(x, p + ".group_norm", ACT_NONE).view(B * S, C)
        q = ops.linear(h, self.w[p + ".to_q.weight"], self.w[p + ".to_q.bias"])
        k = ops.linear(h, self.w[p + ".to_k.weight"], self.w[p + ".to_k.bias"])
        v = ops.linear(h, self.w[p + ".to_v.weight"], self.w[p + ".to_v.bias"])
        o = torch.empty((B * S, C), dtype=torch.float16, device=x.device)
        scores = torch.empty((S, S), dtype=torch.float16, device=x.device)
        vt = torch.empty((1, C, S, 1), dtype=torch.float16, device=x.device)
        for b in range(B):
            rows = slice(b * S, (b + 1) * S)
            ops.linear(q[rows], k[rows], out=scores, out_scale=float(C) ** -0.5)
            ops.softmax_rows(scores, out=scores)
            ops.nhwc_to_nchw(v[rows].view(1, S, 1, C), out=vt)             # V^T: the second GEMM's [N, K] operand
            ops.linear(scores, vt.view(C, S), out=o[rows])
        out = ops.linear(o, self.w[p + ".to_out.0.weight"], self.w[p + ".to_out.0.bias"], residual=x.view(B * S, C))
        return out.view(B, H, W, C)

    def _decode(self, z):
        cfg = self.cfg
        x = ops.nchw_to_nhwc(z, cpad=8)
        x = self._conv(x, "post_quant_conv", ksize=1, pad=0)               # rows 4..7 of the padded weight are zero
        x = self._conv(x, "decoder.conv_in")
        x = self._resnet("decoder.mid_block.resnets.0", x)
        x = self._attention("decoder.mid_block.attentions.0", x)
        x = self._resnet("decoder.mid_block.resnets.1", x)
        n = len(cfg["block_out_channels"])
        for i in range(n):
            for j in range(cfg["layers_per_block"] + 1):
                x = self._resnet("decoder.up_blocks.%d.resnets.%d" % (i, j), x)
            if i != n - 1:
                x = self._conv(x, "decoder.up_blocks.%d.upsamplers.0.conv" % i, upsample=True)
        x = self._gn(x, "decoder.conv_norm_out", ACT_SILU)
        x = self._conv(x, "decoder.conv_out")
        return ops.nhwc_to_nchw(x, c=cfg["out_channels"])

    def decode(self, z):
        """AutoencoderKL.decode(z).sample."""
        if z.device != self.device or z.dtype != torch.float16 or z.dim() != 4 or z.shape[1] != self.cfg["latent_channels"]:
            raise KatzError("decode: z must be a [B, %d, h, w] fp16 tensor on %s" % (self.cfg["latent_channels"], self.device))
        if not self.use_cuda_graph:
            return self._decode(z.contiguous())
        key = tuple(z.shape)
        g = self._graphs.get(key)
        if g is None:
            static = z.contiguous().clone()
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._decode(static)
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self._decode(static)
            g = self._graphs[key] = (graph, static, out)
        else:
            g[1].copy_(z)
        g[0].replay()
        return g[2]

    def decode_latents(self, latents):
        """The pipeline's last step (…katz.py:1702-1706): `latents / scaling_factor`, then decode."""
        return self.decode(latents / self.cfg["scaling_factor"])

    __call__ = decode
