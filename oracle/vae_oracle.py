"""TEST INFRASTRUCTURE — CPU oracle of the SDXL VAE decode that follows the denoising loop.

A functional restatement (plain torch ops over a state dict, fp32 by default) of `AutoencoderKL.decode`
(diffusers/models/autoencoders/autoencoder_kl.py: post_quant_conv, then the decoder) as the reference pipeline calls it
after the last step (pipelines/controlnet/pipeline_controlnet_sd_xl_katz.py:1690-1706: `latents / scaling_factor`, then
`vae.decode`): `Decoder.forward` (models/autoencoders/vae.py:285-347) = conv_in -> UNetMidBlock2D (resnet, one-head
attention over all pixels, resnet; models/unets/unet_2d_blocks.py:640-741) -> UpDecoderBlock2D x N (layers_per_block+1
resnets, nearest-2x upsample + 3x3 conv except in the last; :2680-2743) -> GroupNorm(eps 1e-6) -> SiLU -> conv_out.
The resnets are ResnetBlock2D without a time embedding (models/resnet.py:352-415); the attention is `Attention` built
with `_from_deprecated_attn_block`, GroupNorm inside, biases on every projection, a residual connection, through
AttnProcessor2_0 (models/attention_processor.py:1219-1296).

Only tests/, __graft_entry__.smoke() and bench.py's baseline legs may import this module. Parity pin:
tests/golden/tiny_vae_decode.npz holds the output of the reference's own AutoencoderKL on a tiny seeded configuration
(tests/golden/make_golden.py).
"""
import torch
import torch.nn.functional as F

from .unet_oracle import _conv, _gn

SDXL_VAE_CONFIG = dict(latent_channels=4, out_channels=3, block_out_channels=(128, 256, 512, 512), layers_per_block=2,
                       norm_num_groups=32, scaling_factor=0.13025)


def vae_resnet(sd, p, x, groups):
    """ResnetBlock2D.forward with temb=None, eps 1e-6 (vae.py:236-246 passes resnet_eps=1e-6)."""
    h = F.silu(_gn(sd, (p + ".norm1", p + ".norm_silu1.0"), x, groups, 1e-6))
    h = _conv(sd, p + ".conv1", h)
    h = F.silu(_gn(sd, (p + ".norm2", p + ".norm_silu2.0"), h, groups, 1e-6))
    h = _conv(sd, p + ".conv2", h)
    if p + ".conv_shortcut.weight" in sd:
        x = _conv(sd, p + ".conv_shortcut", x, padding=0)
    return (x + h) / 1.0


def vae_attention(sd, p, x, groups):
    """One head over all H*W positions, head dim = channels (unet_2d_blocks.py:681-694; AttnProcessor2_0)."""
    B, C, H, W = x.shape
    res = x
    h = x.view(B, C, H * W)
    h = F.group_norm(h, groups, sd[p + ".group_norm.weight"], sd[p + ".group_norm.bias"], 1e-6).transpose(1, 2)
    q = F.linear(h, sd[p + ".to_q.weight"], sd[p + ".to_q.bias"])
    k = F.linear(h, sd[p + ".to_k.weight"], sd[p + ".to_k.bias"])
    v = F.linear(h, sd[p + ".to_v.weight"], sd[p + ".to_v.bias"])
    o = F.scaled_dot_product_attention(q[:, None], k[:, None], v[:, None])[:, 0]
    o = F.linear(o, sd[p + ".to_out.0.weight"], sd[p + ".to_out.0.bias"])
    return o.transpose(1, 2).reshape(B, C, H, W) + res


def vae_decode(sd, cfg, z):
    """AutoencoderKL.decode(z).sample: z [B, latent_channels, h, w] -> image [B, out_channels, 8h, 8w] (for four levels)."""
    g = cfg["norm_num_groups"]
    x = _conv(sd, "post_quant_conv", z, padding=0)
    x = _conv(sd, "decoder.conv_in", x)
    x = vae_resnet(sd, "decoder.mid_block.resnets.0", x, g)
    x = vae_attention(sd, "decoder.mid_block.attentions.0", x, g)
    x = vae_resnet(sd, "decoder.mid_block.resnets.1", x, g)
    n = len(cfg["block_out_channels"])
    for i in range(n):
        for j in range(cfg["layers_per_block"] + 1):
            x = vae_resnet(sd, "decoder.up_blocks.%d.resnets.%d" % (i, j), x, g)
        if i != n - 1:
            x = F.interpolate(x, scale_factor=2.0, mode="nearest")
            x = _conv(sd, "decoder.up_blocks.%d.upsamplers.0.conv" % i, x)
    x = F.silu(_gn(sd, ("decoder.conv_norm_out",), x, g, 1e-6))
    return _conv(sd, "decoder.conv_out", x)


def decode_latents(sd, cfg, latents):
    """The pipeline's last step (…katz.py:1702-1706): latents / scaling_factor, then decode."""
    return vae_decode(sd, cfg, latents / cfg["scaling_factor"])
