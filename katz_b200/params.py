"""Parameter inventory of the SDXL UNet / ControlNet (names and shapes as in the reference's state dicts) and a
deterministic random initialiser for them.

Names follow `UNet2DConditionModel.state_dict()` / `ControlNetModel.state_dict()` of the reference fork
(diffusers/models/unets/unet_2d_condition.py:264-562, diffusers/models/controlnet.py:188-430): resnet norms are
`norm_silu1.0` / `norm_silu2.0`, the output norm is `conv_norm_silu.0`, GEGLU is the unsplit `proj`.
"""
from collections import OrderedDict

import numpy as np
import torch

SDXL_UNET_CONFIG = dict(
    in_channels=4, out_channels=4, block_out_channels=(320, 640, 1280),
    down_block_types=("DownBlock2D", "CrossAttnDownBlock2D", "CrossAttnDownBlock2D"),
    up_block_types=("CrossAttnUpBlock2D", "CrossAttnUpBlock2D", "UpBlock2D"),
    layers_per_block=2, transformer_layers_per_block=(1, 2, 10), attention_head_dim=(5, 10, 20),
    cross_attention_dim=2048, addition_time_embed_dim=256, projection_class_embeddings_input_dim=2816,
    norm_num_groups=32, norm_eps=1e-5, sample_size=128,
)

TINY_UNET_CONFIG = dict(
    in_channels=4, out_channels=4, block_out_channels=(64, 128, 256),
    down_block_types=("DownBlock2D", "CrossAttnDownBlock2D", "CrossAttnDownBlock2D"),
    up_block_types=("CrossAttnUpBlock2D", "CrossAttnUpBlock2D", "UpBlock2D"),
    layers_per_block=2, transformer_layers_per_block=(1, 1, 2), attention_head_dim=(1, 2, 4),
    cross_attention_dim=128, addition_time_embed_dim=32, projection_class_embeddings_input_dim=32 * 6 + 64,
    norm_num_groups=32, norm_eps=1e-5, sample_size=16,
)

CONTROLNET_COND_CHANNELS = (16, 32, 96, 256)


def _resnet(out, p, cin, cout, temb):
    out[p + ".norm_silu1.0.weight"] = (cin,)
    out[p + ".norm_silu1.0.bias"] = (cin,)
    out[p + ".conv1.weight"] = (cout, cin, 3, 3)
    out[p + ".conv1.bias"] = (cout,)
    out[p + ".time_emb_proj.weight"] = (cout, temb)
    out[p + ".time_emb_proj.bias"] = (cout,)
    out[p + ".norm_silu2.0.weight"] = (cout,)
    out[p + ".norm_silu2.0.bias"] = (cout,)
    out[p + ".conv2.weight"] = (cout, cout, 3, 3)
    out[p + ".conv2.bias"] = (cout,)
    if cin != cout:
        out[p + ".conv_shortcut.weight"] = (cout, cin, 1, 1)
        out[p + ".conv_shortcut.bias"] = (cout,)


def _transformer(out, p, c, layers, cross):
    out[p + ".norm.weight"] = (c,)
    out[p + ".norm.bias"] = (c,)
    out[p + ".proj_in.weight"] = (c, c)
    out[p + ".proj_in.bias"] = (c,)
    for i in range(layers):
        b = "%s.transformer_blocks.%d" % (p, i)
        out[b + ".norm1.weight"] = (c,)
        out[b + ".norm1.bias"] = (c,)
        for n in ("to_q", "to_k", "to_v"):
            out["%s.attn1.%s.weight" % (b, n)] = (c, c)
        out[b + ".attn1.to_out.0.weight"] = (c, c)
        out[b + ".attn1.to_out.0.bias"] = (c,)
        out[b + ".norm2.weight"] = (c,)
        out[b + ".norm2.bias"] = (c,)
        out[b + ".attn2.to_q.weight"] = (c, c)
        out[b + ".attn2.to_k.weight"] = (c, cross)
        out[b + ".attn2.to_v.weight"] = (c, cross)
        out[b + ".attn2.to_out.0.weight"] = (c, c)
        out[b + ".attn2.to_out.0.bias"] = (c,)
        out[b + ".norm3.weight"] = (c,)
        out[b + ".norm3.bias"] = (c,)
        out[b + ".ff.net.0.proj.weight"] = (8 * c, c)
        out[b + ".ff.net.0.proj.bias"] = (8 * c,)
        out[b + ".ff.net.2.weight"] = (c, 4 * c)
        out[b + ".ff.net.2.bias"] = (c,)
    out[p + ".proj_out.weight"] = (c, c)
    out[p + ".proj_out.bias"] = (c,)


def _encoder(out, cfg):
    """conv_in, embeddings, down blocks, mid block: shared by the UNet and the ControlNet."""
    boc = cfg["block_out_channels"]
    temb = boc[0] * 4
    out["conv_in.weight"] = (boc[0], cfg["in_channels"], 3, 3)
    out["conv_in.bias"] = (boc[0],)
    out["time_embedding.linear_1.weight"] = (temb, boc[0])
    out["time_embedding.linear_1.bias"] = (temb,)
    out["time_embedding.linear_2.weight"] = (temb, temb)
    out["time_embedding.linear_2.bias"] = (temb,)
    out["add_embedding.linear_1.weight"] = (temb, cfg["projection_class_embeddings_input_dim"])
    out["add_embedding.linear_1.bias"] = (temb,)
    out["add_embedding.linear_2.weight"] = (temb, temb)
    out["add_embedding.linear_2.bias"] = (temb,)
    cin = boc[0]
    for bi, btype in enumerate(cfg["down_block_types"]):
        cout = boc[bi]
        p = "down_blocks.%d" % bi
        if btype == "CrossAttnDownBlock2D":
            for li in range(cfg["layers_per_block"]):
                _transformer(out, "%s.attentions.%d" % (p, li), cout, cfg["transformer_layers_per_block"][bi],
                             cfg["cross_attention_dim"])
        for li in range(cfg["layers_per_block"]):
            _resnet(out, "%s.resnets.%d" % (p, li), cin if li == 0 else cout, cout, temb)
        if bi != len(boc) - 1:
            out[p + ".downsamplers.0.conv.weight"] = (cout, cout, 3, 3)
            out[p + ".downsamplers.0.conv.bias"] = (cout,)
        cin = cout
    c = boc[-1]
    _transformer(out, "mid_block.attentions.0", c, cfg["transformer_layers_per_block"][-1], cfg["cross_attention_dim"])
    _resnet(out, "mid_block.resnets.0", c, c, temb)
    _resnet(out, "mid_block.resnets.1", c, c, temb)


def unet_param_shapes(cfg):
    """OrderedDict name -> shape of UNet2DConditionModel for `cfg` (SDXL structure)."""
    out = OrderedDict()
    _encoder(out, cfg)
    boc = cfg["block_out_channels"]
    temb = boc[0] * 4
    # up blocks are appended to the module after the mid block but state_dict order follows registration order:
    # conv_in, embeddings, down_blocks, up_blocks, mid_block, conv_norm, conv_out. Order is irrelevant to users of this
    # dict; keys and shapes are what matters.
    rev = tuple(reversed(boc))
    rev_layers = tuple(reversed(cfg["transformer_layers_per_block"]))
    prev = rev[0]
    for bi, btype in enumerate(cfg["up_block_types"]):
        cout = rev[bi]
        cin_skip = rev[min(bi + 1, len(boc) - 1)]
        p = "up_blocks.%d" % bi
        n = cfg["layers_per_block"] + 1
        if btype == "CrossAttnUpBlock2D":
            for li in range(n):
                _transformer(out, "%s.attentions.%d" % (p, li), cout, rev_layers[bi], cfg["cross_attention_dim"])
        for li in range(n):
            skip = cin_skip if li == n - 1 else cout
            rin = prev if li == 0 else cout
            _resnet(out, "%s.resnets.%d" % (p, li), rin + skip, cout, temb)
        if bi != len(boc) - 1:
            out[p + ".upsamplers.0.conv.weight"] = (cout, cout, 3, 3)
            out[p + ".upsamplers.0.conv.bias"] = (cout,)
        prev = cout
    out["conv_norm_silu.0.weight"] = (boc[0],)
    out["conv_norm_silu.0.bias"] = (boc[0],)
    out["conv_out.weight"] = (cfg["out_channels"], boc[0], 3, 3)
    out["conv_out.bias"] = (cfg["out_channels"],)
    return out


def controlnet_param_shapes(cfg, cond_channels=3):
    """OrderedDict name -> shape of ControlNetModel.from_unet(unet) for `cfg`."""
    out = OrderedDict()
    _encoder(out, cfg)
    boc = cfg["block_out_channels"]
    ch = CONTROLNET_COND_CHANNELS
    p = "controlnet_cond_embedding"
    out[p + ".conv_in.weight"] = (ch[0], cond_channels, 3, 3)
    out[p + ".conv_in.bias"] = (ch[0],)
    for i in range(len(ch) - 1):
        out["%s.blocks.%d.weight" % (p, 2 * i)] = (ch[i], ch[i], 3, 3)
        out["%s.blocks.%d.bias" % (p, 2 * i)] = (ch[i],)
        out["%s.blocks.%d.weight" % (p, 2 * i + 1)] = (ch[i + 1], ch[i], 3, 3)
        out["%s.blocks.%d.bias" % (p, 2 * i + 1)] = (ch[i + 1],)
    out[p + ".conv_out.weight"] = (boc[0], ch[-1], 3, 3)
    out[p + ".conv_out.bias"] = (boc[0],)
    # zero-convs: one for conv_in's output, one per resnet output, one per downsampler output
    idx = 0
    chans = [boc[0]]
    for bi in range(len(boc)):
        chans += [boc[bi]] * cfg["layers_per_block"]
        if bi != len(boc) - 1:
            chans.append(boc[bi])
    for c in chans:
        out["controlnet_down_blocks.%d.weight" % idx] = (c, c, 1, 1)
        out["controlnet_down_blocks.%d.bias" % idx] = (c,)
        idx += 1
    out["controlnet_mid_block.weight"] = (boc[-1], boc[-1], 1, 1)
    out["controlnet_mid_block.bias"] = (boc[-1],)
    return out


def unet_step_flops(cfg, batch, height, width, text_len=77, controlnet=False):
    """Algorithmic FLOPs of one step: 2*M*N*K per linear / convolution-as-GEMM, 4*B*H*Sq*Sk*D per attention.
    Returns a dict by operator class plus 'total'. (height, width) is the latent size."""
    f = dict(linear=0.0, conv3x3=0.0, conv1x1=0.0, self_attn=0.0, cross_attn=0.0)
    boc = cfg["block_out_channels"]
    temb = boc[0] * 4
    cross = cfg["cross_attention_dim"]

    def resnet(cin, cout, h, w):
        m = batch * h * w
        f["conv3x3"] += 2.0 * m * cout * 9 * cin + 2.0 * m * cout * 9 * cout
        f["linear"] += 2.0 * batch * cout * temb
        if cin != cout:
            f["conv1x1"] += 2.0 * m * cout * cin

    def transformer(c, layers, h, w):
        m = batch * h * w
        s = h * w
        f["linear"] += 2 * (2.0 * m * c * c)                       # proj_in, proj_out
        for _ in range(layers):
            f["linear"] += 4 * (2.0 * m * c * c)                   # attn1 q,k,v,out
            f["linear"] += 2 * (2.0 * m * c * c)                   # attn2 q,out
            f["linear"] += 2 * (2.0 * batch * text_len * c * cross)  # attn2 k,v
            f["linear"] += 2.0 * m * 8 * c * c + 2.0 * m * c * 4 * c  # ff
            f["self_attn"] += 4.0 * batch * s * s * c
            f["cross_attn"] += 4.0 * batch * s * text_len * c

    h, w = height, width
    f["conv3x3"] += 2.0 * batch * h * w * boc[0] * 9 * cfg["in_channels"]
    f["linear"] += 2.0 * batch * (temb * boc[0] + temb * temb + temb * cfg["projection_class_embeddings_input_dim"] + temb * temb)
    cin = boc[0]
    skips = [(boc[0], h, w)]
    for bi, btype in enumerate(cfg["down_block_types"]):
        cout = boc[bi]
        for li in range(cfg["layers_per_block"]):
            resnet(cin if li == 0 else cout, cout, h, w)
            if btype == "CrossAttnDownBlock2D":
                transformer(cout, cfg["transformer_layers_per_block"][bi], h, w)
            skips.append((cout, h, w))
        if bi != len(boc) - 1:
            h, w = h // 2, w // 2
            f["conv3x3"] += 2.0 * batch * h * w * cout * 9 * cout
            skips.append((cout, h, w))
        cin = cout
    c = boc[-1]
    resnet(c, c, h, w)
    transformer(c, cfg["transformer_layers_per_block"][-1], h, w)
    resnet(c, c, h, w)
    if controlnet:
        for (sc, sh, sw) in skips:
            f["conv1x1"] += 2.0 * batch * sh * sw * sc * sc
        f["conv1x1"] += 2.0 * batch * h * w * c * c
        ch = CONTROLNET_COND_CHANNELS
        ih, iw = height * 8, width * 8
        f["conv3x3"] += 2.0 * batch * ih * iw * ch[0] * 9 * 3
        for i in range(len(ch) - 1):
            f["conv3x3"] += 2.0 * batch * ih * iw * ch[i] * 9 * ch[i]
            ih, iw = ih // 2, iw // 2
            f["conv3x3"] += 2.0 * batch * ih * iw * ch[i + 1] * 9 * ch[i]
        f["conv3x3"] += 2.0 * batch * ih * iw * boc[0] * 9 * ch[-1]
    else:
        rev = tuple(reversed(boc))
        rev_layers = tuple(reversed(cfg["transformer_layers_per_block"]))
        prev = rev[0]
        for bi, btype in enumerate(cfg["up_block_types"]):
            cout = rev[bi]
            n = cfg["layers_per_block"] + 1
            for li in range(n):
                sc, sh, sw = skips.pop()
                resnet((prev if li == 0 else cout) + sc, cout, h, w)
                if btype == "CrossAttnUpBlock2D":
                    transformer(cout, rev_layers[bi], h, w)
            if bi != len(boc) - 1:
                h, w = h * 2, w * 2
                f["conv3x3"] += 2.0 * batch * h * w * cout * 9 * cout
            prev = cout
        f["conv3x3"] += 2.0 * batch * h * w * cfg["out_channels"] * 9 * boc[0]
    f["total"] = sum(f.values())
    return f


def lora_target_keys(cfg, include_proj=False):
    """UNet linears a LoRA targets, in module order: per transformer block attn1 q/k/v/out, attn2 q/k/v/out, ff proj,
    ff out (700 layers for SDXL); with `include_proj` also each Transformer2DModel's proj_in/proj_out, which is the
    722-entry set of the reference's key-map fixtures (lora_info_shm/*_key_match_unet.json)."""
    keys = []
    for name in unet_param_shapes(cfg):
        if not name.endswith(".weight"):
            continue
        if ".transformer_blocks." in name and (".attn1.to_" in name or ".attn2.to_" in name or ".ff.net.0.proj." in name
                                               or ".ff.net.2." in name):
            keys.append(name)
        elif include_proj and (name.endswith(".proj_in.weight") or name.endswith(".proj_out.weight")):
            keys.append(name)
    return keys


def init_state_dict(shapes, seed=0, dtype=torch.float16, device="cpu", generator_device=None):
    """Deterministic random initialisation: weights and biases U(-1/sqrt(fan_in), 1/sqrt(fan_in)) (torch's default for
    Linear/Conv2d), norm scales 1 + 0.1*U(-1,1), norm shifts 0.1*U(-1,1). With device='cpu' numbers come from numpy's
    PCG64 stream (identical on every machine); with `generator_device='cuda'` they are drawn on the GPU (fast, used by
    the benchmark, not reproducible across devices)."""
    sd = OrderedDict()
    if generator_device is None:
        rng = np.random.default_rng(seed)
        for name, shape in shapes.items():
            n = int(np.prod(shape))
            u = rng.random(n, dtype=np.float32) * 2.0 - 1.0
            t = torch.from_numpy(u).reshape(shape)
            sd[name] = _scale_param(name, shape, t).to(dtype).to(device)
    else:
        g = torch.Generator(device=generator_device)
        g.manual_seed(seed)
        for name, shape in shapes.items():
            t = torch.rand(shape, generator=g, device=generator_device, dtype=torch.float32) * 2.0 - 1.0
            sd[name] = _scale_param(name, shape, t).to(dtype).to(device)
    return sd


def _scale_param(name, shape, t):
    is_norm = (".norm" in name or "_norm" in name or name.startswith("conv_norm")) and len(shape) == 1
    if is_norm:
        return 1.0 + 0.1 * t if name.endswith(".weight") else 0.1 * t
    if name.endswith(".weight"):
        fan_in = int(np.prod(shape[1:]))
    else:
        fan_in = _bias_fan_in.get(name, None) or shape[0]
    return t * (1.0 / float(np.sqrt(fan_in)))


_bias_fan_in = {}


# The two SDXL text encoders as far as a LoRA sees them: (layers, width, mlp width)
TEXT_ENCODER_DIMS = {"text_encoder": (12, 768, 3072), "text_encoder_2": (32, 1280, 5120)}


def text_encoder_lora_key_map(which, layers=None):
    """The reference's key map for a text encoder's LoRA layers (lora_info_shm/*_key_match_text_encoder[_2].json):
    {state-dict key: {"lora_down_key", "lora_up_key"}} over q/k/v/out projections and the two MLP linears of every
    layer, in the reference's order, and {state-dict key: (out, in)}."""
    from collections import OrderedDict
    n, d, f = TEXT_ENCODER_DIMS[which]
    km, shapes = OrderedDict(), OrderedDict()
    for i in range(n if layers is None else layers):
        base = "text_model.encoder.layers.%d." % i
        for proj in ("k", "v", "q", "out"):
            key = base + "self_attn.%s_proj.weight" % proj
            stem = "%s.%sself_attn.to_%s_lora." % (which, base, proj)
            km[key] = {"lora_down_key": stem + "down.weight", "lora_up_key": stem + "up.weight"}
            shapes[key] = (d, d)
        for fc, shp in (("fc1", (f, d)), ("fc2", (d, f))):
            key = base + "mlp.%s.weight" % fc
            stem = "%s.%smlp.%s.lora_linear_layer." % (which, base, fc)
            km[key] = {"lora_down_key": stem + "down.weight", "lora_up_key": stem + "up.weight"}
            shapes[key] = shp
    return km, shapes


def key_map_digest(key_map, shapes, rank):
    """sha256 over the sorted lines `key down_key up_key down_shape up_shape` (what tests/golden pins)."""
    import hashlib
    lines = sorted("%s %s %s %s %s" % (k, m["lora_down_key"], m["lora_up_key"], (rank, shapes[k][1]), (shapes[k][0], rank))
                   for k, m in key_map.items())
    return hashlib.sha256("\n".join(lines).encode()).hexdigest()


# ---- the VAE decoder that follows the denoising loop (AutoencoderKL.decode; models/autoencoders/vae.py:185-347)
SDXL_VAE_CONFIG = dict(latent_channels=4, out_channels=3, block_out_channels=(128, 256, 512, 512), layers_per_block=2,
                       norm_num_groups=32, scaling_factor=0.13025)
TINY_VAE_CONFIG = dict(latent_channels=4, out_channels=3, block_out_channels=(64, 128, 128), layers_per_block=2,
                       norm_num_groups=32, scaling_factor=0.13025)


def vae_decoder_param_shapes(cfg):
    """Decoder-side parameter inventory of AutoencoderKL in the reference fork's state-dict naming, module order."""
    from collections import OrderedDict
    out = OrderedDict()
    boc = cfg["block_out_channels"]
    lc = cfg["latent_channels"]

    def conv(p, cout, cin, k):
        out[p + ".weight"] = (cout, cin, k, k)
        out[p + ".bias"] = (cout,)

    def norm(p, c):
        out[p + ".weight"] = (c,)
        out[p + ".bias"] = (c,)

    def resnet(p, cin, cout):
        norm(p + ".norm_silu1.0", cin)
        conv(p + ".conv1", cout, cin, 3)
        norm(p + ".norm_silu2.0", cout)
        conv(p + ".conv2", cout, cout, 3)
        if cin != cout:
            conv(p + ".conv_shortcut", cout, cin, 1)

    top = boc[-1]
    conv("decoder.conv_in", top, lc, 3)
    rev = list(reversed(boc))
    prev = rev[0]
    for i, c in enumerate(rev):
        for j in range(cfg["layers_per_block"] + 1):
            resnet("decoder.up_blocks.%d.resnets.%d" % (i, j), prev if j == 0 else c, c)
        if i != len(rev) - 1:
            conv("decoder.up_blocks.%d.upsamplers.0.conv" % i, c, c, 3)
        prev = c
    a = "decoder.mid_block.attentions.0"
    norm(a + ".group_norm", top)
    for n in ("to_q", "to_k", "to_v", "to_out.0"):
        out[a + ".%s.weight" % n] = (top, top)
        out[a + ".%s.bias" % n] = (top,)
    resnet("decoder.mid_block.resnets.0", top, top)
    resnet("decoder.mid_block.resnets.1", top, top)
    norm("decoder.conv_norm_out", boc[0])
    conv("decoder.conv_out", cfg["out_channels"], boc[0], 3)
    conv("post_quant_conv", lc, lc, 1)
    return out


def vae_decode_flops(cfg, batch, h, w):
    """Algorithmic FLOPs of one decode of a [batch, latent_channels, h, w] latent: 2*M*N*K per convolution / linear,
    4*S*S*C for the one-head attention."""
    shapes = vae_decoder_param_shapes(cfg)
    boc = cfg["block_out_channels"]
    n = len(boc)
    total = 0.0

    def res_of(key):
        if key.startswith("decoder.up_blocks."):
            i = int(key.split(".")[2])
            lvl = i + 1 if ".upsamplers." in key else i
            return h << lvl, w << lvl
        if key.startswith("decoder.conv_out"):
            return h << (n - 1), w << (n - 1)
        return h, w
    for k, shp in shapes.items():
        if k.endswith(".weight") and len(shp) == 4:
            hh, ww = res_of(k)
            total += 2.0 * batch * hh * ww * shp[0] * shp[1] * shp[2] * shp[3]
        elif k.endswith(".weight") and len(shp) == 2:
            total += 2.0 * batch * h * w * shp[0] * shp[1]
    total += 4.0 * batch * float(h * w) ** 2 * boc[-1]
    return total
