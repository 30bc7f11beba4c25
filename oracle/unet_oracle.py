"""TEST INFRASTRUCTURE — CPU oracle of the SDXL UNet / ControlNet denoising step.

A functional restatement (plain torch ops over a state dict, fp32 on CPU by default) of the reference's torch path
for one UNet step with adapters: `_down_forward` -> ControlNet residual add -> `_up_forward`
(diffusers/models/unets/unet_2d_condition.py:1127-1341), the five SDXL block classes
(diffusers/models/unets/unet_2d_blocks.py:744,1140,1303,2382,2558), ResnetBlock2D (models/resnet.py:352-415),
Transformer2DModel (models/transformers/transformer_2d.py:327-527), BasicTransformerBlock / FeedForward
(models/attention.py:283-404,608-664), AttnProcessor2_0 (models/attention_processor.py:1219-1296), GEGLU with erf
GELU (models/activations.py:146-149), the embeddings (models/embeddings.py:26-66,190-252) and ControlNetModel
(models/controlnet.py:84-127,687-847).

Only tests/, __graft_entry__.smoke() and bench.py's CPU baseline may import this module; it is the checker, never
the product path. Parity pin: tests/golden/*.npz hold outputs of the reference's own classes (imported from the
reference tree, tiny seeded configs) that this file reproduces; tests/golden/make_golden.py regenerates them.

State-dict keys are the reference's (either `norm1`/`norm2`/`conv_norm_out` or the fork's renamed
`norm_silu1.0`/`norm_silu2.0`/`conv_norm_silu.0`; GEGLU as `proj` or as the fork's split `proj_1`/`proj_2`).
"""
import math

import torch
import torch.nn.functional as F

SDXL_UNET_CONFIG = dict(
    in_channels=4, out_channels=4, block_out_channels=(320, 640, 1280),
    down_block_types=("DownBlock2D", "CrossAttnDownBlock2D", "CrossAttnDownBlock2D"),
    up_block_types=("CrossAttnUpBlock2D", "CrossAttnUpBlock2D", "UpBlock2D"),
    layers_per_block=2, transformer_layers_per_block=(1, 2, 10), attention_head_dim=(5, 10, 20),
    cross_attention_dim=2048, addition_time_embed_dim=256, projection_class_embeddings_input_dim=2816,
    norm_num_groups=32, norm_eps=1e-5, sample_size=128,
)

# Small config with the same block structure (used by the golden fixtures and the fast tests).
TINY_UNET_CONFIG = dict(
    in_channels=4, out_channels=4, block_out_channels=(64, 128, 256),
    down_block_types=("DownBlock2D", "CrossAttnDownBlock2D", "CrossAttnDownBlock2D"),
    up_block_types=("CrossAttnUpBlock2D", "CrossAttnUpBlock2D", "UpBlock2D"),
    layers_per_block=2, transformer_layers_per_block=(1, 1, 2), attention_head_dim=(1, 2, 4),
    cross_attention_dim=128, addition_time_embed_dim=32, projection_class_embeddings_input_dim=32 * 6 + 64,
    norm_num_groups=32, norm_eps=1e-5, sample_size=16,
)

CONTROLNET_COND_CHANNELS = (16, 32, 96, 256)


def _get(sd, *names):
    for n in names:
        if n in sd:
            return sd[n]
    raise KeyError(names[0])


def timestep_embedding(t, dim):
    """get_timestep_embedding (embeddings.py:26-66) with flip_sin_to_cos=True, downscale_freq_shift=0."""
    half = dim // 2
    exponent = -math.log(10000) * torch.arange(0, half, dtype=torch.float32, device=t.device) / half
    emb = t[:, None].float() * torch.exp(exponent)[None, :]
    emb = torch.cat([torch.sin(emb), torch.cos(emb)], dim=-1)
    return torch.cat([emb[:, half:], emb[:, :half]], dim=-1)


def _linear(sd, p, x):
    return F.linear(x, sd[p + ".weight"], sd.get(p + ".bias"))


def _conv(sd, p, x, stride=1, padding=1):
    return F.conv2d(x, sd[p + ".weight"], sd.get(p + ".bias"), stride=stride, padding=padding)


def _gn(sd, names, x, groups, eps):
    w = _get(sd, *[n + ".weight" for n in names])
    b = _get(sd, *[n + ".bias" for n in names])
    return F.group_norm(x, groups, w, b, eps)


def resnet(sd, p, x, temb, groups, eps):
    """ResnetBlock2D.forward (resnet.py:352-415), time_embedding_norm='default', output_scale_factor=1."""
    h = F.silu(_gn(sd, (p + ".norm1", p + ".norm_silu1.0"), x, groups, eps))
    h = _conv(sd, p + ".conv1", h)
    h = h + _linear(sd, p + ".time_emb_proj", F.silu(temb))[:, :, None, None]
    h = F.silu(_gn(sd, (p + ".norm2", p + ".norm_silu2.0"), h, groups, eps))
    h = _conv(sd, p + ".conv2", h)
    if p + ".conv_shortcut.weight" in sd:
        x = _conv(sd, p + ".conv_shortcut", x, padding=0)
    return (x + h) / 1.0


def attention(sd, p, x, ctx, heads):
    """Attention + AttnProcessor2_0 (attention_processor.py:1256-1296): no mask, scale 1/sqrt(head_dim)."""
    ctx = x if ctx is None else ctx
    q = F.linear(x, sd[p + ".to_q.weight"])
    k = F.linear(ctx, sd[p + ".to_k.weight"])
    v = F.linear(ctx, sd[p + ".to_v.weight"])
    B, S, C = q.shape
    d = C // heads
    q = q.view(B, -1, heads, d).transpose(1, 2)
    k = k.view(B, -1, heads, d).transpose(1, 2)
    v = v.view(B, -1, heads, d).transpose(1, 2)
    o = F.scaled_dot_product_attention(q, k, v)
    o = o.transpose(1, 2).reshape(B, -1, C)
    return _linear(sd, p + ".to_out.0", o)


def geglu(sd, p, x):
    """GEGLU.forward, unfused branch (activations.py:146-149)."""
    if p + ".proj.weight" in sd:
        h, g = _linear(sd, p + ".proj", x).chunk(2, dim=-1)
    else:
        h, g = _linear(sd, p + ".proj_1", x), _linear(sd, p + ".proj_2", x)
    return h * F.gelu(g)


def transformer_block(sd, p, x, ctx, heads):
    """BasicTransformerBlock.forward (attention.py:283-404), norm_type='layer_norm', eps 1e-5."""
    C = x.shape[-1]
    n = F.layer_norm(x, (C,), sd[p + ".norm1.weight"], sd[p + ".norm1.bias"], 1e-5)
    x = attention(sd, p + ".attn1", n, None, heads) + x
    n = F.layer_norm(x, (C,), sd[p + ".norm2.weight"], sd[p + ".norm2.bias"], 1e-5)
    x = attention(sd, p + ".attn2", n, ctx, heads) + x
    n = F.layer_norm(x, (C,), sd[p + ".norm3.weight"], sd[p + ".norm3.bias"], 1e-5)
    x = _linear(sd, p + ".ff.net.2", geglu(sd, p + ".ff.net.0", n)) + x
    return x


def transformer_2d(sd, p, x, ctx, heads, n_layers, groups):
    """Transformer2DModel.forward, continuous input + use_linear_projection (transformer_2d.py:404-409,479-527)."""
    B, C, H, W = x.shape
    res = x
    h = _gn(sd, (p + ".norm",), x, groups, 1e-6)
    h = h.permute(0, 2, 3, 1).reshape(B, H * W, C)
    h = _linear(sd, p + ".proj_in", h)
    for i in range(n_layers):
        h = transformer_block(sd, "%s.transformer_blocks.%d" % (p, i), h, ctx, heads)
    h = _linear(sd, p + ".proj_out", h)
    h = h.reshape(B, H, W, C).permute(0, 3, 1, 2).contiguous()
    return h + res


def time_and_aug_embedding(sd, cfg, timestep, text_embeds, time_ids, batch, dtype):
    """get_time_embed + TimestepEmbedding + text_time get_aug_embed (unet_2d_condition.py:997-1075,1147-1165)."""
    t = torch.as_tensor(timestep, dtype=torch.float32, device=text_embeds.device).reshape(-1).expand(batch)
    t_emb = timestep_embedding(t, cfg["block_out_channels"][0]).to(dtype)
    emb = _linear(sd, "time_embedding.linear_2", F.silu(_linear(sd, "time_embedding.linear_1", t_emb)))
    tid = timestep_embedding(time_ids.flatten().float(), cfg["addition_time_embed_dim"])
    tid = tid.reshape(text_embeds.shape[0], -1)
    add = torch.cat([text_embeds.float(), tid], dim=-1).to(dtype)
    aug = _linear(sd, "add_embedding.linear_2", F.silu(_linear(sd, "add_embedding.linear_1", add)))
    return emb + aug


def _down_blocks(sd, cfg, sample, emb, ctx):
    groups, eps = cfg["norm_num_groups"], cfg["norm_eps"]
    res = (sample,)
    nb = len(cfg["block_out_channels"])
    for bi, btype in enumerate(cfg["down_block_types"]):
        heads = cfg["attention_head_dim"][bi]
        for li in range(cfg["layers_per_block"]):
            sample = resnet(sd, "down_blocks.%d.resnets.%d" % (bi, li), sample, emb, groups, eps)
            if btype == "CrossAttnDownBlock2D":
                sample = transformer_2d(sd, "down_blocks.%d.attentions.%d" % (bi, li), sample, ctx, heads,
                                        cfg["transformer_layers_per_block"][bi], groups)
            res += (sample,)
        if bi != nb - 1:
            sample = _conv(sd, "down_blocks.%d.downsamplers.0.conv" % bi, sample, stride=2, padding=1)
            res += (sample,)
    return sample, res


def _mid_block(sd, cfg, sample, emb, ctx):
    groups, eps = cfg["norm_num_groups"], cfg["norm_eps"]
    heads = cfg["attention_head_dim"][-1]
    sample = resnet(sd, "mid_block.resnets.0", sample, emb, groups, eps)
    sample = transformer_2d(sd, "mid_block.attentions.0", sample, ctx, heads, cfg["transformer_layers_per_block"][-1], groups)
    sample = resnet(sd, "mid_block.resnets.1", sample, emb, groups, eps)
    return sample


def unet_down_forward(sd, cfg, sample, timestep, ctx, text_embeds, time_ids):
    """UNet2DConditionModel._down_forward (unet_2d_condition.py:1127-1252)."""
    emb = time_and_aug_embedding(sd, cfg, timestep, text_embeds, time_ids, sample.shape[0], sample.dtype)
    sample = _conv(sd, "conv_in", sample)
    sample, res = _down_blocks(sd, cfg, sample, emb, ctx)
    sample = _mid_block(sd, cfg, sample, emb, ctx)
    return sample, emb, res


def unet_up_forward(sd, cfg, sample, emb, res, ctx, down_residuals=None, mid_residual=None):
    """UNet2DConditionModel._up_forward (unet_2d_condition.py:1254-1341)."""
    groups, eps = cfg["norm_num_groups"], cfg["norm_eps"]
    if down_residuals is not None:
        res = tuple(r + a for r, a in zip(res, down_residuals))
    if mid_residual is not None:
        sample = sample + mid_residual
    nb = len(cfg["block_out_channels"])
    rev_heads = tuple(reversed(cfg["attention_head_dim"]))
    rev_layers = tuple(reversed(cfg["transformer_layers_per_block"]))
    for bi, btype in enumerate(cfg["up_block_types"]):
        n_res = cfg["layers_per_block"] + 1
        skips, res = res[-n_res:], res[:-n_res]
        for li in range(n_res):
            sample = torch.cat([sample, skips[-1 - li]], dim=1)
            sample = resnet(sd, "up_blocks.%d.resnets.%d" % (bi, li), sample, emb, groups, eps)
            if btype == "CrossAttnUpBlock2D":
                sample = transformer_2d(sd, "up_blocks.%d.attentions.%d" % (bi, li), sample, ctx, rev_heads[bi],
                                        rev_layers[bi], groups)
        if bi != nb - 1:
            sample = F.interpolate(sample, scale_factor=2.0, mode="nearest")
            sample = _conv(sd, "up_blocks.%d.upsamplers.0.conv" % bi, sample)
    sample = F.silu(_gn(sd, ("conv_norm_out", "conv_norm_silu.0"), sample, groups, eps))
    return _conv(sd, "conv_out", sample)


def unet_step(sd, cfg, sample, timestep, ctx, text_embeds, time_ids, down_residuals=None, mid_residual=None):
    """One UNet denoising step: `_down_forward` -> residual add -> `_up_forward` (the CUDA-graph path of the
    reference, unet_2d_condition.py:1344-1526, which adds all 9 down residuals and the mid residual)."""
    mid, emb, res = unet_down_forward(sd, cfg, sample, timestep, ctx, text_embeds, time_ids)
    return unet_up_forward(sd, cfg, mid, emb, res, ctx, down_residuals, mid_residual)


def controlnet_cond_embedding(sd, cond, p="controlnet_cond_embedding"):
    """ControlNetConditioningEmbedding.forward (controlnet.py:113-127): conv_in, 3 x (conv, conv stride 2), conv_out."""
    h = F.silu(_conv(sd, p + ".conv_in", cond))
    n_blocks = 2 * (len(CONTROLNET_COND_CHANNELS) - 1)
    for i in range(n_blocks):
        h = F.silu(_conv(sd, "%s.blocks.%d" % (p, i), h, stride=2 if i % 2 == 1 else 1))
    return _conv(sd, p + ".conv_out", h)


def controlnet_step(sd, cfg, sample, timestep, ctx, cond, text_embeds, time_ids, conditioning_scale=0.5):
    """ControlNetModel._controlnet_forward (controlnet.py:687-847): returns (9 down residuals, mid residual), each
    already multiplied by conditioning_scale (default 0.5 in the reference fork, controlnet.py:693)."""
    emb = time_and_aug_embedding(sd, cfg, timestep, text_embeds, time_ids, sample.shape[0], sample.dtype)
    sample = _conv(sd, "conv_in", sample) + controlnet_cond_embedding(sd, cond)
    sample, res = _down_blocks(sd, cfg, sample, emb, ctx)
    sample = _mid_block(sd, cfg, sample, emb, ctx)
    outs = [_conv(sd, "controlnet_down_blocks.%d" % i, r, padding=0) * conditioning_scale for i, r in enumerate(res)]
    mid = _conv(sd, "controlnet_mid_block", sample, padding=0) * conditioning_scale
    return outs, mid


# ------------------------------------------------------------------------------------------------ Euler / CFG ----
def euler_sigmas(num_inference_steps, num_train_timesteps=1000, beta_start=0.00085, beta_end=0.012, steps_offset=1,
                 beta_schedule="scaled_linear", timestep_spacing="leading"):
    """EulerDiscreteScheduler.__init__ + set_timesteps, interpolation 'linear'
    (scheduling_euler_discrete.py:195-211,300-362). Defaults are the SDXL scheduler config
    (tests/pipelines/controlnet/test_controlnet_sdxl.py:116-122). Returns (timesteps fp32, sigmas fp32 with a trailing 0,
    init_noise_sigma)."""
    import numpy as np
    if beta_schedule == "linear":
        betas = torch.linspace(beta_start, beta_end, num_train_timesteps, dtype=torch.float32)
    elif beta_schedule == "scaled_linear":
        betas = torch.linspace(beta_start ** 0.5, beta_end ** 0.5, num_train_timesteps, dtype=torch.float32) ** 2
    else:
        raise NotImplementedError(beta_schedule)
    alphas_cumprod = torch.cumprod(1.0 - betas, dim=0)
    if timestep_spacing == "linspace":
        timesteps = np.linspace(0, num_train_timesteps - 1, num_inference_steps, dtype=np.float32)[::-1].copy()
    elif timestep_spacing == "leading":
        step_ratio = num_train_timesteps // num_inference_steps
        timesteps = (np.arange(0, num_inference_steps) * step_ratio).round()[::-1].copy().astype(np.float32)
        timesteps += steps_offset
    else:
        raise NotImplementedError(timestep_spacing)
    sigmas = (((1 - alphas_cumprod) / alphas_cumprod) ** 0.5).numpy()
    sigmas = np.interp(timesteps, np.arange(0, len(sigmas)), sigmas)
    sigmas = torch.cat([torch.from_numpy(sigmas).to(torch.float32), torch.zeros(1)])
    max_sigma = sigmas.max()
    init_sigma = max_sigma if timestep_spacing == "linspace" else (max_sigma ** 2 + 1) ** 0.5
    return torch.from_numpy(timesteps.astype(np.float32)), sigmas, float(init_sigma)


def euler_scale_model_input(x, sigma):
    """scale_model_input (scheduling_euler_discrete.py:294-295); x keeps its dtype (sigma is a 0-dim fp32 tensor)."""
    sigma = torch.as_tensor(sigma, dtype=torch.float32)
    return x / ((sigma ** 2 + 1) ** 0.5)


def cfg_combine(uncond, cond, guidance):
    """pipeline_controlnet_sd_xl_katz.py:1649-1655."""
    return uncond + guidance * (cond - uncond)


def euler_step(x, eps, sigma, sigma_next):
    """EulerDiscreteScheduler.step, epsilon prediction, s_churn=0 (scheduling_euler_discrete.py:498-537)."""
    sigma = torch.as_tensor(sigma, dtype=torch.float32)
    sigma_next = torch.as_tensor(sigma_next, dtype=torch.float32)
    sample = x.to(torch.float32)
    pred = sample - sigma * eps
    derivative = (sample - pred) / sigma
    prev = sample + derivative * (sigma_next - sigma)
    return prev.to(eps.dtype)


def denoise_loop(sd, cfg, latents, prompt_embeds, text_embeds, time_ids, num_inference_steps, guidance_scale=5.0,
                 controlnets=(), controlnet_cond=None, conditioning_scales=None, combine="sum", half_latents=True):
    """The denoise loop of pipeline_controlnet_sd_xl_katz.py:1508-1675 for this path: per step scale_model_input on the
    CFG batch, ControlNets (residuals summed as multicontrolnet.py:47-73 does, or averaged as
    unet_2d_condition.py:1418-1439 does), UNet, guidance combine, Euler step. The model runs in the dtype of `sd`
    (fp32 in the tests); the latent is kept in fp16 between steps as the reference does when `half_latents`."""
    ts, sig, _ = euler_sigmas(num_inference_steps)
    scales = list(conditioning_scales) if conditioning_scales else [0.5] * len(controlnets)
    wdt = next(iter(sd.values())).dtype
    for i in range(num_inference_steps):
        x = euler_scale_model_input(latents, sig[i])
        x2 = torch.cat([x, x]).to(wdt)
        down = mid = None
        for cn_sd, s in zip(controlnets, scales):
            d, m = controlnet_step(cn_sd, cfg, x2, float(ts[i]), prompt_embeds.to(wdt), controlnet_cond.to(wdt),
                                   text_embeds.to(wdt), time_ids.to(wdt), s)
            down = d if down is None else [a + b for a, b in zip(down, d)]
            mid = m if mid is None else mid + m
        if down is not None and combine == "mean":
            down = [a / len(controlnets) for a in down]
            mid = mid / len(controlnets)
        eps = unet_step(sd, cfg, x2, float(ts[i]), prompt_embeds.to(wdt), text_embeds.to(wdt), time_ids.to(wdt), down, mid)
        eps = eps.to(latents.dtype) if half_latents else eps
        e = cfg_combine(eps[0:1], eps[1:2], guidance_scale)
        latents = euler_step(latents, e, sig[i], sig[i + 1])
    return latents
