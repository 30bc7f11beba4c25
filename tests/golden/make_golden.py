"""Generates tests/golden/*.npz / *.json by running the REFERENCE's own classes (imported from the reference tree) on
small seeded configs. Run it where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It needs three import shims (the reference pins older dependency versions): an empty `fast_kernel` stub package (the
fused ops are never called with ENABLE_FUSED_* unset), `huggingface_hub.cached_download`, and
`transformers.utils.FLAX_WEIGHTS_NAME`. Weights and inputs come from numpy's PCG64 streams through
katz_b200.params.init_state_dict, so the tests can rebuild them anywhere and only outputs are stored.
"""
import hashlib
import json
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def _import_reference(ref_root):
    shim = tempfile.mkdtemp(prefix="katz_shim_")
    os.makedirs(os.path.join(shim, "fast_kernel"))
    open(os.path.join(shim, "fast_kernel", "__init__.py"), "w").close()
    sys.path.insert(0, shim)
    sys.path.insert(0, os.path.join(ref_root, "diffusers-hf", "src"))
    for k in ("ENABLE_FUSED_GEGLU", "ENABLE_FUSED_NORM_SILU", "ENABLE_CUDA_GRAPH", "ENABLE_CHANNELS_LAST"):
        os.environ.pop(k, None)
    import huggingface_hub
    if not hasattr(huggingface_hub, "cached_download"):
        huggingface_hub.cached_download = huggingface_hub.hf_hub_download
    import transformers.utils as tu
    if not hasattr(tu, "FLAX_WEIGHTS_NAME"):
        tu.FLAX_WEIGHTS_NAME = "flax_model.msgpack"
    import diffusers
    return diffusers


def _ref_unet_kwargs(cfg):
    return dict(sample_size=cfg["sample_size"], in_channels=4, out_channels=4,
                block_out_channels=cfg["block_out_channels"], down_block_types=cfg["down_block_types"],
                up_block_types=cfg["up_block_types"], layers_per_block=cfg["layers_per_block"],
                transformer_layers_per_block=cfg["transformer_layers_per_block"],
                attention_head_dim=cfg["attention_head_dim"], cross_attention_dim=cfg["cross_attention_dim"],
                use_linear_projection=True, addition_embed_type="text_time",
                addition_time_embed_dim=cfg["addition_time_embed_dim"],
                projection_class_embeddings_input_dim=cfg["projection_class_embeddings_input_dim"],
                norm_num_groups=cfg["norm_num_groups"], act_fn="silu")


def _shape_digest(shapes):
    lines = sorted("%s %s" % (k, tuple(int(x) for x in v)) for k, v in shapes.items())
    return hashlib.sha256("\n".join(lines).encode()).hexdigest()


def tiny_inputs(cfg, seed=1, batch=2):
    rng = np.random.default_rng(seed)
    s = cfg["sample_size"]
    sample = torch.from_numpy(rng.standard_normal((batch, 4, s, s), dtype=np.float32))
    ctx = torch.from_numpy(rng.standard_normal((batch, 77, cfg["cross_attention_dim"]), dtype=np.float32))
    n_text = cfg["projection_class_embeddings_input_dim"] - 6 * cfg["addition_time_embed_dim"]
    text_embeds = torch.from_numpy(rng.standard_normal((batch, n_text), dtype=np.float32))
    time_ids = torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * batch)
    low = torch.from_numpy(rng.random((1, 3, 4, 4), dtype=np.float32))
    cond = torch.nn.functional.interpolate(low, size=(8 * s, 8 * s), mode="bicubic", align_corners=False).clamp(0, 1)
    cond = cond.repeat(batch, 1, 1, 1)
    return sample, ctx, text_embeds, time_ids, cond


def kohya_names():
    """Synthetic kohya-ss LoRA module names with the structure of an SDXL adapter (SGM block numbering for the UNet, both
    text encoders): every block position, two transformer layers per attention, resnet convolutions, time-embedding
    projections, shortcuts, down/upsamplers. Names only: no file of any adapter is reproduced."""
    names = []
    attn = ["attn1_to_q", "attn1_to_k", "attn1_to_v", "attn1_to_out_0", "attn2_to_q", "attn2_to_k", "attn2_to_v", "attn2_to_out_0",
            "ff_net_0_proj", "ff_net_2"]
    res = ["in_layers_2", "emb_layers_1", "out_layers_3"]

    def transformer(prefix):
        return [prefix + "_proj_in", prefix + "_proj_out"] + ["%s_transformer_blocks_%d_%s" % (prefix, j, leaf) for j in range(2) for leaf in attn]
    for n in (1, 2, 4, 5, 7, 8):
        names += ["lora_unet_input_blocks_%d_0_%s" % (n, leaf) for leaf in res]
        if n in (4, 7):
            names.append("lora_unet_input_blocks_%d_0_skip_connection" % n)
        if n >= 4:
            names += transformer("lora_unet_input_blocks_%d_1" % n)
    names += ["lora_unet_input_blocks_3_0_op", "lora_unet_input_blocks_6_0_op"]
    for m in (0, 2):
        names += ["lora_unet_middle_block_%d_%s" % (m, leaf) for leaf in res]
    names += transformer("lora_unet_middle_block_1")
    for n in range(9):
        names += ["lora_unet_output_blocks_%d_0_%s" % (n, leaf) for leaf in res + ["skip_connection"]]
        if n < 6:
            names += transformer("lora_unet_output_blocks_%d_1" % n)
    names += ["lora_unet_output_blocks_2_2_conv", "lora_unet_output_blocks_5_2_conv"]
    for te in ("lora_te1", "lora_te2"):
        for i in (0, 11):
            names += ["%s_text_model_encoder_layers_%d_self_attn_%s_proj" % (te, i, p) for p in ("q", "k", "v", "out")]
            names += ["%s_text_model_encoder_layers_%d_mlp_fc%d" % (te, i, f) for f in (1, 2)]
    return names


def kohya_state_dict(names):
    """One-element tensors whose VALUE identifies the entry, so a renamed dict can be matched back to its source."""
    sd = {}
    for i, n in enumerate(names):
        sd[n + ".lora_down.weight"] = torch.full((1,), float(2 * i))
        sd[n + ".lora_up.weight"] = torch.full((1,), float(2 * i + 1))
        sd[n + ".alpha"] = torch.tensor(float(i % 7 + 1))
    return sd


def kohya_fixture(out_dir):
    """kohya_keys.json: what the reference's own conversion (lora_conversion_utils.py:23-287, as LoraLoaderMixin.lora_state_dict
    chains it, loaders/lora.py:290-305) makes of kohya_names(): {kohya tensor key: diffusers key} and the alphas."""
    import types
    from diffusers.loaders.lora_conversion_utils import _convert_kohya_lora_to_diffusers, _maybe_map_sgm_blocks_to_diffusers
    sd = kohya_state_dict(kohya_names())
    by_value = {float(v): k for k, v in sd.items() if not k.endswith(".alpha")}
    new_sd, alphas = _convert_kohya_lora_to_diffusers(_maybe_map_sgm_blocks_to_diffusers(dict(sd), types.SimpleNamespace(layers_per_block=2)))
    mapping = {by_value[float(v)]: k for k, v in new_sd.items()}
    assert len(mapping) == len(by_value)
    with open(os.path.join(out_dir, "kohya_keys.json"), "w") as fw:
        json.dump({"keys": mapping, "alphas": alphas}, fw, indent=0, sort_keys=True)


def cache_fixture(ref_root, out_dir):
    """cache_counts.json: the loads the reference's own analysis (trace/adapter_loading_analysis.py:48-200) counts on a
    seeded synthetic trace (katz_b200.adapter_cache.zipf_trace; the production trace is not distributed), for LRU and
    LFU and cache sizes 1..10. The analysis plots its result; a do-nothing stand-in for the plotting library is put
    in its way, and the counts are read from what it prints."""
    import contextlib
    import importlib.util
    import io
    import re
    import types
    sys.path.insert(0, os.path.normpath(os.path.join(HERE, "..", "..")))
    from katz_b200.adapter_cache import zipf_trace
    trace = zipf_trace(600, n_loras=24, n_controlnets=6, alpha=1.1, instances=3, seed=7, scene_id="A")

    class _Quiet(types.ModuleType):
        def __getattr__(self, name):
            return lambda *a, **k: None
    mpl, plt = _Quiet("matplotlib"), _Quiet("matplotlib.pyplot")
    mpl.rcParams = {}
    mpl.pyplot = plt
    saved = {k: sys.modules.get(k) for k in ("matplotlib", "matplotlib.pyplot")}
    sys.modules["matplotlib"], sys.modules["matplotlib.pyplot"] = mpl, plt
    work = tempfile.mkdtemp(prefix="katz_trace_")
    cwd = os.getcwd()
    counts = {}
    try:
        os.chdir(work)
        with open("trace.json", "w") as fw:
            json.dump(trace, fw)
        spec = importlib.util.spec_from_file_location("ref_adapter_loading", os.path.join(ref_root, "trace", "adapter_loading_analysis.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        for policy in ("LRU", "LFU"):
            buf = io.StringIO()
            with contextlib.redirect_stdout(buf):
                mod.adapter_loading_analysis("trace.json", "A", policy)
            counts[policy] = {"loras": {}, "controlnets": {}}
            for size, kind, n in re.findall(r"Cache size: (\d+), overall switch (controlnet|lora) times: (\d+)", buf.getvalue()):
                counts[policy][kind + "s"][size] = int(n)
            assert len(counts[policy]["loras"]) == 10 and len(counts[policy]["controlnets"]) == 10
    finally:
        os.chdir(cwd)
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    with open(os.path.join(out_dir, "cache_counts.json"), "w") as fw:
        json.dump({"trace": trace, "loads": counts}, fw, sort_keys=True)


def text_encoder_key_map_fixture(ref_root, out_dir):
    """text_encoder_key_maps.json: digest and size of the reference's two text-encoder key maps together with the adapter
    tensor shapes its shape inventory lists for them (lora_info_shm/TheLastBen_Filmic*.json)."""
    info = os.path.join(ref_root, "lora_info_shm")
    with open(os.path.join(info, "TheLastBen_Filmic.json")) as fr:
        inventory = json.load(fr)
    out = {}
    for which in ("text_encoder", "text_encoder_2"):
        with open(os.path.join(info, "TheLastBen_Filmic_key_match_%s.json" % which)) as fr:
            km = json.load(fr)
        lines = sorted("%s %s %s %s %s" % (k, m["lora_down_key"], m["lora_up_key"], tuple(inventory[m["lora_down_key"]]["shape"]),
                                           tuple(inventory[m["lora_up_key"]]["shape"])) for k, m in km.items())
        out[which] = {"entries": len(km), "order": list(km)[:6], "digest": hashlib.sha256("\n".join(lines).encode()).hexdigest()}
    with open(os.path.join(out_dir, "text_encoder_key_maps.json"), "w") as fw:
        json.dump(out, fw, indent=1, sort_keys=True)


def vae_fixture(out_dir):
    """tiny_vae_decode.npz: what the reference's AutoencoderKL.decode (models/autoencoders/autoencoder_kl.py) returns for a
    tiny three-level decoder with seeded weights (katz_b200.params.init_state_dict, seed 3) on a seeded latent, fp32."""
    from diffusers import AutoencoderKL
    from katz_b200.params import TINY_VAE_CONFIG, init_state_dict, vae_decoder_param_shapes
    cfg = TINY_VAE_CONFIG
    n = len(cfg["block_out_channels"])
    vae = AutoencoderKL(in_channels=3, out_channels=cfg["out_channels"], down_block_types=("DownEncoderBlock2D",) * n,
                        up_block_types=("UpDecoderBlock2D",) * n, block_out_channels=cfg["block_out_channels"],
                        layers_per_block=cfg["layers_per_block"], latent_channels=cfg["latent_channels"],
                        norm_num_groups=cfg["norm_num_groups"], sample_size=32, scaling_factor=cfg["scaling_factor"]).eval()
    shapes = vae_decoder_param_shapes(cfg)
    ref_shapes = {k: tuple(v.shape) for k, v in vae.state_dict().items() if k.startswith("decoder.") or k.startswith("post_quant_conv.")}
    assert ref_shapes == {k: tuple(v) for k, v in shapes.items()}, "decoder parameter inventory differs from the reference's"
    sd = init_state_dict(shapes, seed=3, dtype=torch.float32)
    missing, unexpected = vae.load_state_dict(sd, strict=False)
    assert not unexpected and all(k.startswith("encoder.") or k.startswith("quant_conv.") for k in missing)
    rng = np.random.default_rng(11)
    z = torch.from_numpy(rng.standard_normal((2, cfg["latent_channels"], 8, 8), dtype=np.float32))
    with torch.no_grad():
        img = vae.decode(z, return_dict=False)[0]
    np.savez_compressed(os.path.join(out_dir, "tiny_vae_decode.npz"), z=z.numpy(), image=img.numpy())
    return _shape_digest(ref_shapes)


def main(ref_root):
    diffusers = _import_reference(ref_root)
    kohya_fixture(HERE)
    vae_fixture(HERE)
    cache_fixture(ref_root, HERE)
    text_encoder_key_map_fixture(ref_root, HERE)
    from diffusers import ControlNetModel, EulerDiscreteScheduler, UNet2DConditionModel
    from diffusers.models.lora import LoRACompatibleLinear, LoRALinearLayer
    from katz_b200.params import (SDXL_UNET_CONFIG, TINY_UNET_CONFIG, controlnet_param_shapes, init_state_dict,
                                  lora_target_keys, unet_param_shapes)

    meta = {}
    # ---- 1. parameter inventory of the full SDXL models equals the reference's
    with torch.device("meta"):
        ref_unet = UNet2DConditionModel(**_ref_unet_kwargs(SDXL_UNET_CONFIG))
        ref_cn = ControlNetModel.from_unet(ref_unet, load_weights_from_unet=False)
    ref_shapes = {k: tuple(v.shape) for k, v in ref_unet.state_dict().items()}
    mine = {k: tuple(v) for k, v in unet_param_shapes(SDXL_UNET_CONFIG).items()}
    assert ref_shapes == mine, set(ref_shapes.items()) ^ set(mine.items())
    ref_cn_shapes = {k: tuple(v.shape) for k, v in ref_cn.state_dict().items()}
    mine_cn = {k: tuple(v) for k, v in controlnet_param_shapes(SDXL_UNET_CONFIG).items()}
    assert ref_cn_shapes == mine_cn, set(ref_cn_shapes.items()) ^ set(mine_cn.items())
    meta["sdxl_unet_shape_digest"] = _shape_digest(ref_shapes)
    meta["sdxl_unet_params"] = int(sum(int(np.prod(s)) for s in ref_shapes.values()))
    meta["sdxl_controlnet_shape_digest"] = _shape_digest(ref_cn_shapes)
    meta["sdxl_controlnet_params"] = int(sum(int(np.prod(s)) for s in ref_cn_shapes.values()))
    from diffusers import AutoencoderKL
    from katz_b200.params import SDXL_VAE_CONFIG, vae_decoder_param_shapes
    with torch.device("meta"):
        ref_vae = AutoencoderKL(in_channels=3, out_channels=3, down_block_types=("DownEncoderBlock2D",) * 4,
                                up_block_types=("UpDecoderBlock2D",) * 4, block_out_channels=SDXL_VAE_CONFIG["block_out_channels"],
                                layers_per_block=2, latent_channels=4, norm_num_groups=32, sample_size=1024)
    ref_vae_shapes = {k: tuple(v.shape) for k, v in ref_vae.state_dict().items() if k.startswith("decoder.") or k.startswith("post_quant_conv.")}
    assert ref_vae_shapes == {k: tuple(v) for k, v in vae_decoder_param_shapes(SDXL_VAE_CONFIG).items()}
    meta["sdxl_vae_decoder_shape_digest"] = _shape_digest(ref_vae_shapes)
    meta["sdxl_vae_decoder_params"] = int(sum(int(np.prod(s)) for s in ref_vae_shapes.values()))
    # the 722-entry LoRA target set of the reference's key-map fixture
    with open(os.path.join(ref_root, "lora_info_shm", "TheLastBen_Papercut_SDXL_key_match_unet.json")) as fr:
        km = json.load(fr)
    assert sorted(km.keys()) == sorted(lora_target_keys(SDXL_UNET_CONFIG, include_proj=True))
    assert len(lora_target_keys(SDXL_UNET_CONFIG)) == 700
    meta["lora_key_map_digest"] = hashlib.sha256("\n".join(sorted(km.keys())).encode()).hexdigest()
    meta["lora_key_map_entries"] = len(km)

    # ---- 2. tiny UNet + ControlNet step through the reference classes (fp32, CPU)
    cfg = TINY_UNET_CONFIG
    torch.manual_seed(0)
    unet = UNet2DConditionModel(**_ref_unet_kwargs(cfg)).eval()
    sd = init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float32)
    unet.load_state_dict(sd, strict=True)
    cn = ControlNetModel.from_unet(unet, load_weights_from_unet=False).eval()
    cn_sd = init_state_dict(controlnet_param_shapes(cfg), seed=2, dtype=torch.float32)
    cn.load_state_dict(cn_sd, strict=True)
    sample, ctx, te, ti, cond = tiny_inputs(cfg)
    added = {"text_embeds": te, "time_ids": ti}
    t = torch.tensor(500.0)
    out = {}
    with torch.no_grad():
        down, mid = cn._controlnet_forward(sample, t, ctx, cond, conditioning_scale=0.5, added_cond_kwargs=added)
        mid_sample, emb, res, ehs = unet._down_forward(sample, t, ctx, added_cond_kwargs=added)
        zeros = [torch.zeros_like(r) for r in res]
        plain = unet._up_forward(mid_sample, emb, res, zeros, torch.zeros_like(mid_sample), ehs, None, None, None,
                                 return_dict=False)[0]
        with_cn = unet._up_forward(mid_sample, emb, res, down, mid, ehs, None, None, None, return_dict=False)[0]
    assert len(down) == 9
    out["noise_pred_plain"] = plain.numpy()
    out["noise_pred_controlnet"] = with_cn.numpy()
    out["unet_mid_sample"] = mid_sample.numpy()
    out["emb"] = emb.numpy()
    out["cn_mid"] = mid.numpy()
    for i, d in enumerate(down):
        out["cn_down_%d" % i] = d[:, :, ::2, ::2].contiguous().numpy()
    np.savez_compressed(os.path.join(HERE, "tiny_unet_step.npz"), **out)

    # ---- 3. Euler schedule + fp16 step arithmetic through the reference scheduler (SDXL config)
    sch = EulerDiscreteScheduler(num_train_timesteps=1000, beta_start=0.00085, beta_end=0.012, beta_schedule="scaled_linear",
                                 steps_offset=1, timestep_spacing="leading")
    sch.set_timesteps(50)
    eu = {"timesteps": sch.timesteps.numpy(), "sigmas": sch.sigmas.numpy(),
          "init_noise_sigma": np.float32(float(sch.init_noise_sigma))}
    rng = np.random.default_rng(3)
    lat = torch.from_numpy(rng.standard_normal((1, 4, 16, 16), dtype=np.float32)).half() * sch.init_noise_sigma
    lat = lat.half()
    eu["latent0"] = lat.numpy()
    guidance = 5.0
    for i, tt in enumerate(sch.timesteps[:4]):
        inp = sch.scale_model_input(lat, tt)
        eu["scaled_%d" % i] = inp.numpy()
        u = torch.from_numpy(rng.standard_normal((1, 4, 16, 16), dtype=np.float32)).half()
        c = torch.from_numpy(rng.standard_normal((1, 4, 16, 16), dtype=np.float32)).half()
        eu["eps_u_%d" % i], eu["eps_c_%d" % i] = u.numpy(), c.numpy()
        eps = u + guidance * (c - u)
        lat = sch.step(eps, tt, lat, return_dict=False)[0]
        eu["latent_%d" % (i + 1)] = lat.numpy()
    np.savez_compressed(os.path.join(HERE, "euler_sdxl.npz"), **eu)

    # ---- 4. LoRA: the vendored fuse/unfuse arithmetic (models/lora.py:403-449) and the Katz merge formula
    rng = np.random.default_rng(4)
    lo = {}
    out_f, in_f, r = 96, 128, 16
    W = torch.from_numpy(rng.standard_normal((out_f, in_f), dtype=np.float32)) * 0.02
    up = torch.from_numpy(rng.standard_normal((out_f, r), dtype=np.float32)) * 0.01
    down = torch.from_numpy(rng.standard_normal((r, in_f), dtype=np.float32)) / r
    lin = LoRACompatibleLinear(in_f, out_f, bias=False)
    lin.weight.data.copy_(W)
    ll = LoRALinearLayer(in_f, out_f, rank=r, network_alpha=float(r))
    ll.up.weight.data.copy_(up)
    ll.down.weight.data.copy_(down)
    lin.set_lora_layer(ll)
    lin._fuse_lora(lora_scale=1.0)
    lo["W"], lo["up"], lo["down"] = W.numpy(), up.numpy(), down.numpy()
    lo["W_fused"] = lin.weight.data.clone().numpy()
    lin._unfuse_lora()
    lo["W_unfused"] = lin.weight.data.clone().numpy()
    # lora_utils.py:29-33 in fp16 on CPU with the hard-coded scale
    scale = torch.tensor(20000.0 / 64.0, dtype=torch.float16)
    W16 = W.half()
    up16, down16 = (up * 0.05).half(), (down * 0.05).half()
    Wm = W16.clone()
    Wm += up16 @ down16 * scale
    lo["W16"], lo["up16"], lo["down16"], lo["W16_merged"] = W16.numpy(), up16.numpy(), down16.numpy(), Wm.numpy()
    np.savez_compressed(os.path.join(HERE, "lora_small.npz"), **lo)

    meta["torch"] = torch.__version__
    meta["reference"] = "modelscope/Katz (diffusers fork 0.28.0.dev0)"
    with open(os.path.join(HERE, "meta.json"), "w") as fw:
        json.dump(meta, fw, indent=1, sort_keys=True)
    print(json.dumps(meta, indent=1))


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("KATZ_REFERENCE_ROOT"):
        raise SystemExit("usage: python tests/golden/make_golden.py <path of a checkout of the reference project>")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["KATZ_REFERENCE_ROOT"])
