"""CPU: the oracle reproduces what the reference's own classes produced (tests/golden, made by make_golden.py) and the
known answers of the reference's scheduler tests."""
import json
import os

import numpy as np
import torch

from katz_b200.params import (SDXL_UNET_CONFIG, TINY_UNET_CONFIG, controlnet_param_shapes, init_state_dict,
                              lora_target_keys, unet_param_shapes)
from oracle import lora_oracle, unet_oracle
from tests.golden.make_golden import _shape_digest, tiny_inputs


def test_parameter_inventory_matches_reference(golden_dir):
    meta = json.load(open(os.path.join(golden_dir, "meta.json")))
    shapes = unet_param_shapes(SDXL_UNET_CONFIG)
    assert _shape_digest(shapes) == meta["sdxl_unet_shape_digest"]
    assert sum(int(np.prod(s)) for s in shapes.values()) == meta["sdxl_unet_params"] == 2567463684
    cn = controlnet_param_shapes(SDXL_UNET_CONFIG)
    assert _shape_digest(cn) == meta["sdxl_controlnet_shape_digest"]
    assert len(shapes) == 1680
    # LoRA target sets: 700 transformer-block linears (2,183,987,200 weights); 722 with proj_in/proj_out
    k700 = lora_target_keys(SDXL_UNET_CONFIG)
    k722 = lora_target_keys(SDXL_UNET_CONFIG, include_proj=True)
    assert len(k700) == 700 and len(k722) == meta["lora_key_map_entries"] == 722
    assert sum(int(np.prod(shapes[k])) for k in k700) == 2183987200
    assert sum(int(np.prod(shapes[k])) for k in k722) == 2207744000


def test_tiny_unet_step_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "tiny_unet_step.npz"))
    cfg = TINY_UNET_CONFIG
    sd = init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float32)
    cn_sd = init_state_dict(controlnet_param_shapes(cfg), seed=2, dtype=torch.float32)
    sample, ctx, te, ti, cond = tiny_inputs(cfg)
    with torch.no_grad():
        down, mid = unet_oracle.controlnet_step(cn_sd, cfg, sample, 500.0, ctx, cond, te, ti, 0.5)
        plain = unet_oracle.unet_step(sd, cfg, sample, 500.0, ctx, te, ti)
        with_cn = unet_oracle.unet_step(sd, cfg, sample, 500.0, ctx, te, ti, down, mid)
        mid_sample, emb, res = unet_oracle.unet_down_forward(sd, cfg, sample, 500.0, ctx, te, ti)
    assert len(down) == 9 and len(res) == 9
    np.testing.assert_allclose(emb.numpy(), g["emb"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(mid_sample.numpy(), g["unet_mid_sample"], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(plain.numpy(), g["noise_pred_plain"], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(with_cn.numpy(), g["noise_pred_controlnet"], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(mid.numpy(), g["cn_mid"], rtol=1e-4, atol=1e-4)
    for i, d in enumerate(down):
        np.testing.assert_allclose(d[:, :, ::2, ::2].numpy(), g["cn_down_%d" % i], rtol=1e-4, atol=1e-4)
    # the residuals matter: the two predictions differ
    assert np.abs(g["noise_pred_plain"] - g["noise_pred_controlnet"]).max() > 1e-3


def test_euler_schedule_and_fp16_steps_match_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "euler_sdxl.npz"))
    ts, sig, init = unet_oracle.euler_sigmas(50)
    np.testing.assert_array_equal(ts.numpy(), g["timesteps"])
    np.testing.assert_array_equal(sig.numpy(), g["sigmas"])
    assert abs(init - float(g["init_noise_sigma"])) < 1e-6
    assert ts[0] == 981 and ts[-1] == 1 and abs(float(sig[0]) - 13.12) < 0.01
    lat = torch.from_numpy(g["latent0"])
    for i in range(4):
        inp = unet_oracle.euler_scale_model_input(lat, sig[i])
        assert torch.equal(inp, torch.from_numpy(g["scaled_%d" % i]))
        u, c = torch.from_numpy(g["eps_u_%d" % i]), torch.from_numpy(g["eps_c_%d" % i])
        eps = unet_oracle.cfg_combine(u, c, 5.0)
        lat = unet_oracle.euler_step(lat, eps, sig[i], sig[i + 1])
        assert torch.equal(lat, torch.from_numpy(g["latent_%d" % (i + 1)]))


def test_euler_known_answer_full_loop():
    """tests/schedulers/test_scheduler_euler.py:52-77 of the reference: linear betas 1e-4..0.02, 1100 train steps,
    10 linspace steps, model(sample,t) = sample*t/(t+1): |sum| = 10.0807, mean|x| = 0.0131."""
    ts, sig, init = unet_oracle.euler_sigmas(10, num_train_timesteps=1100, beta_start=0.0001, beta_end=0.02,
                                             steps_offset=0, beta_schedule="linear", timestep_spacing="linspace")
    n = 4 * 3 * 8 * 8
    sample = (torch.arange(n).reshape(3, 8, 8, 4) / n).permute(3, 0, 1, 2) * init
    for i, t in enumerate(ts):
        sample = unet_oracle.euler_scale_model_input(sample, sig[i])   # the reference test overwrites the sample
        out = sample * t / (t + 1)
        sample = unet_oracle.euler_step(sample, out, sig[i], sig[i + 1])
    assert abs(float(sample.abs().sum()) - 10.0807) < 1e-2
    assert abs(float(sample.abs().mean()) - 0.0131) < 1e-3


def test_lora_oracle_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "lora_small.npz"))
    W, up, down = (torch.from_numpy(g[k]) for k in ("W", "up", "down"))
    fused = lora_oracle.fuse_lora_vendored(W, up, down, 16.0, 16)
    assert torch.equal(fused, torch.from_numpy(g["W_fused"]))
    un = lora_oracle.unfuse_lora_vendored(fused, up, down, 16.0, 16)
    assert torch.equal(un, torch.from_numpy(g["W_unfused"]))
    # subtractive unmerge is close to, but not bit-equal to, the original weights
    assert not torch.equal(un, W) and (un - W).abs().max() < 1e-7
    W16, up16, down16 = (torch.from_numpy(g[k]) for k in ("W16", "up16", "down16"))
    merged = lora_oracle.merge_katz(W16, up16, down16, 20000.0 / 64.0)
    assert torch.equal(merged, torch.from_numpy(g["W16_merged"]))
    # copy restore is bit-exact
    assert torch.equal(lora_oracle.restore({"w": W16})["w"], W16)


def test_vae_oracle_equals_reference_autoencoder(golden_dir):
    """oracle.vae_oracle.vae_decode against the reference's AutoencoderKL.decode on the tiny seeded decoder."""
    import os
    import numpy as np
    import torch
    from katz_b200.params import (SDXL_VAE_CONFIG, TINY_VAE_CONFIG, init_state_dict, vae_decode_flops,
                                  vae_decoder_param_shapes)
    from oracle import vae_oracle
    gold = np.load(os.path.join(golden_dir, "tiny_vae_decode.npz"))
    sd = init_state_dict(vae_decoder_param_shapes(TINY_VAE_CONFIG), seed=3, dtype=torch.float32)
    out = vae_oracle.vae_decode(sd, TINY_VAE_CONFIG, torch.from_numpy(gold["z"]))
    assert float((out - torch.from_numpy(gold["image"])).abs().max()) <= 1e-5
    import json
    with open(os.path.join(golden_dir, "meta.json")) as fr:
        meta = json.load(fr)
    shapes = vae_decoder_param_shapes(SDXL_VAE_CONFIG)
    assert sum(int(np.prod(s)) for s in shapes.values()) == meta["sdxl_vae_decoder_params"] == 49490199
    assert abs(vae_decode_flops(SDXL_VAE_CONFIG, 1, 128, 128) / 1e12 - 10.47) < 0.01
    assert vae_oracle.SDXL_VAE_CONFIG == SDXL_VAE_CONFIG
