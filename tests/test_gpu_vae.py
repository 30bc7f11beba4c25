"""VAE decode on the library's kernels against the oracle (itself equal to the reference's AutoencoderKL on the tiny
fixture, tests/test_oracle_golden.py) — tiny configuration, then the SDXL decoder at 1024x1024 pixels."""
import os

import numpy as np
import pytest
import torch

from katz_b200.params import SDXL_VAE_CONFIG, TINY_VAE_CONFIG, init_state_dict, vae_decode_flops, vae_decoder_param_shapes

pytestmark = pytest.mark.gpu


def _rel_l2(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm())


def test_softmax_rows(cuda_device):
    from katz_b200 import ops
    g = torch.Generator().manual_seed(2)
    for rows, cols in ((7, 64), (300, 1000), (64, 16384), (5, 8)):
        x = (torch.randn(rows, cols, generator=g) * 3).half().cuda()
        ref = torch.softmax(x.float(), dim=1)
        y = ops.softmax_rows(x)
        assert float((y.float() - ref).abs().max()) <= 2 ** -10 * float(ref.max()) + 1e-7, (rows, cols)
        assert float((y.float().sum(1) - 1).abs().max()) < 2e-3
        z = x.clone()
        ops.softmax_rows(z, out=z)                       # in place
        assert torch.equal(z, y)
    wide = torch.zeros(4, 2048, dtype=torch.float16, device="cuda")
    view = wide[:, :1000]                                # strided rows
    view.copy_(torch.randn(4, 1000, generator=g).half())
    assert torch.equal(ops.softmax_rows(view), ops.softmax_rows(view.contiguous()))
    with pytest.raises(Exception):
        ops.softmax_rows(torch.zeros(2, 16392, dtype=torch.float16, device="cuda"))   # longer than a row held in registers
    with pytest.raises(Exception):
        ops.softmax_rows(torch.zeros(2, 12, dtype=torch.float16, device="cuda"))


def test_tiny_vae_decode_against_reference_fixture_and_oracle(cuda_device, golden_dir):
    from katz_b200 import ops
    from katz_b200.vae import KatzVaeDecoder
    from oracle import vae_oracle
    cfg = TINY_VAE_CONFIG
    gold = np.load(os.path.join(golden_dir, "tiny_vae_decode.npz"))
    sd16 = init_state_dict(vae_decoder_param_shapes(cfg), seed=3, dtype=torch.float16)
    dec = KatzVaeDecoder(cfg, cuda_device, sd16)
    z = torch.from_numpy(gold["z"]).half()
    out = dec.decode(z.cuda())
    assert out.shape == (2, 3, 32, 32) and out.dtype == torch.float16 and ops.tc05_status() == 0
    # against the oracle on the same fp16-rounded weights and latent (fp32 arithmetic) ...
    ref = vae_oracle.vae_decode({k: v.float() for k, v in sd16.items()}, cfg, z.float())
    assert _rel_l2(out, ref) <= 2e-3 and float((out.float().cpu() - ref).abs().max()) <= 1e-2
    # ... and against what the reference's own AutoencoderKL returned for the fp32 weights (fp16 rounding of weights included)
    assert _rel_l2(out, torch.from_numpy(gold["image"])) <= 4e-3
    # graph replay gives the same bits, follows a new latent, and the scaling entry matches a manual division
    dec.use_cuda_graph = True
    assert torch.equal(dec.decode(z.cuda()), out)
    z2 = (z * 0.5 + 0.1).cuda()
    g2 = dec.decode(z2).clone()
    dec.use_cuda_graph = False
    assert torch.equal(g2, dec.decode(z2))
    assert torch.equal(dec.decode_latents(z2), dec.decode(z2 / cfg["scaling_factor"]))
    # state dict round trip in the reference layout; upstream's norm1/norm2 spelling is accepted
    back = dec.state_dict()
    for k, v in sd16.items():
        assert torch.equal(back[k].cpu(), v), k
    renamed = {k.replace(".norm_silu1.0.", ".norm1.").replace(".norm_silu2.0.", ".norm2."): v for k, v in sd16.items()}
    assert torch.equal(KatzVaeDecoder(cfg, cuda_device, renamed).decode(z.cuda()), out)
    with pytest.raises(Exception):
        dec.decode(z.cuda().float())
    with pytest.raises(Exception):
        KatzVaeDecoder(cfg, cuda_device, {k: v for k, v in list(sd16.items())[:-2]})


def test_sdxl_vae_decode_1024_against_oracle(cuda_device):
    """The SDXL decoder (49.5 M parameters) on a 128x128 latent -> 1024x1024 pixels: every kernel at the size the
    pipeline uses, the 16384-token one-head attention included, against the oracle in strict fp32 on the GPU."""
    from katz_b200 import ops
    from katz_b200.vae import KatzVaeDecoder
    from oracle import vae_oracle
    cfg = SDXL_VAE_CONFIG
    sd16 = init_state_dict(vae_decoder_param_shapes(cfg), seed=5, dtype=torch.float16, device=cuda_device, generator_device=cuda_device)
    g = torch.Generator().manual_seed(6)
    lat = (torch.randn(1, 4, 128, 128, generator=g) * cfg["scaling_factor"]).half().cuda()
    dec = KatzVaeDecoder(cfg, cuda_device, sd16)
    out = dec.decode_latents(lat)
    assert out.shape == (1, 3, 1024, 1024) and ops.tc05_status() == 0 and bool(torch.isfinite(out).all())
    tf32 = (torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32)
    torch.backends.cuda.matmul.allow_tf32 = torch.backends.cudnn.allow_tf32 = False
    try:
        ref = vae_oracle.decode_latents({k: v.float() for k, v in sd16.items()}, cfg, lat.float())
    finally:
        torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = tf32
    rel, mx = _rel_l2(out, ref), float((out.float() - ref).abs().max())
    print("sdxl vae decode 1024: rel-l2 %.2e max-abs %.2e (output rms %.3f)" % (rel, mx, float(ref.pow(2).mean().sqrt())))
    assert rel <= 2e-3, rel
    assert vae_decode_flops(cfg, 1, 128, 128) > 1e13
