"""GPU parity of the UNet / ControlNet step against the CPU fp32 oracle (which tests/test_oracle_golden.py pins to the
reference's own classes). Tolerances are the ones the baseline states for this path: <= 1e-2 max-abs on the fp16 UNet
output and <= 2e-3 relative L2."""
from collections import OrderedDict

import pytest
import torch

from katz_b200.params import (SDXL_UNET_CONFIG, TINY_UNET_CONFIG, controlnet_param_shapes, init_state_dict,
                              lora_target_keys, unet_param_shapes)
from tests.golden.make_golden import tiny_inputs

pytestmark = pytest.mark.gpu


def _rel_l2(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm())


def _maxabs(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max())


def _f32(sd):
    return OrderedDict((k, v.float()) for k, v in sd.items())


@pytest.fixture(scope="module")
def tiny(cuda_device):
    from katz_b200.unet import KatzControlNet, KatzUNet
    cfg = TINY_UNET_CONFIG
    sd = init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16)
    cn_sd = init_state_dict(controlnet_param_shapes(cfg), seed=2, dtype=torch.float16)
    unet = KatzUNet(cfg, cuda_device, sd)
    cn = KatzControlNet(cfg, cuda_device, cn_sd)
    sample, ctx, te, ti, cond = (t.half() for t in tiny_inputs(cfg))
    return dict(cfg=cfg, sd=sd, cn_sd=cn_sd, unet=unet, cn=cn, inputs=(sample, ctx, te, ti, cond))


def test_state_dict_round_trip(tiny):
    out = tiny["unet"].state_dict()
    assert list(out.keys()) == list(tiny["sd"].keys())
    for k, v in tiny["sd"].items():
        assert torch.equal(out[k].cpu(), v), k


def test_tiny_unet_step_plain(tiny):
    from oracle import unet_oracle
    sample, ctx, te, ti, cond = tiny["inputs"]
    with torch.no_grad():
        ref = unet_oracle.unet_step(_f32(tiny["sd"]), tiny["cfg"], sample.float(), 500.0, ctx.float(), te.float(), ti.float())
    out = tiny["unet"](sample.cuda(), torch.tensor(500.0), encoder_hidden_states=ctx.cuda(),
                       added_cond_kwargs={"text_embeds": te.cuda(), "time_ids": ti.cuda()}, return_dict=False)[0]
    assert out.shape == ref.shape and out.dtype == torch.float16
    assert _maxabs(out, ref) <= 1e-2 and _rel_l2(out, ref) <= 2e-3, (_maxabs(out, ref), _rel_l2(out, ref))


def test_tiny_controlnet_and_intake(tiny):
    from oracle import unet_oracle
    sample, ctx, te, ti, cond = tiny["inputs"]
    cfg = tiny["cfg"]
    with torch.no_grad():
        rdown, rmid = unet_oracle.controlnet_step(_f32(tiny["cn_sd"]), cfg, sample.float(), 500.0, ctx.float(), cond.float(),
                                                  te.float(), ti.float(), 0.5)
        ref = unet_oracle.unet_step(_f32(tiny["sd"]), cfg, sample.float(), 500.0, ctx.float(), te.float(), ti.float(),
                                    rdown, rmid)
    added = {"text_embeds": te.cuda(), "time_ids": ti.cuda()}
    down, mid = tiny["cn"](sample.cuda(), torch.tensor(500.0), encoder_hidden_states=ctx.cuda(), controlnet_cond=cond.cuda(),
                           added_cond_kwargs=added)
    assert len(down) == 9
    for d, r in zip(down, rdown):
        assert d.shape == r.shape
        assert _maxabs(d, r) <= 1e-2 and _rel_l2(d, r) <= 2e-3, (_maxabs(d, r), _rel_l2(d, r))
    assert _rel_l2(mid, rmid) <= 2e-3
    out = tiny["unet"](sample.cuda(), torch.tensor(500.0), encoder_hidden_states=ctx.cuda(), added_cond_kwargs=added,
                       down_block_additional_residuals=down, mid_block_additional_residual=mid, return_dict=False)[0]
    assert _maxabs(out, ref) <= 1e-2 and _rel_l2(out, ref) <= 2e-3, (_maxabs(out, ref), _rel_l2(out, ref))
    # NHWC hand-off between an in-process ControlNet and the UNet gives the same bits as the NCHW round trip
    down2, mid2 = tiny["cn"](sample.cuda(), torch.tensor(500.0), encoder_hidden_states=ctx.cuda(), controlnet_cond=cond.cuda(),
                             added_cond_kwargs=added, nhwc_out=True)
    out2 = tiny["unet"](sample.cuda(), torch.tensor(500.0), encoder_hidden_states=ctx.cuda(), added_cond_kwargs=added,
                        down_block_additional_residuals=down2, mid_block_additional_residual=mid2, return_dict=False)[0]
    assert torch.equal(out, out2)


def test_tiny_unet_with_lora_merged_then_restored(tiny):
    """Configuration 2 in small: one LoRA merged into every targeted linear, step, restore, step."""
    from katz_b200.lora import LoraMerger, merge_lora_state_dicts, synthetic_key_map
    from oracle import lora_oracle, unet_oracle
    cfg, unet = tiny["cfg"], tiny["unet"]
    sample, ctx, te, ti, cond = tiny["inputs"]
    keys = lora_target_keys(cfg, include_proj=True)
    km = synthetic_key_map(keys)
    shapes = unet_param_shapes(cfg)
    g = torch.Generator().manual_seed(11)
    lora_sd = {}
    for k in keys:
        o, n = shapes[k]
        lora_sd[km[k]["lora_down_key"]] = (torch.randn(16, n, generator=g) / 16).half()
        lora_sd[km[k]["lora_up_key"]] = (torch.randn(o, 16, generator=g) * 0.02).half()
    merger = LoraMerger(unet.lora_targets(keys))
    added = {"text_embeds": te.cuda(), "time_ids": ti.cuda()}
    args = (sample.cuda(), torch.tensor(500.0))
    before = unet(*args, encoder_hidden_states=ctx.cuda(), added_cond_kwargs=added)[0]
    merge_lora_state_dicts(unet, merger, lora_sd, km, scale=1.0)
    merged_sd = dict(tiny["sd"])
    ad = {k: (lora_sd[km[k]["lora_up_key"]], lora_sd[km[k]["lora_down_key"]]) for k in keys}
    merged_sd.update(lora_oracle.merge_set({k: tiny["sd"][k] for k in keys}, [ad], [1.0]))
    with torch.no_grad():
        ref = unet_oracle.unet_step(_f32(merged_sd), cfg, sample.float(), 500.0, ctx.float(), te.float(), ti.float())
    out = unet(*args, encoder_hidden_states=ctx.cuda(), added_cond_kwargs=added)[0]
    assert _maxabs(out, ref) <= 1e-2 and _rel_l2(out, ref) <= 2e-3, (_maxabs(out, ref), _rel_l2(out, ref))
    assert _rel_l2(out, before) > 1e-2       # the adapter changed the prediction
    merger.restore()
    unet.invalidate_caches()
    after = unet(*args, encoder_hidden_states=ctx.cuda(), added_cond_kwargs=added)[0]
    assert torch.equal(after, before)         # bit-exact restore -> bit-identical step
    sd_after = unet.state_dict()
    for k in keys:
        assert torch.equal(sd_after[k].cpu(), tiny["sd"][k])


def test_unet_requires_added_cond_kwargs(tiny):
    sample, ctx, te, ti, cond = tiny["inputs"]
    with pytest.raises(ValueError):
        tiny["unet"](sample.cuda(), torch.tensor(1.0), encoder_hidden_states=ctx.cuda(), added_cond_kwargs={"text_embeds": te})


def test_tiny_unet_step_with_layer_norms_folded_into_their_gemms(tiny):
    """`fuse_ln`: every transformer LayerNorm applied in the epilogue of the GEMM that consumes it (off by default: slower on
    the SDXL step, see KatzUNet). Same oracle, same bounds; a LoRA merge must reach the folded copies of the weights."""
    from katz_b200.params import lora_target_keys
    from oracle import unet_oracle
    sample, ctx, te, ti, cond = tiny["inputs"]
    unet = tiny["unet"]
    with torch.no_grad():
        ref = unet_oracle.unet_step(_f32(tiny["sd"]), tiny["cfg"], sample.float(), 500.0, ctx.float(), te.float(), ti.float())
    kw = dict(encoder_hidden_states=ctx.cuda(), added_cond_kwargs={"text_embeds": te.cuda(), "time_ids": ti.cuda()})
    plain = unet(sample.cuda(), torch.tensor(500.0), **kw)[0].clone()
    unet.fuse_ln = True
    try:
        out = unet(sample.cuda(), torch.tensor(500.0), **kw)[0].clone()
        assert unet._folds and _maxabs(out, ref) <= 1e-2 and _rel_l2(out, ref) <= 2e-3, (_maxabs(out, ref), _rel_l2(out, ref))
        assert _rel_l2(out, plain) <= 2e-3 and not torch.equal(out, plain)      # a different rounding sequence, the same result
        keys = lora_target_keys(tiny["cfg"], include_proj=True)
        merger = unet.lora_merger(keys)
        g = torch.Generator().manual_seed(5)
        ad = {k: ((torch.randn(w.shape[0], 8, generator=g) * 0.05).half().cuda(), (torch.randn(8, w.shape[1], generator=g) / 8).half().cuda())
              for k, w in unet.lora_targets(keys).items()}
        merger.merge(ad, 1.0)
        merged = unet(sample.cuda(), torch.tensor(500.0), **kw)[0].clone()
        unet.fuse_ln = False
        merged_plain = unet(sample.cuda(), torch.tensor(500.0), **kw)[0].clone()
        assert _rel_l2(merged, merged_plain) <= 2e-3 and _rel_l2(merged, out) > 1e-2
        merger.restore()
        unet.fuse_ln = True
        assert torch.equal(unet(sample.cuda(), torch.tensor(500.0), **kw)[0], out)
    finally:
        unet.fuse_ln = False
