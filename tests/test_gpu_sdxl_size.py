"""GPU parity at the sizes the baseline configurations state (full SDXL UNet, 2.57 B parameters), against the oracle.

  configuration 1   700-layer fp32 LoRA merge -> restore (bit-exact), in-place +/- round trip with the count of elements
                    that do not come back, every layer checked against oracle.lora_oracle
  722-layer table   the fp16 merge the benchmark times, every layer against the oracle
  configuration 2   one UNet step, fp16, batch 2, latent 128x128, one rank-64 LoRA merged
  configuration 3   the same step with one ControlNet (conditioning scale 0.5, 9 + 1 residuals)
  configuration 4   short form: 4 Euler steps, three ControlNets (0.5 / 0.5 / 0.3, summed), LoRAs of rank 64 and 32

Tolerances are the baseline's: UNet output <= 1e-2 max-abs and <= 2e-3 relative L2 against the fp32 oracle, final
latent <= 2e-3 relative L2, restore bit-exact. The oracle runs in fp32 on the CPU for configurations 2 and 3; the same
oracle code in fp32 on the GPU (TF32 off) is first shown to agree with the CPU run and then serves configuration 4, whose
sixteen network evaluations would take minutes on the host cores. Weights are random (seeded, drawn on the device): the
hub checkpoints are not available offline.
"""
import contextlib
from collections import OrderedDict

import pytest
import torch

from katz_b200.params import SDXL_UNET_CONFIG, controlnet_param_shapes, init_state_dict, lora_target_keys, unet_param_shapes

pytestmark = pytest.mark.gpu

CFG = SDXL_UNET_CONFIG
B, HW = 2, 128


def _rel_l2(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm())


def _maxabs(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max())


@contextlib.contextmanager
def _strict_fp32():
    """fp32 torch on the GPU without TF32, so that it is the same arithmetic class as the CPU oracle."""
    a, b = torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    try:
        yield
    finally:
        torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = a, b


def _make_lora(targets, rank, seed, dtype=torch.float16):
    """A ~ N(0, 1/rank), B ~ N(0, 0.01), drawn on the device (configurations 1 and 2)."""
    dev = next(iter(targets.values())).device
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    ad = OrderedDict()
    for k, w in targets.items():
        o, n = w.shape
        down = (torch.randn(rank, n, generator=g, device=dev) / rank).to(dtype)
        up = (torch.randn(o, rank, generator=g, device=dev) * 0.01).to(dtype)
        ad[k] = (up, down)
    return ad


def _cpu(ad):
    return OrderedDict((k, (u.cpu(), d.cpu())) for k, (u, d) in ad.items())


def _inputs(seed=0):
    g = torch.Generator().manual_seed(seed)
    sample = torch.randn(B, 4, HW, HW, generator=g).half()
    ctx = torch.randn(B, 77, 2048, generator=g).half()
    te = torch.randn(B, 1280, generator=g).half()
    ti = torch.tensor([[1024., 1024., 0., 0., 1024., 1024.]] * B).half()
    field = torch.rand(1, 3, 16, 16, generator=g)
    cond = torch.nn.functional.interpolate(field, scale_factor=64, mode="bicubic", align_corners=False).clamp(0, 1)
    return sample, ctx, te, ti, cond.repeat(B, 1, 1, 1).half()


@pytest.fixture(scope="module")
def sdxl(cuda_device):
    from katz_b200.lora import LoraMerger
    from katz_b200.unet import KatzUNet
    dev = cuda_device
    sd = init_state_dict(unet_param_shapes(CFG), seed=0, dtype=torch.float16, device=dev, generator_device=dev)
    unet = KatzUNet(CFG, dev, sd)
    sd16 = OrderedDict((k, v.cpu()) for k, v in sd.items())
    del sd
    keys = lora_target_keys(CFG, include_proj=True)
    assert len(keys) == 722
    merger = LoraMerger(unet.lora_targets(keys), on_change=unet.invalidate_caches)
    return dict(unet=unet, sd16=sd16, keys=keys, merger=merger, inputs=_inputs())


def _oracle_weights(sdxl, adapters_cpu, scales):
    """fp32 state dict of the oracle: the fp16 weights with the adapters merged by the ORACLE's arithmetic."""
    from oracle import lora_oracle
    sd = OrderedDict((k, v.float()) for k, v in sdxl["sd16"].items())
    if adapters_cpu:
        merged = lora_oracle.merge_set({k: sdxl["sd16"][k] for k in sdxl["keys"]}, adapters_cpu, scales)
        for k, v in merged.items():
            sd[k] = v.float()
    return sd


def test_fp16_merge_722_layer_table_every_layer_against_oracle(sdxl):
    from katz_b200 import ops
    from oracle import lora_oracle
    unet, merger, keys = sdxl["unet"], sdxl["merger"], sdxl["keys"]
    targets = unet.lora_targets(keys)
    ad = _make_lora(targets, 64, 100)
    merger.merge(ad, 1.0)
    torch.cuda.synchronize()
    worst, worst_frac = 0.0, 0.0
    for k in keys:
        up, down = ad[k]
        ref = lora_oracle.merge_katz(sdxl["sd16"][k], up.cpu(), down.cpu(), 1.0)
        d = (targets[k].cpu().float() - ref.float()).abs()
        lim = 2 ** -9 * float(ref.float().abs().max())
        frac = float((d > 0).float().mean())
        # same rounding sequence as the reference; fp32 accumulation order may move a product across a rounding boundary
        assert float(d.max()) <= lim and frac < 0.02, (k, float(d.max()), lim, frac)
        worst, worst_frac = max(worst, float(d.max()) / lim), max(worst_frac, frac)
    print("fp16 merge, 722 layers: worst error %.2f of the bound, at most %.3f%% of a layer's elements differ" % (worst, 100 * worst_frac))
    merger.restore()
    torch.cuda.synchronize()
    for k in keys:
        assert torch.equal(targets[k].cpu(), sdxl["sd16"][k]), k
    assert ops.tc05_status() == 0


def test_config2_unet_step_with_lora_merged(sdxl):
    """Configuration 2 against the fp32 CPU oracle; the same oracle on the GPU (fp32, TF32 off) must agree with it."""
    from katz_b200 import ops
    from oracle import unet_oracle
    unet, merger, keys = sdxl["unet"], sdxl["merger"], sdxl["keys"]
    dev = unet.device
    sample, ctx, te, ti, _ = sdxl["inputs"]
    ad = _make_lora(unet.lora_targets(keys), 64, 100)
    merger.merge(ad, 1.0)
    unet.invalidate_caches()
    osd = _oracle_weights(sdxl, [_cpu(ad)], [1.0])
    with torch.no_grad():
        ref = unet_oracle.unet_step(osd, CFG, sample.float(), 500.0, ctx.float(), te.float(), ti.float())
    added = {"text_embeds": te.to(dev), "time_ids": ti.to(dev)}
    out = unet(sample.to(dev), torch.tensor([500.0], device=dev), encoder_hidden_states=ctx.to(dev), added_cond_kwargs=added)[0]
    torch.cuda.synchronize()
    err, rel = _maxabs(out, ref), _rel_l2(out, ref)
    print("configuration 2: max-abs %.3e rel-l2 %.3e (|ref| max %.2f)" % (err, rel, float(ref.abs().max())))
    assert out.shape == (B, 4, HW, HW) and out.dtype == torch.float16
    assert err <= 1e-2 and rel <= 2e-3, (err, rel)
    assert ops.tc05_status() == 0
    # the CUDA-graph replay the benchmark times gives the same bits as the eager step
    unet.use_cuda_graph = True
    try:
        out_g = unet(sample.to(dev), torch.tensor([500.0], device=dev), encoder_hidden_states=ctx.to(dev), added_cond_kwargs=added)[0]
        out_g2 = unet(sample.to(dev), torch.tensor([500.0], device=dev), encoder_hidden_states=ctx.to(dev), added_cond_kwargs=added)[0]
        torch.cuda.synchronize()
        assert torch.equal(out_g, out) and torch.equal(out_g2, out)
    finally:
        unet.use_cuda_graph = False
        unet._graphs.clear()
    # oracle on the GPU in strict fp32 == oracle on the CPU (justifies its use where the CPU would take minutes)
    with torch.no_grad(), _strict_fp32():
        gsd = OrderedDict((k, v.to(dev)) for k, v in osd.items())
        ref_g = unet_oracle.unet_step(gsd, CFG, sample.float().to(dev), 500.0, ctx.float().to(dev), te.float().to(dev),
                                      ti.float().to(dev))
        del gsd
    assert _rel_l2(ref_g, ref) <= 2e-4, _rel_l2(ref_g, ref)
    merger.restore()
    unet.invalidate_caches()


def test_config3_unet_step_with_one_controlnet(sdxl):
    from katz_b200 import ops
    from katz_b200.unet import KatzControlNet
    from oracle import unet_oracle
    unet, merger, keys = sdxl["unet"], sdxl["merger"], sdxl["keys"]
    dev = unet.device
    sample, ctx, te, ti, cond = sdxl["inputs"]
    ad = _make_lora(unet.lora_targets(keys), 64, 100)
    merger.merge(ad, 1.0)
    unet.invalidate_caches()
    cn_sd = init_state_dict(controlnet_param_shapes(CFG), seed=1, dtype=torch.float16, device=dev, generator_device=dev)
    cn = KatzControlNet(CFG, dev, cn_sd)
    cn32 = OrderedDict((k, v.float().cpu()) for k, v in cn_sd.items())
    del cn_sd
    osd = _oracle_weights(sdxl, [_cpu(ad)], [1.0])
    with torch.no_grad():
        rdown, rmid = unet_oracle.controlnet_step(cn32, CFG, sample.float(), 500.0, ctx.float(), cond.float(), te.float(),
                                                  ti.float(), 0.5)
        umid, emb, res = unet_oracle.unet_down_forward(osd, CFG, sample.float(), 500.0, ctx.float(), te.float(), ti.float())
        ref = unet_oracle.unet_up_forward(osd, CFG, umid, emb, res, ctx.float(), rdown, rmid)
        ref_plain = unet_oracle.unet_up_forward(osd, CFG, umid, emb, res, ctx.float())
    added = {"text_embeds": te.to(dev), "time_ids": ti.to(dev)}
    t = torch.tensor([500.0], device=dev)
    down, mid = cn(sample.to(dev), t, encoder_hidden_states=ctx.to(dev), controlnet_cond=cond.to(dev), conditioning_scale=0.5,
                   added_cond_kwargs=added)
    assert len(down) == 9
    for i, (d, r) in enumerate(zip(down, rdown)):
        assert d.shape == r.shape
        assert _rel_l2(d, r) <= 2e-3, (i, _rel_l2(d, r))
    assert _rel_l2(mid, rmid) <= 2e-3
    out = unet(sample.to(dev), t, encoder_hidden_states=ctx.to(dev), added_cond_kwargs=added,
               down_block_additional_residuals=down, mid_block_additional_residual=mid)[0]
    torch.cuda.synchronize()
    err, rel = _maxabs(out, ref), _rel_l2(out, ref)
    print("configuration 3: max-abs %.3e rel-l2 %.3e; residuals move the prediction by rel-l2 %.3e" % (err, rel, _rel_l2(ref, ref_plain)))
    assert err <= 1e-2 and rel <= 2e-3, (err, rel)
    assert _rel_l2(ref, ref_plain) > 1e-2          # the residuals are not a no-op (random zero-convs)
    assert ops.tc05_status() == 0
    merger.restore()
    unet.invalidate_caches()


def test_config4_short_three_controlnets_two_loras(sdxl):
    """Four Euler steps of the 50-step schedule, CFG 5.0, three ControlNets summed at 0.5 / 0.5 / 0.3, LoRAs of rank 64 and
    32 (alpha = rank) merged as one pass; final latent against the oracle loop run in strict fp32 on the GPU."""
    from katz_b200 import ops
    from katz_b200.pipeline import KatzDenoiser
    from katz_b200.scheduler import EulerSchedule
    from katz_b200.unet import KatzControlNet
    from oracle import unet_oracle
    unet, merger, keys = sdxl["unet"], sdxl["merger"], sdxl["keys"]
    dev = unet.device
    _, ctx, te, ti, cond = sdxl["inputs"]
    targets = unet.lora_targets(keys)
    ad64, ad32 = _make_lora(targets, 64, 100), _make_lora(targets, 32, 101)
    merger.merge([ad64, ad32], [1.0, 1.0])
    unet.invalidate_caches()
    nets, nets32 = [], []
    for s in (0, 1, 2):
        cn_sd = init_state_dict(controlnet_param_shapes(CFG), seed=10 + s, dtype=torch.float16, device=dev, generator_device=dev)
        nets.append(KatzControlNet(CFG, dev, cn_sd))
        nets32.append(OrderedDict((k, v.float()) for k, v in cn_sd.items()))
        del cn_sd
    scales = [0.5, 0.5, 0.3]
    steps = 4
    sched = EulerSchedule()
    den = KatzDenoiser(unet, HW, HW, controlnets=nets, conditioning_scales=scales, combine="sum", guidance_scale=5.0,
                       schedule=sched)
    # the first four steps of the 50-step schedule
    sched.set_timesteps(50)
    lat0 = den.prepare_latents(seed=5)
    out = _denoise_first_steps(den, lat0.clone(), ctx.to(dev), te.to(dev), ti.to(dev), cond.to(dev), steps)
    torch.cuda.synchronize()
    assert ops.tc05_status() == 0
    osd = _oracle_weights(sdxl, [_cpu(ad64), _cpu(ad32)], [1.0, 1.0])
    with torch.no_grad(), _strict_fp32():
        gsd = OrderedDict((k, v.to(dev)) for k, v in osd.items())
        del osd
        ref = _oracle_first_steps(gsd, nets32, lat0.clone(), ctx.to(dev), te.to(dev), ti.to(dev), cond.to(dev), steps, scales)
    rel = _rel_l2(out, ref)
    print("configuration 4 (first %d of 50 steps): final-latent rel-l2 %.3e" % (steps, rel))
    assert rel <= 2e-3, rel
    merger.restore()
    unet.invalidate_caches()


def _denoise_first_steps(den, latents, ctx, te, ti, cond, steps):
    """KatzDenoiser.denoise restricted to the first `steps` steps of the schedule already set."""
    from katz_b200 import ops
    st = den.step.static
    st["encoder_hidden_states"].copy_(ctx)
    st["text_embeds"].copy_(te)
    st["time_ids"].copy_(ti)
    st["controlnet_cond"].copy_(cond)
    den.step.refresh_hoisted()
    sig, ts = den.schedule.sigmas, den.schedule.timesteps
    for i in range(steps):
        ops.euler_scale_input(latents, float(sig[i]), copies=2, out=st["sample"])
        st["timestep"].fill_(float(ts[i]))
        den.step.graph.replay()
        o = den.step.out
        ops.euler_cfg_step(latents, o[0:1], o[1:2], den.guidance_scale, float(sig[i]), float(sig[i + 1]))
    return latents


def _oracle_first_steps(sd, cn_sds, latents, ctx, te, ti, cond, steps, scales):
    """oracle.unet_oracle.denoise_loop's body over the first `steps` steps of the 50-step schedule."""
    from oracle import unet_oracle as uo
    ts, sig, _ = uo.euler_sigmas(50)
    for i in range(steps):
        x = uo.euler_scale_model_input(latents, sig[i])
        x2 = torch.cat([x, x]).float()
        down = mid = None
        for cn_sd, s in zip(cn_sds, scales):
            d, m = uo.controlnet_step(cn_sd, CFG, x2, float(ts[i]), ctx.float(), cond.float(), te.float(), ti.float(), s)
            down = d if down is None else [a + b for a, b in zip(down, d)]
            mid = m if mid is None else mid + m
        eps = uo.unet_step(sd, CFG, x2, float(ts[i]), ctx.float(), te.float(), ti.float(), down, mid).to(latents.dtype)
        latents = uo.euler_step(latents, uo.cfg_combine(eps[0:1], eps[1:2], 5.0), sig[i], sig[i + 1])
    return latents


def test_config1_fp32_merge_restore_700_layers(cuda_device):
    """Configuration 1 at size: 700 linears (2.18 G elements, fp32), rank 64, alpha 64 -> scale 1. Merge against the
    oracle layer by layer, restore bit-exactly, then the subtractive round trip with its mismatch count."""
    from katz_b200.lora import LoraMerger
    from oracle import lora_oracle
    dev = cuda_device
    shapes = unet_param_shapes(CFG)
    keys = lora_target_keys(CFG, include_proj=False)
    assert len(keys) == 700 and sum(shapes[k][0] * shapes[k][1] for k in keys) == 2183987200
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    W = OrderedDict((k, torch.randn(shapes[k], generator=g, device=dev) * 0.02) for k in keys)
    W0 = OrderedDict((k, w.cpu()) for k, w in W.items())
    ad = _make_lora(W, 64, 0, dtype=torch.float32)
    merger = LoraMerger(W)
    merger.merge(ad, 1.0)
    torch.cuda.synchronize()
    worst = 0.0
    for k in keys:
        up, down = ad[k]
        ref = lora_oracle.merge_katz(W0[k], up.cpu(), down.cpu(), 1.0)
        delta = float((ref - W0[k]).abs().max())
        err = float((W[k].cpu() - ref).abs().max())
        assert err <= 1e-5 * delta + 4e-9, (k, err, delta)
        worst = max(worst, err / delta)
    merger.restore()
    torch.cuda.synchronize()
    bad = [k for k in keys if not torch.equal(W[k].cpu(), W0[k])]
    assert not bad, bad[:3]
    # W += BA; W -= BA (LoRACompatibleLinear._fuse_lora/_unfuse_lora arithmetic): floating point does not undo it
    merger.merge_in_place(ad, 1.0)
    merger.unmerge_in_place(ad, 1.0)
    torch.cuda.synchronize()
    mism, total, maxd = 0, 0, 0.0
    for k in keys:
        d = (W[k].cpu() - W0[k]).abs()
        mism += int((d > 0).sum())
        total += d.numel()
        maxd = max(maxd, float(d.max()))
    # the oracle's own count on one layer of each shape class, for the record
    o_mism, o_total = 0, 0
    for k in keys[:10]:
        up, down = ad[k]
        f = lora_oracle.fuse_lora_vendored(W0[k], up.cpu(), down.cpu(), 64.0, 64)
        u = lora_oracle.unfuse_lora_vendored(f, up.cpu(), down.cpu(), 64.0, 64)
        o_mism += int((u != W0[k]).sum())
        o_total += u.numel()
    print("configuration 1: merge worst error %.2e of the delta; restore bit-exact on 700 layers; +/- round trip leaves "
          "%d of %d elements changed (%.2f%%, max %.2e); the oracle's fp32 +/- leaves %.2f%% on the first 10 layers"
          % (worst, mism, total, 100.0 * mism / total, maxd, 100.0 * o_mism / o_total))
    assert maxd < 1e-7 and 0 < mism < total


def test_in_place_fuse_unfuse_against_vendored_oracle(cuda_device):
    """merge_in_place / unmerge_in_place against LoRACompatibleLinear._fuse_lora / _unfuse_lora (models/lora.py:403-449)
    as restated by the oracle, fp32 weights, alpha/rank folded into the scale."""
    from katz_b200.lora import LoraMerger
    from oracle import lora_oracle
    g = torch.Generator().manual_seed(7)
    shapes = [(640, 640), (1280, 2048), (5120, 640), (1280, 5120)]
    W = OrderedDict(("l%d" % i, torch.randn(s, generator=g) * 0.02) for i, s in enumerate(shapes))
    ad = OrderedDict((k, (torch.randn(w.shape[0], 16, generator=g) * 0.01, torch.randn(16, w.shape[1], generator=g) / 16)) for k, w in W.items())
    Wg = OrderedDict((k, w.cuda()) for k, w in W.items())
    adg = OrderedDict((k, (u.cuda(), d.cuda())) for k, (u, d) in ad.items())
    alpha, rank, lora_scale = 8.0, 16, 0.7
    m = LoraMerger(Wg, keep_pristine=False)
    m.merge_in_place(adg, lora_scale * alpha / rank)
    torch.cuda.synchronize()
    fused = {}
    for k in W:
        fused[k] = lora_oracle.fuse_lora_vendored(W[k], ad[k][0], ad[k][1], alpha, rank, lora_scale)
        delta = float((fused[k] - W[k]).abs().max())
        assert float((Wg[k].cpu() - fused[k]).abs().max()) <= 1e-5 * delta + 4e-9, k
    m.unmerge_in_place(adg, lora_scale * alpha / rank)
    torch.cuda.synchronize()
    n_gpu = n_ref = total = 0
    for k in W:
        un = lora_oracle.unfuse_lora_vendored(fused[k], ad[k][0], ad[k][1], alpha, rank, lora_scale)
        delta = float((fused[k] - W[k]).abs().max())
        assert float((Wg[k].cpu() - un).abs().max()) <= 1e-5 * delta + 4e-9, k
        n_gpu += int((Wg[k].cpu() != W[k]).sum())
        n_ref += int((un != W[k]).sum())
        total += un.numel()
    print("in-place +/-: %d of %d elements not restored on the GPU, %d in the vendored fp32 arithmetic" % (n_gpu, total, n_ref))
    assert n_gpu > 0 and n_ref > 0      # neither restores W bit-exactly: copy restore is what ships
