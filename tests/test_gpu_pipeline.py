"""GPU: the denoise loop (scale -> ControlNets -> UNet -> CFG -> Euler) and the LoRA-switching request stream on the
tiny configuration against the CPU oracle loop. Tolerance: relative L2 of the final latent <= 2e-3 per step count used
here (the baseline's bound for the final latent)."""
from collections import OrderedDict

import pytest
import torch

from katz_b200.params import (TINY_UNET_CONFIG, controlnet_param_shapes, init_state_dict, lora_target_keys,
                              unet_param_shapes)
from tests.golden.make_golden import tiny_inputs

pytestmark = pytest.mark.gpu


def _f32(sd):
    return OrderedDict((k, v.float()) for k, v in sd.items())


def _rel_l2(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm())


def test_denoise_loop_with_two_controlnets(cuda_device):
    from katz_b200.pipeline import KatzDenoiser
    from katz_b200.unet import KatzControlNet, KatzUNet
    from oracle import unet_oracle
    cfg = TINY_UNET_CONFIG
    sd = init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16)
    cns = [init_state_dict(controlnet_param_shapes(cfg), seed=s, dtype=torch.float16) for s in (2, 3)]
    unet = KatzUNet(cfg, cuda_device, sd)
    nets = [KatzControlNet(cfg, cuda_device, c) for c in cns]
    _, ctx, te, ti, cond = (t.half() for t in tiny_inputs(cfg))
    steps = 4
    den = KatzDenoiser(unet, 16, 16, controlnets=nets, conditioning_scales=[0.5, 0.3], combine="sum", guidance_scale=5.0)
    den.schedule.set_timesteps(steps)
    lat0 = den.prepare_latents(seed=5)
    ref = unet_oracle.denoise_loop(_f32(sd), cfg, lat0.cpu().clone(), ctx, te, ti, steps, 5.0, [_f32(c) for c in cns],
                                   cond, [0.5, 0.3], "sum")
    out = den.denoise(lat0.clone(), ctx.cuda(), te.cuda(), ti.cuda(), cond.cuda(), num_inference_steps=steps)
    assert out.dtype == torch.float16 and _rel_l2(out, ref) <= 2e-3, _rel_l2(out, ref)
    # the mean combine of the service path differs from the sum
    den2 = KatzDenoiser(unet, 16, 16, controlnets=nets, conditioning_scales=[0.5, 0.5], combine="mean")
    ref2 = unet_oracle.denoise_loop(_f32(sd), cfg, lat0.cpu().clone(), ctx, te, ti, 2, 5.0, [_f32(c) for c in cns], cond,
                                    [0.5, 0.5], "mean")
    out2 = den2.denoise(lat0.clone(), ctx.cuda(), te.cuda(), ti.cuda(), cond.cuda(), num_inference_steps=2)
    assert _rel_l2(out2, ref2) <= 2e-3


def test_request_stream_switches_loras(cuda_device):
    from katz_b200.lora import LoraMerger
    from katz_b200.pipeline import KatzDenoiser, LoraRequestStream
    from katz_b200.unet import KatzUNet
    cfg = TINY_UNET_CONFIG
    sd = init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16)
    unet = KatzUNet(cfg, cuda_device, sd)
    keys = lora_target_keys(cfg, include_proj=True)
    targets = unet.lora_targets(keys)
    merger = LoraMerger(targets)
    g = torch.Generator().manual_seed(1)
    pool = []
    for _ in range(3):
        pool.append(OrderedDict((k, ((torch.randn(w.shape[0], 16, generator=g) * 0.02).half().cuda(),
                                     (torch.randn(16, w.shape[1], generator=g) / 16).half().cuda())) for k, w in targets.items()))
    _, ctx, te, ti, _ = (t.half().cuda() for t in tiny_inputs(cfg))
    den = KatzDenoiser(unet, 16, 16)
    stream = LoraRequestStream(den, merger, pool)
    inputs = lambda i: dict(prompt_embeds=ctx, text_embeds=te, time_ids=ti)   # noqa: E731
    res = stream.run([0, 1, 0, 0, 2], inputs, num_inference_steps=2, seed=0)
    assert len(res) == 5 and all(ms > 0 for _, ms in res)
    lat = [r[0] for r in res]
    # same adapter + same seed-independent inputs: request 0 and 2 differ only by their initial noise
    again = stream.run([0], inputs, num_inference_steps=2, seed=0)[0][0]
    assert torch.equal(again, lat[0])          # LoRA 0 re-merged after 1 and 2: bit-identical request
    assert not torch.equal(lat[0], lat[1])
    merger.restore()
    for k, w in targets.items():
        assert torch.equal(w.cpu(), sd[k])


def test_cached_stream_loads_adapters_from_pinned_host_copies(cuda_device):
    """Requests name adapter ids; the adapters live in pinned host memory and reach the GPU through the cache: the
    results equal those of the stream whose whole pool is resident, and the loads are what the policy predicts."""
    from katz_b200.adapter_cache import CachedLoraStream, replay_loads
    from katz_b200.lora import LoraMerger
    from katz_b200.pipeline import KatzDenoiser, LoraRequestStream
    from katz_b200.unet import KatzUNet
    cfg = TINY_UNET_CONFIG
    sd = init_state_dict(unet_param_shapes(cfg), seed=0, dtype=torch.float16)
    unet = KatzUNet(cfg, cuda_device, sd)
    targets = unet.lora_targets(lora_target_keys(cfg, include_proj=True))
    merger = LoraMerger(targets, on_change=unet.invalidate_caches)
    g = torch.Generator().manual_seed(4)
    host = []
    for _ in range(4):
        host.append(OrderedDict((k, ((torch.randn(w.shape[0], 8, generator=g) * 0.02).half().pin_memory(),
                                     (torch.randn(8, w.shape[1], generator=g) / 8).half().pin_memory())) for k, w in targets.items()))
    loads = []

    def loader(i):
        loads.append(i)
        return OrderedDict((k, (u.to(cuda_device, non_blocking=True), d.to(cuda_device, non_blocking=True))) for k, (u, d) in host[i].items())

    _, ctx, te, ti, _ = (t.half().cuda() for t in tiny_inputs(cfg))
    den = KatzDenoiser(unet, 16, 16)
    inputs = lambda i: dict(prompt_embeds=ctx, text_embeds=te, time_ids=ti)   # noqa: E731
    ids = [0, 1, 0, 2, 3, 0, 1, 1]
    cached = CachedLoraStream(den, merger, loader, capacity=2, policy="LRU")
    got = cached.run([(i,) for i in ids], inputs, num_inference_steps=2, seed=0)
    # consecutive equal requests do not look the adapter up again
    lookups = [i for n, i in enumerate(ids) if n == 0 or ids[n - 1] != i]
    assert loads == [0, 1, 2, 3, 0, 1] and cached.cache.loads == replay_loads(lookups, 2, "LRU")
    st = cached.cache.stats()
    assert st["resident"] == 2 and st["hits"] == 1 and st["bytes_loaded"] == 6 * st["resident_bytes"] // 2
    resident = LoraRequestStream(den, merger, [loader(i) for i in range(4)])
    want = resident.run(ids, inputs, num_inference_steps=2, seed=0)
    for (a, _), (b, _) in zip(got, want):
        assert torch.equal(a, b)
    # a request with no adapter runs on the pristine weights; two adapters in one request are summed by the merge
    more = cached.run([(), (2, 3)], inputs, num_inference_steps=2, seed=0)
    merger.restore()
    plain = den.denoise(den.prepare_latents(seed=0), num_inference_steps=2, **inputs(0))
    assert torch.equal(more[0][0], plain)
    merger.merge([loader(2), loader(3)], [1.0, 1.0])
    both = den.denoise(den.prepare_latents(seed=1), num_inference_steps=2, **inputs(0))
    assert torch.equal(more[1][0], both)
    merger.restore()
