"""The denoise loop around the UNet step, and the request stream that switches LoRAs between requests.

Mirrors the loop of StableDiffusionXLControlNetPipelineKatz.__call__
(diffusers/pipelines/controlnet/pipeline_controlnet_sd_xl_katz.py:1508-1675) for the part that belongs to this path:
per step `scale_model_input` -> ControlNets -> UNet on the CFG batch [uncond, cond] -> guidance combine ->
`EulerDiscreteScheduler.step`. Text encoding, VAE decoding and image I/O stay with the caller. The ControlNets and the
UNet run as ONE CUDA graph (engine.GraphedStep); the two Euler kernels run around it, so a 50-step request is 50 graph
replays and 100 small launches with no host synchronisation.
"""
import torch

from . import ops
from .engine import GraphedStep
from .ops import KatzError
from .scheduler import EulerSchedule


class KatzDenoiser:
    """unet: KatzUNet; controlnets: list of KatzControlNet sharing the UNet's config.

    combine='sum' adds the per-net-scaled residuals (MultiControlNetModel, pipelines/controlnet/multicontrolnet.py:47-73);
    combine='mean' divides the sum by the number of nets (the service path, unet_2d_condition.py:1418-1439)."""

    def __init__(self, unet, height, width, controlnets=(), conditioning_scales=None, combine="sum", guidance_scale=5.0,
                 schedule=None, text_len=77, hoist=False):
        self.unet = unet
        self.guidance_scale = float(guidance_scale)
        self.schedule = schedule or EulerSchedule()
        self.height, self.width = height, width
        self.step = GraphedStep(unet, 2, height, width, text_len=text_len, controlnets=controlnets,
                                conditioning_scales=conditioning_scales, combine=combine, hoist=hoist)

    def prepare_latents(self, generator=None, seed=0):
        """`randn * init_noise_sigma` in fp16 (prepare_latents of the reference pipeline)."""
        if self.schedule.sigmas is None:
            raise KatzError("call schedule.set_timesteps() first")
        g = generator or torch.Generator().manual_seed(seed)
        c = self.unet.cfg["in_channels"]
        lat = torch.randn((1, c, self.height, self.width), generator=g).half()
        return (lat.to(self.unet.device) * self.schedule.init_noise_sigma).half()

    def denoise(self, latents, prompt_embeds, text_embeds, time_ids, controlnet_cond=None, num_inference_steps=50,
                callback=None, check=False):
        """latents: fp16 [1,4,H,W] on the device (modified in place and returned). prompt_embeds [2,77,D], text_embeds
        [2,E], time_ids [2,6] ordered [negative, positive] as the reference concatenates them."""
        sch = self.schedule.set_timesteps(num_inference_steps)
        st = self.step.static
        st["encoder_hidden_states"].copy_(prompt_embeds, non_blocking=True)
        st["text_embeds"].copy_(text_embeds, non_blocking=True)
        st["time_ids"].copy_(time_ids, non_blocking=True)
        if "controlnet_cond" in st:
            if controlnet_cond is None:
                raise KatzError("this denoiser was built with ControlNets: controlnet_cond is required")
            st["controlnet_cond"].copy_(controlnet_cond, non_blocking=True)
        self.step.refresh_hoisted()       # hoist=True: text K/V and conditioning embeddings once per request
        sig, ts = sch.sigmas, sch.timesteps
        n = latents.numel()
        for i in range(num_inference_steps):
            ops.euler_scale_input(latents, float(sig[i]), copies=2, out=st["sample"])
            st["timestep"].fill_(float(ts[i]))
            self.step.graph.replay()
            out = self.step.out                       # [2,4,H,W]: [uncond, cond]
            ops.euler_cfg_step(latents, out[0:1], out[1:2], self.guidance_scale, float(sig[i]), float(sig[i + 1]))
            if callback is not None:
                callback(i, latents)
        assert latents.numel() == n
        if check:
            self.step.check()      # one device synchronisation per request: did any bounded wait give up?
        return latents


class LoraRequestStream:
    """A stream of requests, each naming one adapter from a pool: consecutive requests with different adapters force an
    unmerge/merge between them (configuration 5 of the baseline). With the pristine weights resident, the switch is ONE
    merge pass `W = W0 + s*B*A` regardless of what was merged before."""

    def __init__(self, denoiser, merger, adapters, scale=1.0):
        self.denoiser, self.merger, self.scale = denoiser, merger, scale
        # validated once: a switch then costs one table upload and one merge launch, no per-layer host work
        self.adapters = [merger.register_adapter(a) for a in adapters]
        self.current = None

    def run(self, lora_ids, request_inputs, num_inference_steps=50, seed=0):
        """request_inputs: callable(i) -> dict(prompt_embeds, text_embeds, time_ids, controlnet_cond). Returns the
        list of (final latent, milliseconds) per request, timed with CUDA events."""
        results = []
        self.denoiser.schedule.set_timesteps(num_inference_steps)
        for i, lid in enumerate(lora_ids):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if lid != self.current:
                self.merger.merge(self.adapters[lid], self.scale)
                self.denoiser.unet.invalidate_caches()
                self.current = lid
            lat = self.denoiser.prepare_latents(seed=seed + i)
            lat = self.denoiser.denoise(lat, num_inference_steps=num_inference_steps, **request_inputs(i))
            e1.record()
            results.append((lat.clone(), e0, e1))
        torch.cuda.synchronize()
        self.denoiser.step.check()
        return [(lat, a.elapsed_time(b)) for lat, a, b in results]
