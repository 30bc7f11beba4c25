"""Euler-discrete sampling schedule for the denoise loop (host side; the per-step arithmetic runs in the
`katz_euler_*` kernels).

Mirrors EulerDiscreteScheduler.__init__ / set_timesteps / init_noise_sigma
(diffusers/schedulers/scheduling_euler_discrete.py:177-255,300-362) for the SDXL configuration
(scaled_linear betas 0.00085 -> 0.012, 1000 train steps, `leading` spacing, steps_offset 1, linear sigma
interpolation); `linear` betas and `linspace` spacing are kept because the reference's own known-answer tests use them.
"""
import numpy as np
import torch


class EulerSchedule:
    def __init__(self, num_train_timesteps=1000, beta_start=0.00085, beta_end=0.012, beta_schedule="scaled_linear",
                 timestep_spacing="leading", steps_offset=1):
        if beta_schedule == "linear":
            betas = torch.linspace(beta_start, beta_end, num_train_timesteps, dtype=torch.float32)
        elif beta_schedule == "scaled_linear":
            betas = torch.linspace(beta_start ** 0.5, beta_end ** 0.5, num_train_timesteps, dtype=torch.float32) ** 2
        else:
            raise NotImplementedError("%s is not implemented for EulerSchedule" % beta_schedule)
        if timestep_spacing not in ("linspace", "leading"):
            raise ValueError("%s is not supported; choose 'linspace' or 'leading'" % timestep_spacing)
        self.num_train_timesteps = num_train_timesteps
        self.timestep_spacing = timestep_spacing
        self.steps_offset = steps_offset
        self.alphas_cumprod = torch.cumprod(1.0 - betas, dim=0)
        self.timesteps = None
        self.sigmas = None

    def set_timesteps(self, num_inference_steps):
        n = self.num_train_timesteps
        if self.timestep_spacing == "linspace":
            ts = np.linspace(0, n - 1, num_inference_steps, dtype=np.float32)[::-1].copy()
        else:
            ratio = n // num_inference_steps
            ts = (np.arange(0, num_inference_steps) * ratio).round()[::-1].copy().astype(np.float32)
            ts += self.steps_offset
        sig = (((1 - self.alphas_cumprod) / self.alphas_cumprod) ** 0.5).numpy()
        sig = np.interp(ts, np.arange(0, len(sig)), sig)
        self.sigmas = torch.cat([torch.from_numpy(sig).to(torch.float32), torch.zeros(1)])
        self.timesteps = torch.from_numpy(ts.astype(np.float32))
        return self

    @property
    def init_noise_sigma(self):
        m = self.sigmas.max()
        return float(m if self.timestep_spacing == "linspace" else (m ** 2 + 1) ** 0.5)
