"""Stochastic DPM-Solver++ (2M, SDE variant) on an EDM-style noise scale, the sampler of Stable Audio
Open (diffusers' ``CosineDPMSolverMultistepScheduler``, which the reference instantiates from the
checkpoint's ``scheduler/`` folder: vllm_omni/diffusion/models/stable_audio/pipeline_stable_audio.py).

Noise levels run exponentially from ``sigma_max`` down to ``sigma_min`` and end at 0.  The network
sees ``x / sqrt(sigma^2 + sigma_data^2)`` and the time ``atan(sigma) * 2 / pi``; its v-prediction is
turned into a clean-sample estimate ``x0 = c_skip x + c_out v`` with ``c_skip = sd^2 / (s^2 + sd^2)``,
``c_out = -s sd / sqrt(s^2 + sd^2)``.  With lambda = -log(sigma) and h the lambda step, one update is

    x' = (s'/s) e^{-h} x + (1 - e^{-2h}) D0 [+ 1/2 (1 - e^{-2h}) D1] + s' sqrt(1 - e^{-2h}) z

where D0 is the current estimate, D1 the scaled difference to the previous one (second order, not on
the first and the last step) and z fresh standard-normal noise.  The reference draws z from a
Brownian tree; on a fixed step grid independent Gaussian draws have the same distribution.
"""
from __future__ import annotations

import math

import torch


class CosineDPMSolverMultistepScheduler:
    order = 1

    def __init__(self, sigma_min: float = 0.3, sigma_max: float = 500.0, sigma_data: float = 1.0,
                 sigma_schedule: str = "exponential", num_train_timesteps: int = 1000, solver_order: int = 2,
                 prediction_type: str = "v_prediction", rho: float = 7.0, solver_type: str = "midpoint",
                 lower_order_final: bool = True, euler_at_final: bool = False, final_sigmas_type: str = "zero", **_):
        self.config = dict(sigma_min=sigma_min, sigma_max=sigma_max, sigma_data=sigma_data, sigma_schedule=sigma_schedule,
                           num_train_timesteps=num_train_timesteps, solver_order=solver_order, prediction_type=prediction_type,
                           rho=rho, solver_type=solver_type, lower_order_final=lower_order_final, euler_at_final=euler_at_final,
                           final_sigmas_type=final_sigmas_type)
        self.sigmas = self.timesteps = None
        self._outputs: list = []
        self._step = 0

    @classmethod
    def from_config(cls, cfg: dict):
        return cls(**cfg)

    @property
    def init_noise_sigma(self) -> float:
        return (self.config["sigma_max"] ** 2 + 1) ** 0.5

    def _sigmas(self, n: int) -> torch.Tensor:
        c = self.config
        if c["sigma_schedule"] == "karras":
            ramp = torch.linspace(0, 1, n, dtype=torch.float64)
            lo, hi = c["sigma_min"] ** (1 / c["rho"]), c["sigma_max"] ** (1 / c["rho"])
            return (hi + ramp * (lo - hi)) ** c["rho"]
        return torch.linspace(math.log(c["sigma_min"]), math.log(c["sigma_max"]), n, dtype=torch.float64).exp().flip(0)

    def set_timesteps(self, num_inference_steps: int, device=None) -> torch.Tensor:
        s = self._sigmas(num_inference_steps)
        last = self.config["sigma_min"] if self.config["final_sigmas_type"] == "sigma_min" else 0.0
        self.sigmas = torch.cat([s, torch.tensor([last], dtype=torch.float64)])
        self.timesteps = (torch.atan(s) / math.pi * 2).float().to(device)
        self._outputs, self._step = [], 0
        return self.timesteps

    # ---- preconditioning
    def scale_model_input(self, sample: torch.Tensor) -> torch.Tensor:
        s = float(self.sigmas[self._step])
        return sample * (1.0 / math.sqrt(s * s + self.config["sigma_data"] ** 2))

    def denoised(self, sample: torch.Tensor, model_output: torch.Tensor) -> torch.Tensor:
        s, sd = float(self.sigmas[self._step]), self.config["sigma_data"]
        c_skip = sd * sd / (s * s + sd * sd)
        c_out = s * sd / math.sqrt(s * s + sd * sd)
        if self.config["prediction_type"] == "v_prediction":
            c_out = -c_out
        return c_skip * sample + c_out * model_output

    # ---- update
    def step(self, model_output: torch.Tensor, sample: torch.Tensor, generator=None, noise: torch.Tensor | None = None):
        """One update from sigma[i] to sigma[i + 1]; ``model_output`` is the network's raw prediction on
        the scaled input.  Returns the next sample (fp32)."""
        c = self.config
        i, n = self._step, len(self.timesteps)
        sample = sample.float()
        x0 = self.denoised(sample, model_output.float())
        self._outputs = (self._outputs + [x0])[-c["solver_order"]:]
        s_t, s_0 = float(self.sigmas[i + 1]), float(self.sigmas[i])
        final_first_order = i == n - 1 and (c["euler_at_final"] or (c["lower_order_final"] and n < 15)
                                            or c["final_sigmas_type"] == "zero")
        if s_t == 0.0:                                   # h = inf: the update lands on the estimate itself
            nxt = x0
        else:
            if noise is None:
                noise = torch.randn(sample.shape, generator=generator, device=generator.device if generator is not None
                                    else sample.device).to(sample.device)
            h = math.log(s_0) - math.log(s_t)
            e1, e2 = math.exp(-h), 1.0 - math.exp(-2.0 * h)
            nxt = (s_t / s_0 * e1) * sample + e2 * x0 + s_t * math.sqrt(e2) * noise.float()
            if c["solver_order"] >= 2 and len(self._outputs) >= 2 and not final_first_order:
                h0 = math.log(float(self.sigmas[i - 1])) - math.log(s_0)
                d1 = (x0 - self._outputs[-2]) * (h / h0)
                if c["solver_type"] == "heun":
                    nxt = nxt + (e2 / (-2.0 * h) + 1.0) * d1
                else:
                    nxt = nxt + 0.5 * e2 * d1
        self._step += 1
        return nxt
