"""Flow-matching Euler scheduler.

Numerics of diffusers' ``FlowMatchEulerDiscreteScheduler`` (imported, not re-implemented,
by the reference: vllm_omni/diffusion/models/qwen_image/pipeline_qwen_image.py:19-22):
sigma schedule with static or resolution-dependent ("dynamic") shift, optional terminal
stretch, and the update x_{i+1} = x_i + (sigma_{i+1} - sigma_i) * v.  The per-step update
itself runs inside the fused CFG + Euler kernel; this class owns the schedule.
"""
from __future__ import annotations

import math

import numpy as np
import torch


def calculate_shift(image_seq_len, base_seq_len=256, max_seq_len=4096, base_shift=0.5, max_shift=1.15):
    m = (max_shift - base_shift) / (max_seq_len - base_seq_len)
    b = base_shift - m * base_seq_len
    return image_seq_len * m + b


class FlowMatchEulerDiscreteScheduler:
    order = 1

    def __init__(self, num_train_timesteps=1000, shift=1.0, use_dynamic_shifting=False, base_shift=0.5,
                 max_shift=1.15, base_image_seq_len=256, max_image_seq_len=4096, shift_terminal=None,
                 time_shift_type="exponential", invert_sigmas=False, **_):
        self.config = dict(num_train_timesteps=num_train_timesteps, shift=shift,
                           use_dynamic_shifting=use_dynamic_shifting, base_shift=base_shift, max_shift=max_shift,
                           base_image_seq_len=base_image_seq_len, max_image_seq_len=max_image_seq_len,
                           shift_terminal=shift_terminal, time_shift_type=time_shift_type)
        self.sigmas = None
        self.timesteps = None
        self._step_index = None

    @classmethod
    def from_config(cls, cfg: dict):
        return cls(**cfg)

    def time_shift(self, mu: float, sigma: float, t: np.ndarray) -> np.ndarray:
        if self.config["time_shift_type"] == "linear":
            return mu / (mu + (1 / t - 1) ** sigma)
        return math.exp(mu) / (math.exp(mu) + (1 / t - 1) ** sigma)

    def stretch_shift_to_terminal(self, t: np.ndarray) -> np.ndarray:
        one_minus = 1 - t
        scale = one_minus[-1] / (1 - self.config["shift_terminal"])
        return 1 - one_minus / scale

    def set_timesteps(self, num_inference_steps=None, device=None, sigmas=None, mu=None, **_):
        n_train = self.config["num_train_timesteps"]
        if sigmas is None:
            ts = np.linspace(n_train, 1, num_inference_steps)
            sigmas = ts / n_train
        sigmas = np.asarray(sigmas, dtype=np.float64)
        if self.config["use_dynamic_shifting"]:
            if mu is None:
                raise ValueError("mu is required with use_dynamic_shifting")
            sigmas = self.time_shift(mu, 1.0, sigmas)
        else:
            s = self.config["shift"]
            sigmas = s * sigmas / (1 + (s - 1) * sigmas)
        if self.config["shift_terminal"]:
            sigmas = self.stretch_shift_to_terminal(sigmas)
        self.timesteps = torch.tensor(sigmas * n_train, dtype=torch.float32, device=device)
        self.sigmas = np.concatenate([sigmas, [0.0]]).astype(np.float64)
        self.num_inference_steps = len(sigmas)
        self._step_index = 0
        return self.timesteps

    def dt(self, i: int) -> float:
        return float(self.sigmas[i + 1] - self.sigmas[i])

    def step(self, model_output: torch.Tensor, timestep, sample: torch.Tensor, step_index: int | None = None):
        i = self._step_index if step_index is None else step_index
        prev = sample.float() + self.dt(i) * model_output.float()
        self._step_index = i + 1
        return prev.to(sample.dtype)

    def scale_noise(self, sample, sigma: float, noise):
        return sigma * noise + (1.0 - sigma) * sample
