"""Flow-matching Euler scheduler with the call surface the reference's denoising loop uses
(`set_timesteps`, `set_begin_index`, `step(..., return_dict=False)`), restated from the published
algorithm: sigmas shifted by exp(mu), sample <- sample + (sigma_next - sigma) * velocity in fp32."""
import math

import numpy as np
import torch


class FlowMatchEulerDiscreteScheduler:
    order = 1

    def __init__(self, num_train_timesteps=1000, shift=1.0, use_dynamic_shifting=True, base_shift=0.5, max_shift=0.9,
                 base_image_seq_len=256, max_image_seq_len=8192, shift_terminal=0.02, **kwargs):
        self.num_train_timesteps = num_train_timesteps
        self.shift = shift
        self.use_dynamic_shifting = use_dynamic_shifting
        self.shift_terminal = shift_terminal
        self.config = type("Cfg", (), dict(base_shift=base_shift, max_shift=max_shift,
                                           base_image_seq_len=base_image_seq_len,
                                           max_image_seq_len=max_image_seq_len,
                                           num_train_timesteps=num_train_timesteps))()
        self._step_index = None
        self._begin_index = None
        self.timesteps = None
        self.sigmas = None

    def set_begin_index(self, begin_index=0):
        self._begin_index = begin_index

    def set_timesteps(self, num_inference_steps=None, device=None, sigmas=None, mu=None):
        if sigmas is None:
            sigmas = np.linspace(1.0, 1.0 / num_inference_steps, num_inference_steps)
        sigmas = np.asarray(sigmas, dtype=np.float64)
        if self.use_dynamic_shifting:
            sigmas = math.exp(mu) / (math.exp(mu) + (1.0 / sigmas - 1.0))
        else:
            sigmas = self.shift * sigmas / (1 + (self.shift - 1) * sigmas)
        if self.shift_terminal:
            one_minus = 1.0 - sigmas
            sigmas = 1.0 - one_minus / (one_minus[-1] / (1.0 - self.shift_terminal))
        s = torch.tensor(sigmas, dtype=torch.float32, device=device)
        self.timesteps = s * self.num_train_timesteps
        self.sigmas = torch.cat([s, torch.zeros(1, device=device)])
        self._sigmas_host = self.sigmas.tolist()
        self._step_index = None

    def step(self, model_output, timestep, sample, return_dict=True, **kwargs):
        if self._step_index is None:
            self._step_index = self._begin_index or 0
        i = self._step_index
        dt = self._sigmas_host[i + 1] - self._sigmas_host[i]
        prev = (sample.to(torch.float32) + dt * model_output.to(torch.float32)).to(model_output.dtype)
        self._step_index += 1
        return (prev,)
