"""UniPC multistep scheduler for flow-matching models (B(h) = expm1(h) "bh2" variant, data
prediction), the numerics of ``FlowUniPCMultistepScheduler``
(vllm_omni/diffusion/models/schedulers/scheduling_flow_unipc_multistep.py:157-741):
``set_timesteps`` with static shift, ``convert_model_output`` (x0 = x - sigma * v), the UniP
predictor and UniC corrector updates, lower-order warm-up and lower-order final steps.
Used by the Wan video pipelines (shift 5.0 for 720p, 3.0 for 480p).
"""
from __future__ import annotations

import math

import numpy as np
import torch


class FlowUniPCMultistepScheduler:
    order = 1

    def __init__(self, num_train_timesteps: int = 1000, solver_order: int = 2, shift: float = 1.0,
                 lower_order_final: bool = True, disable_corrector: tuple = (), final_sigmas_type: str = "zero", **_):
        self.config = dict(num_train_timesteps=num_train_timesteps, solver_order=solver_order, shift=shift,
                           lower_order_final=lower_order_final, final_sigmas_type=final_sigmas_type)
        self.solver_order = solver_order
        self.disable_corrector = set(disable_corrector)
        self.sigmas = None
        self.timesteps = None

    def set_timesteps(self, num_inference_steps: int, device=None, shift: float | None = None, sigmas=None, **_):
        shift = self.config["shift"] if shift is None else shift
        n_train = self.config["num_train_timesteps"]
        if sigmas is None:
            smax, smin = 1.0, 1.0 / n_train
            sigmas = np.linspace(smax, smin, num_inference_steps + 1)[:-1]
        sigmas = np.asarray(sigmas, dtype=np.float64)
        sigmas = shift * sigmas / (1 + (shift - 1) * sigmas)
        self.timesteps = torch.tensor(sigmas * n_train, dtype=torch.float32, device=device)
        self.sigmas = np.concatenate([sigmas, [0.0]])
        self.num_inference_steps = len(sigmas)
        self.model_outputs = [None] * self.solver_order
        self.lower_order_nums = 0
        self.last_sample = None
        self._step_index = 0
        self.this_order = 1
        return self.timesteps

    @staticmethod
    def _alpha_sigma(sigma: float):
        return 1.0 - sigma, sigma

    @staticmethod
    def _lambda(sigma: float) -> float:
        a, s = 1.0 - sigma, sigma
        if s <= 0:
            return math.inf
        if a <= 0:
            return -math.inf
        return math.log(a) - math.log(s)

    def convert_model_output(self, model_output: torch.Tensor, sample: torch.Tensor, step_index: int) -> torch.Tensor:
        return sample.float() - self.sigmas[step_index] * model_output.float()

    def _coeffs(self, h: float, rks: list[float], order: int):
        hh = -h
        h_phi_1 = math.expm1(hh) if math.isfinite(hh) else -1.0
        B_h = h_phi_1
        h_phi_k = (h_phi_1 / hh - 1.0) if math.isfinite(hh) else -1.0
        fact = 1.0
        R, b = [], []
        for i in range(1, order + 1):
            R.append([rk ** (i - 1) for rk in rks])
            b.append(h_phi_k * fact / B_h)
            fact *= (i + 1)
            h_phi_k = (h_phi_k / hh - 1.0 / fact) if math.isfinite(hh) else -1.0 / fact
        return h_phi_1, B_h, np.array(R, dtype=np.float64), np.array(b, dtype=np.float64)

    def multistep_uni_p_bh_update(self, sample: torch.Tensor, order: int) -> torch.Tensor:
        i = self._step_index
        m0 = self.model_outputs[-1]
        sig_t, sig_s0 = self.sigmas[i + 1], self.sigmas[i]
        alpha_t = 1.0 - sig_t
        lam_t, lam_s0 = self._lambda(sig_t), self._lambda(sig_s0)
        h = lam_t - lam_s0
        rks, D1s = [], []
        for k in range(1, order):
            mk = self.model_outputs[-(k + 1)]
            rk = (self._lambda(self.sigmas[i - k]) - lam_s0) / h
            rks.append(rk)
            D1s.append((mk - m0) / rk)
        rks.append(1.0)
        h_phi_1, B_h, R, b = self._coeffs(h, rks, order)
        x_t_ = (sig_t / sig_s0) * sample.float() - alpha_t * h_phi_1 * m0
        if D1s:
            rhos = [0.5] if order == 2 else np.linalg.solve(R[:-1, :-1], b[:-1]).tolist()
            pred = sum(r * d for r, d in zip(rhos, D1s))
            x_t_ = x_t_ - alpha_t * B_h * pred
        return x_t_

    def multistep_uni_c_bh_update(self, this_model_output: torch.Tensor, last_sample: torch.Tensor, order: int):
        i = self._step_index
        m0 = self.model_outputs[-1]
        sig_t, sig_s0 = self.sigmas[i], self.sigmas[i - 1]
        alpha_t = 1.0 - sig_t
        lam_t, lam_s0 = self._lambda(sig_t), self._lambda(sig_s0)
        h = lam_t - lam_s0
        rks, D1s = [], []
        for k in range(1, order):
            mk = self.model_outputs[-(k + 1)]
            rk = (self._lambda(self.sigmas[i - (k + 1)]) - lam_s0) / h
            rks.append(rk)
            D1s.append((mk - m0) / rk)
        rks.append(1.0)
        h_phi_1, B_h, R, b = self._coeffs(h, rks, order)
        rhos = [0.5] if order == 1 else np.linalg.solve(R, b).tolist()
        x_t_ = (sig_t / sig_s0) * last_sample.float() - alpha_t * h_phi_1 * m0
        corr = sum(r * d for r, d in zip(rhos[:-1], D1s)) if D1s else 0.0
        return x_t_ - alpha_t * B_h * (corr + rhos[-1] * (this_model_output - m0))

    def step(self, model_output: torch.Tensor, timestep, sample: torch.Tensor, **_) -> torch.Tensor:
        i = self._step_index
        use_corrector = i > 0 and (i - 1) not in self.disable_corrector and self.last_sample is not None
        x0 = self.convert_model_output(model_output, sample, i)
        if use_corrector:
            sample = self.multistep_uni_c_bh_update(x0, self.last_sample, self.this_order)
        for k in range(self.solver_order - 1):
            self.model_outputs[k] = self.model_outputs[k + 1]
        self.model_outputs[-1] = x0
        order = min(self.solver_order, self.num_inference_steps - i) if self.config["lower_order_final"] \
            else self.solver_order
        self.this_order = min(order, self.lower_order_nums + 1)
        self.last_sample = sample.float()
        prev = self.multistep_uni_p_bh_update(sample, self.this_order)
        if self.lower_order_nums < self.solver_order:
            self.lower_order_nums += 1
        self._step_index += 1
        return prev.to(sample.dtype)
