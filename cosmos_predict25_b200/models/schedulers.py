"""Noise schedules and samplers for rectified-flow models.

* ``RectifiedFlowSchedule``: train-time sampling (uniform / logit-normal u), the 1000-entry shifted
  sigma/timestep table and the interpolation x_t = sigma*eps + (1-sigma)*x0, target eps - x0
  (cosmos_predict2/_src/predict2/schedulers/rectified_flow.py:22-173; the table is the one
  diffusers' FlowMatchEulerDiscreteScheduler(shift=s) builds).
* ``FlowUniPCSolver``: order-2 UniPC (B(h)=expm1 variant "bh2", x0-prediction, lower-order final
  step, corrector from the second step) over shifted flow sigmas, with the Karras-sigma override
  (cosmos_predict2/_src/predict2/models/fm_solvers_unipc.py:15-766).
* ``FlowEulerSolver``: plain Euler over the same sigmas (used by the CPU test configuration).

All schedule arithmetic happens on the host in float32 so the sampling loop never synchronises
with the GPU; only the per-step tensor update touches device memory.
"""

from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from ..ops import functional as ops


class RectifiedFlowSchedule:
    def __init__(self, shift: float = 5.0, num_train_timesteps: int = 1000,
                 train_time_distribution: str = "logitnormal", train_time_weight: str = "uniform"):
        if train_time_weight == "reweighting":
            train_time_weight = "uniform"
        assert train_time_weight == "uniform", "only the uniform loss weight exists for rectified flow"
        assert train_time_distribution in ("uniform", "logitnormal"), train_time_distribution
        self.shift = float(shift)
        self.num_train_timesteps = num_train_timesteps
        self.train_time_distribution = train_time_distribution
        tau = np.linspace(1.0, 1.0 / num_train_timesteps, num_train_timesteps, dtype=np.float32)
        sig = self.shift * tau / (1.0 + (self.shift - 1.0) * tau)
        self.sigmas = torch.from_numpy(sig.astype(np.float32))
        self.timesteps = self.sigmas * num_train_timesteps

    def sample_train_time(self, batch_size: int, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        if self.train_time_distribution == "uniform":
            return torch.rand((batch_size,), generator=generator)
        return torch.sigmoid(torch.randn((batch_size,), generator=generator))

    def indices(self, u: torch.Tensor) -> torch.Tensor:
        return (u.reshape(-1) * self.num_train_timesteps).long().clamp_(0, self.num_train_timesteps - 1)

    def discrete_timesteps(self, u: torch.Tensor) -> torch.Tensor:
        return self.timesteps[self.indices(u.cpu())]

    def sigmas_for(self, u: torch.Tensor) -> torch.Tensor:
        return self.sigmas[self.indices(u.cpu())]

    def loss_weight(self, t: torch.Tensor) -> torch.Tensor:
        return torch.ones_like(t)

    @staticmethod
    def interpolate(eps: torch.Tensor, x0: torch.Tensor, sigma: torch.Tensor):
        """Returns (x_t, velocity target)."""
        s = sigma.view(-1, *([1] * (x0.ndim - 1))).to(x0)
        return eps * s + x0 * (1 - s), eps - x0


def flow_sigmas(num_steps: int, shift: float, sigma_max: float, sigma_min: float, use_karras: bool = False) -> np.ndarray:
    """Sampling sigmas including the trailing 0 (length num_steps+1, or num_steps+2 for Karras)."""
    if use_karras:
        ramp = np.arange(num_steps + 1) / num_steps
        lo, hi = 0.01 ** (1 / 7), 200 ** (1 / 7)
        sig = (hi + ramp * (lo - hi)) ** 7
        sig = sig / (1 + sig)
    else:
        sig = np.linspace(sigma_max, sigma_min, num_steps + 1).copy()[:-1]
        sig = shift * sig / (1 + (shift - 1) * sig)
    return np.concatenate([sig, [0.0]]).astype(np.float32)


class _FlowSolverBase:
    def __init__(self, num_train_timesteps: int = 1000, shift: float = 1.0):
        self.num_train_timesteps = num_train_timesteps
        self.shift = shift
        alphas = np.linspace(1, 1 / num_train_timesteps, num_train_timesteps)[::-1].copy()
        base = (1.0 - alphas).astype(np.float32)
        base = shift * base / (1 + (shift - 1) * base)
        # the table runs from the noisiest entry (0.999 at shift 1) down to 0
        self.sigma_min = float(base[-1])
        self.sigma_max = float(base[0])
        self.sigmas = base
        self.timesteps = torch.from_numpy(base * num_train_timesteps)
        self.num_inference_steps = None
        self.step_index = None

    def set_timesteps(self, num_inference_steps: int, device=None, shift: Optional[float] = None,
                      use_kerras_sigma: bool = False, sigmas: Optional[Sequence[float]] = None):
        shift = self.shift if shift is None else shift
        if sigmas is not None:
            sig = np.asarray(sigmas, dtype=np.float64)
            sig = shift * sig / (1 + (shift - 1) * sig)
            sig = np.concatenate([sig, [0.0]]).astype(np.float32)
        else:
            sig = flow_sigmas(num_inference_steps, shift, self.sigma_max, self.sigma_min, use_kerras_sigma)
        self.sigmas = sig
        self.timesteps = torch.from_numpy((sig[:-1] * self.num_train_timesteps)).to(dtype=torch.int64, device=device)
        self.num_inference_steps = len(self.timesteps)
        self.step_index = None
        self._reset()

    def _reset(self):
        pass


class FlowEulerSolver(_FlowSolverBase):
    """x <- x + (sigma_next - sigma) * v."""

    def __init__(self, num_train_timesteps: int = 1000, shift: float = 1.0):
        super().__init__(num_train_timesteps, shift)

    def step(self, model_output: torch.Tensor, timestep, sample: torch.Tensor) -> torch.Tensor:
        if self.step_index is None:
            self.step_index = 0
        i = self.step_index
        dt = float(self.sigmas[i + 1]) - float(self.sigmas[i])
        self.step_index += 1
        return ops.lincomb([sample, model_output.to(sample.dtype)], [1.0, dt])


class FlowUniPCSolver(_FlowSolverBase):
    """Unified predictor-corrector multistep solver specialised to flow prediction.

    With sigma the noise level, alpha = 1 - sigma and lambda = log(alpha/sigma). The network's
    velocity v is converted to a data prediction x0 = x - sigma*v; updates are exponential
    integrator steps in lambda with the B(h) = expm1(h) ("bh2") or B(h) = h ("bh1") weighting.
    """

    def __init__(self, num_train_timesteps: int = 1000, solver_order: int = 2, shift: float = 1.0,
                 solver_type: str = "bh2", lower_order_final: bool = True, disable_corrector: Sequence[int] = (),
                 predict_x0: bool = True):
        assert solver_type in ("bh1", "bh2")
        assert predict_x0, "only the data-prediction form is used by flow models"
        super().__init__(num_train_timesteps, shift)
        self.solver_order = solver_order
        self.solver_type = solver_type
        self.lower_order_final = lower_order_final
        self.disable_corrector = list(disable_corrector)
        self._reset()

    def _reset(self):
        self.model_outputs: List[Optional[torch.Tensor]] = [None] * self.solver_order
        self.lower_order_nums = 0
        self.last_sample = None
        self.this_order = 1

    # ---- host-side coefficient maths (float32 to mirror the reference's tensor arithmetic) ----
    @staticmethod
    def _lam(sigma: np.float32) -> np.float32:
        with np.errstate(divide="ignore"):
            return np.float32(np.log(np.float32(1.0) - sigma) - np.log(sigma))

    def _coeffs(self, sigma_t, sigma_s0, prev_sigmas: Sequence, order: int, corrector: bool):
        """Returns (c_x, c_m0, B_h*alpha_t, rhos) for x_t = c_x*x + c_m0*m0 - alpha_t*B_h*(sum rho_k D1_k)."""
        f32 = np.float32
        sigma_t, sigma_s0 = f32(sigma_t), f32(sigma_s0)
        alpha_t = f32(1.0) - sigma_t
        lam_t, lam_s0 = self._lam(sigma_t), self._lam(sigma_s0)
        h = f32(lam_t - lam_s0)
        rks = []
        for s in prev_sigmas:
            rks.append(f32((self._lam(f32(s)) - lam_s0) / h))
        rks.append(f32(1.0))
        rks = np.asarray(rks, dtype=np.float32)
        hh = f32(-h)
        h_phi_1 = f32(np.expm1(hh))
        with np.errstate(invalid="ignore", divide="ignore"):
            h_phi_k = f32(h_phi_1 / hh - 1.0)
            B_h = h_phi_1 if self.solver_type == "bh2" else hh
            R, b = [], []
            fact = 1
            for i in range(1, order + 1):
                R.append(rks ** (i - 1))
                b.append(f32(h_phi_k * fact / B_h))
                fact *= i + 1
                h_phi_k = f32(h_phi_k / hh - 1.0 / fact)
        R = np.stack(R).astype(np.float32)
        b = np.asarray(b, dtype=np.float32)
        if corrector:
            rhos = np.asarray([0.5], dtype=np.float32) if order == 1 else np.linalg.solve(R, b).astype(np.float32)
        else:
            if order == 1:
                rhos = np.zeros((0,), dtype=np.float32)
            elif order == 2:
                rhos = np.asarray([0.5], dtype=np.float32)
            else:
                rhos = np.linalg.solve(R[:-1, :-1], b[:-1]).astype(np.float32)
        c_x = f32(sigma_t / sigma_s0)
        c_m0 = f32(-alpha_t * h_phi_1)
        return float(c_x), float(c_m0), float(alpha_t * B_h), rks, rhos

    # ---- tensor updates -------------------------------------------------------------------
    def _combine(self, base: torch.Tensor, c_x: float, c_m0: float, terms) -> torch.Tensor:
        """``c_x * base + c_m0 * m0 - sum_k a_k * (t_k - m0)`` for ``terms = [(a_k, t_k)]``. fp32 state on a GPU: the coefficients of
        m0 are folded on the host and the update is ONE pass over memory (``ops.lincomb``); elsewhere term by term."""
        m0 = self.model_outputs[-1]
        ts = [t for _, t in terms]
        if base.is_cuda and base.dtype == torch.float32 and all(t.dtype == torch.float32 and t.shape == base.shape for t in [m0] + ts):
            return ops.lincomb([base, m0] + ts, [c_x, c_m0 + sum(a for a, _ in terms)] + [-a for a, _ in terms])
        x = c_x * base + c_m0 * m0
        for a, t in terms:
            x = x - a * (t - m0)
        return x.to(base.dtype)

    def _predict(self, sample: torch.Tensor, order: int) -> torch.Tensor:
        i = self.step_index
        prev = [self.sigmas[i - k] for k in range(1, order)]
        c_x, c_m0, aB, rks, rhos = self._coeffs(self.sigmas[i + 1], self.sigmas[i], prev, order, corrector=False)
        terms = [(aB * float(rhos[k]) / float(rks[k]), self.model_outputs[-(k + 2)]) for k in range(order - 1)]
        return self._combine(sample, c_x, c_m0, terms)

    def _correct(self, this_x0: torch.Tensor, order: int) -> torch.Tensor:
        i = self.step_index
        prev = [self.sigmas[i - (k + 1)] for k in range(1, order)]
        c_x, c_m0, aB, rks, rhos = self._coeffs(self.sigmas[i], self.sigmas[i - 1], prev, order, corrector=True)
        terms = [(aB * float(rhos[k]) / float(rks[k]), self.model_outputs[-(k + 2)]) for k in range(order - 1)]
        terms.append((aB * float(rhos[-1]), this_x0))
        return self._combine(self.last_sample, c_x, c_m0, terms)

    def step(self, model_output: torch.Tensor, timestep, sample: torch.Tensor) -> torch.Tensor:
        """One solver step: optional corrector on ``sample`` with the new evaluation, then predictor."""
        if self.num_inference_steps is None:
            raise ValueError("call set_timesteps first")
        if self.step_index is None:
            self.step_index = 0
        i = self.step_index
        x0 = ops.lincomb([sample, model_output.to(sample.dtype)], [1.0, -float(self.sigmas[i])])
        use_corrector = i > 0 and (i - 1) not in self.disable_corrector and self.last_sample is not None
        if use_corrector:
            sample = self._correct(x0, self.this_order)
        self.model_outputs = self.model_outputs[1:] + [x0]
        if self.lower_order_final:
            order = min(self.solver_order, self.num_inference_steps - i)
        else:
            order = self.solver_order
        self.this_order = min(order, self.lower_order_nums + 1)
        self.last_sample = sample
        prev = self._predict(sample, self.this_order)
        if self.lower_order_nums < self.solver_order:
            self.lower_order_nums += 1
        self.step_index += 1
        return prev


def sample_loop(velocity_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], noise: torch.Tensor,
                solver: _FlowSolverBase, num_steps: int, shift: float, use_kerras_sigma: bool = False,
                callback: Optional[Callable] = None) -> torch.Tensor:
    """Integrate from noise to data. ``velocity_fn(x, t)`` takes the per-sample timestep tensor [B]."""
    solver.set_timesteps(num_steps, device="cpu", shift=shift, use_kerras_sigma=use_kerras_sigma)
    x = noise
    ones = torch.ones(noise.shape[0], device=noise.device, dtype=torch.float32)
    for i, t in enumerate(solver.timesteps.tolist()):
        v = velocity_fn(x, ones * float(t))
        x = solver.step(v, t, x)
        if callback is not None:
            callback(i, x)
    return x
