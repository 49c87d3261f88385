"""EDM-era (Predict2) diffusion models and samplers, kept for checkpoint and experiment parity.

Parity targets: ``EDMScaling`` / ``RectifiedFlowScaling`` (cosmos_predict2/_src/common/modules/denoiser_scaling.py:21-64),
``EDMSDE`` (.../edm_sde.py:22), ``Sampler`` with multistep "2ab" and Runge-Kutta solvers (.../res_sampler.py:108,
cosmos_predict2/_src/common/functional/{runge_kutta,multi_step}.py), the EDM Euler/Heun sampler (.../edm_sampler.py:23),
``DiffusionModel`` (cosmos_predict2/_src/predict2/models/text2world_model.py:123-874) and ``Video2WorldModel`` with
sigma-conditional clean frames and the high-sigma sampling strategies (cosmos_predict2/_src/predict2/models/video2world_model.py:44-166).

Sampler arithmetic runs in float64 on the solver side exactly as in the reference (the denoiser is called in its own
precision); coefficients are computed on the host so the loop does not synchronise with the GPU.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch

from .conditioner import DataType
from .schedulers import FlowUniPCSolver
from .rectified_flow import (NUM_CONDITIONAL_FRAMES_KEY, Text2WorldModelRectifiedFlow, Text2WorldRFConfig,
                             Video2WorldModelRectifiedFlow)


# ---- preconditioning ----------------------------------------------------------------------------------------------
class EDMScaling:
    def __init__(self, sigma_data: float = 0.5):
        self.sigma_data = sigma_data

    def __call__(self, sigma: torch.Tensor):
        sd = self.sigma_data
        c_skip = sd ** 2 / (sigma ** 2 + sd ** 2)
        c_out = sigma * sd / (sigma ** 2 + sd ** 2).sqrt()
        c_in = 1 / (sigma ** 2 + sd ** 2).sqrt()
        c_noise = 0.25 * sigma.log()
        return c_skip, c_out, c_in, c_noise


class RectifiedFlowScaling:
    """Runs a rectified-flow network inside the EDM interface: t = sigma / (1 + sigma)."""

    def __init__(self, sigma_data: float = 1.0, t_scaling_factor: float = 1.0, loss_weight_uniform: bool = True):
        assert abs(sigma_data - 1.0) < 1e-6, "sigma_data must be 1.0 for rectified-flow scaling"
        self.t_scaling_factor = t_scaling_factor
        self.loss_weight_uniform = loss_weight_uniform
        if not loss_weight_uniform:
            # a bell over t in [0, 1] centred on 0.5, shifted to zero at the ends and scaled to mean 1: the middle of the
            # trajectory weighs most (denoiser_scaling.py:38-45 of the reference)
            self.num_steps = 1000
            bell = torch.exp(-2 * (torch.linspace(0, 1, self.num_steps) - 0.5) ** 2)
            bell = bell - bell.min()
            self.weights = bell * (self.num_steps / bell.sum())

    def __call__(self, sigma: torch.Tensor):
        t = sigma / (sigma + 1)
        return 1.0 - t, -t, 1.0 - t, t * self.t_scaling_factor

    def sigma_loss_weights(self, sigma: torch.Tensor) -> torch.Tensor:
        if self.loss_weight_uniform:
            return (1.0 + sigma) ** 2 / sigma ** 2
        index = (sigma / (sigma + 1) * self.num_steps).round().long().clamp_(0, self.num_steps - 1)
        return self.weights.to(sigma.device)[index].type_as(sigma)


class EDMSDE:
    """log-normal training noise levels: sigma = exp(p_mean + p_std * N(0,1))."""

    def __init__(self, p_mean: float = -1.2, p_std: float = 1.2, sigma_max: float = 80.0, sigma_min: float = 0.002):
        self.p_mean, self.p_std, self.sigma_max, self.sigma_min = p_mean, p_std, sigma_max, sigma_min

    def sample_t(self, batch_size: int, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """With a torch generator: exp(p_mean + p_std N(0,1)) from it. Without: uniform draws from NumPy's global generator
        pushed through the inverse normal CDF, like the reference (edm_sde.py:34-39 there), so ``np.random.seed`` reproduces its
        noise levels."""
        if generator is not None:
            return torch.exp(torch.randn(batch_size, generator=generator) * self.p_std + self.p_mean)
        from statistics import NormalDist
        dist = NormalDist(mu=self.p_mean, sigma=self.p_std)
        return torch.exp(torch.tensor([dist.inv_cdf(float(u)) for u in np.random.uniform(size=(batch_size))]))

    def marginal_prob(self, x0: torch.Tensor, sigma: torch.Tensor):
        return x0, sigma


# ---- solver steps (x0 / "data prediction" form, time variable = sigma) --------------------------------------------------
def _bm(c, x):
    c = torch.as_tensor(c, dtype=x.dtype, device=x.device)
    return c.view(-1, *([1] * (x.ndim - 1))) * x if c.ndim > 0 else c * x


def phi1(t):
    return np.expm1(t) / t


def phi2(t):
    return (phi1(t) - 1.0) / t


def reg_x0_euler_step(x_s, s: float, t: float, x0_s):
    return ((s - t) / s) * x0_s + (t / s) * x_s, x0_s


def res_x0_rk2_step(x_s, t: float, s: float, x0_s, s1: float, x0_s1):
    """Exponential-integrator second-order step in lambda = -log(sigma) using two data predictions."""
    ls, lt, lm = -math.log(s), -math.log(t), -math.log(s1)
    dt = lt - ls
    assert abs(dt) > 1e-6 and abs(lm - ls) > 1e-6, "step size is too small"
    c2 = (lm - ls) / dt
    p1, p2 = phi1(-dt), phi2(-dt)
    b1 = float(np.nan_to_num(p1 - p2 / c2))
    b2 = float(np.nan_to_num(p2 / c2))
    return math.exp(-dt) * x_s + dt * (b1 * x0_s + b2 * x0_s1)


def order2_ab_step(x_s, s, t, x0_s, history):
    """Second-order Adams-Bashforth multistep ("2ab"): reuses the previous step's data prediction."""
    if history:
        x0_prev, s_prev = history[0]
        x_t = res_x0_rk2_step(x_s, t, s, x0_s, s_prev, x0_prev)
    else:
        x_t = reg_x0_euler_step(x_s, s, t, x0_s)[0]
    return x_t, [(x0_s, s)]


def rk1_euler(x_s, s, t, x0_fn):
    return reg_x0_euler_step(x_s, s, t, x0_fn(x_s, s))


def rk2_mid(x_s, s, t, x0_fn):
    s1 = math.sqrt(s * t)
    x_s1, x0_s = rk1_euler(x_s, s, s1, x0_fn)
    x0_s1 = x0_fn(x_s1, s1)
    return res_x0_rk2_step(x_s, t, s, x0_s, s1, x0_s1), x0_s1


def rk2_heun_edm(x_s, s, t, x0_fn):
    x_t, x0_s = rk1_euler(x_s, s, t, x0_fn)
    x0_t = x0_fn(x_t, t)
    return reg_x0_euler_step(x_s, s, t, (x0_s + x0_t) / 2)


RUNGE_KUTTA = {"1euler": rk1_euler, "2mid": rk2_mid, "2heun": rk2_heun_edm}
MULTISTEP = {"2ab": order2_ab_step}


def get_rev_ts(t_min: float, t_max: float, num_steps: int, ts_order: float = 7.0) -> np.ndarray:
    """Karras spacing from t_max down to t_min (num_steps + 1 points)."""
    if t_min >= t_max:
        raise ValueError("t_min must be less than t_max")
    i = np.arange(num_steps + 1, dtype=np.float64)
    return (t_max ** (1 / ts_order) + i / num_steps * (t_min ** (1 / ts_order) - t_max ** (1 / ts_order))) ** ts_order


class RESSampler:
    """Multistep / Runge-Kutta ODE sampler over Karras sigmas with optional churn, then one clean-up denoise."""

    @torch.no_grad()
    def __call__(self, x0_fn: Callable, x_sigma_max: torch.Tensor, num_steps: int = 35, sigma_min: float = 0.002,
                 sigma_max: float = 80.0, rho: float = 7.0, S_churn: float = 0.0, S_min: float = 0.0, S_max: float = float("inf"),
                 S_noise: float = 1.0, solver_option: str = "2ab", sample_clean: bool = True) -> torch.Tensor:
        in_dtype = x_sigma_max.dtype
        B = x_sigma_max.shape[0]
        dev = x_sigma_max.device

        def f64(x, sig: float):
            return x0_fn(x.to(in_dtype), torch.full((B,), sig, device=dev, dtype=in_dtype)).to(torch.float64)

        multi = solver_option in MULTISTEP
        assert multi or solver_option in RUNGE_KUTTA, f"unsupported solver {solver_option}"
        order = 1 if multi else int(solver_option[0])
        sig = get_rev_ts(sigma_min, sigma_max, num_steps // order, rho)
        n = len(sig) - 1
        eta = min(S_churn / (n + 1), math.sqrt(1.2) - 1)
        x = x_sigma_max.to(torch.float64)
        hist: List = []
        for i in range(n):
            s, t = float(sig[i]), float(sig[i + 1])
            if S_min < s < S_max and eta > 0:
                s_hat = s + eta * s
                x = x + math.sqrt(s_hat ** 2 - s ** 2) * S_noise * torch.randn_like(x)
                s = s_hat
            if multi:
                x0 = f64(x, s)
                x, hist = MULTISTEP[solver_option](x, s, t, x0, hist)
            else:
                x, _ = RUNGE_KUTTA[solver_option](x, s, t, f64)
        if sample_clean:
            x = f64(x, float(sig[-1]))
        return x.to(in_dtype)


class EDMEulerSampler:
    """Plain EDM sampler (Euler, optional Heun correction) in the eps form d = (x - x0) / sigma."""

    @torch.no_grad()
    def __call__(self, x0_fn: Callable, x_sigma_max: torch.Tensor, num_steps: int = 35, sigma_min: float = 0.002,
                 sigma_max: float = 80.0, rho: float = 7.0, heun: bool = True) -> torch.Tensor:
        sig = np.append(get_rev_ts(sigma_min, sigma_max, num_steps - 1, rho), 0.0)
        x = x_sigma_max.to(torch.float64)
        B, dev, dt_in = x.shape[0], x.device, x_sigma_max.dtype
        call = lambda xx, s: x0_fn(xx.to(dt_in), torch.full((B,), s, device=dev, dtype=dt_in)).to(torch.float64)
        for i in range(len(sig) - 1):
            s, t = float(sig[i]), float(sig[i + 1])
            d = (x - call(x, s)) / s
            x_next = x + (t - s) * d
            if heun and t > 0:
                d2 = (x_next - call(x_next, t)) / t
                x_next = x + (t - s) * 0.5 * (d + d2)
            x = x_next
        return x.to(dt_in)


# ---- models ------------------------------------------------------------------------------------------------------------
class HighSigmaStrategy:
    NONE = "none"
    UNIFORM80_2000 = "uniform80_2000"
    LOGUNIFORM200_100000 = "LOGUNIFORM200_100000"      # spelled like the reference's value; compared without regard to case
    SHIFT24 = "shift24"
    BALANCED_TWO_HEADS_V1 = "balanced_two_heads_v1"
    HARDCODED_20steps = "hardcoded_20steps"


@dataclass
class EDMConfig(Text2WorldRFConfig):
    sigma_data: float = 0.5                  # 1.0 with the rectified-flow scaling
    scaling: str = "edm"                     # "edm" | "rectified_flow"
    denoise_replace_gt_frames: bool = True   # Video2World: the prediction on conditioning frames is their clean latent
    use_flowunipc_scheduler: bool = False    # sample with the flow UniPC solver instead of the noise-level samplers
    adjust_video_noise: bool = True          # video batches: noise levels x sqrt(state_t) (more frames share one level)
    loss_reduce: str = "mean"                # "mean" | "sum" (sum over channels, mean over the rest)
    p_mean: float = 0.0
    p_std: float = 1.0
    sigma_max: float = 80.0
    sigma_min: float = 0.0002
    loss_scale: float = 10.0
    rectified_flow_t_scaling_factor: float = 1.0
    rectified_flow_loss_weight_uniform: bool = True
    sigma_conditional: float = 0.0001
    min_num_conditional_frames: int = 1
    max_num_conditional_frames: int = 2
    conditional_frames_probs: Optional[Dict[int, float]] = None
    high_sigma_strategy: str = HighSigmaStrategy.NONE
    high_sigma_ratio: float = 0.05
    low_sigma_ratio: float = 0.05


class DiffusionModel(Text2WorldModelRectifiedFlow):
    """EDM-preconditioned denoiser D(x, sigma) = c_skip x + c_out F(c_in x, c_noise) with per-sigma loss weights."""

    def __init__(self, config: EDMConfig, **kw):
        super().__init__(config, **kw)
        c = config
        self.sde = EDMSDE(c.p_mean, c.p_std, c.sigma_max, c.sigma_min)
        self.scaling = (RectifiedFlowScaling(c.sigma_data, c.rectified_flow_t_scaling_factor, c.rectified_flow_loss_weight_uniform)
                        if c.scaling == "rectified_flow" else EDMScaling(c.sigma_data))
        self.sampler = RESSampler()
        self.sigma_data = c.sigma_data
        self.video_noise_multiplier = math.sqrt(c.state_t) if c.adjust_video_noise else 1.0
        assert c.loss_reduce in ("mean", "sum")

    @torch.no_grad()
    def encode(self, state: torch.Tensor) -> torch.Tensor:
        return super().encode(state) * self.sigma_data            # latents are kept at the data scale the preconditioning assumes

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        return super().decode(latent / self.sigma_data)

    def get_data_and_condition(self, batch: Dict):
        raw, latent, condition = super().get_data_and_condition(batch)
        if raw is None:                                            # pre-computed tokenizer latents: same scale as ``encode`` gives
            latent = latent * self.sigma_data
        return raw, latent, condition

    def draw_training_sigma(self, B: int, is_video: bool) -> torch.Tensor:
        """[B] noise levels: log-normal, times sqrt(state_t) for video; Video2World models then apply the high-noise strategy
        (``_high_sigma``)."""
        sigma = self.sde.sample_t(B)
        if is_video:
            sigma = sigma * self.video_noise_multiplier
        return sigma

    def sigma_loss_weights(self, sigma: torch.Tensor) -> torch.Tensor:
        if isinstance(self.scaling, RectifiedFlowScaling):
            return self.scaling.sigma_loss_weights(sigma)
        sd = self.config.sigma_data
        return (sigma ** 2 + sd ** 2) / (sigma * sd) ** 2

    def denoise_edm(self, xt: torch.Tensor, sigma: torch.Tensor, condition) -> torch.Tensor:
        """x0 prediction. sigma [B] or [B,T]."""
        B = xt.shape[0]
        sig = sigma.view(B, 1, -1, 1, 1) if sigma.ndim == 2 else sigma.view(B, 1, 1, 1, 1)
        c_skip, c_out, c_in, c_noise = self.scaling(sig.float())
        t_net = c_noise.view(B, -1)
        net_out = self.net((xt.float() * c_in).to(**self.tensor_kwargs), t_net, **self._net_kwargs(condition)).float()
        return c_skip * xt.float() + c_out * net_out

    def training_step(self, data_batch: Dict, iteration: int):
        _, x0, condition = self.get_data_and_condition(data_batch)
        B = x0.shape[0]
        is_video = condition.data_type == DataType.VIDEO
        eps = torch.randn(x0.shape, **self.tensor_kwargs_fp32)          # noise first, then the levels: the reference's draw order
        sigma = self.draw_training_sigma(B, is_video).to(**self.tensor_kwargs_fp32)
        x0, condition, eps, sigma = self.broadcast_split_for_model_parallelsim(x0, condition, eps, sigma)
        xt = x0 + eps * sigma.view(B, 1, 1, 1, 1)
        x0_pred = self.denoise_edm(xt, sigma, condition)
        w = self.sigma_loss_weights(sigma).view(B, 1, 1, 1, 1)
        weighted = w * (x0_pred - x0) ** 2
        if self.config.loss_reduce == "mean":
            loss = weighted.mean() * self.config.loss_scale
        else:
            loss = weighted.sum(dim=1).mean() * self.config.loss_scale
        out = {"x0": x0, "xt": xt, "sigma": sigma, "weights_per_sigma": w.view(B, -1), "condition": condition, "model_pred": x0_pred,
               "mse_loss": ((x0_pred - x0) ** 2).mean().detach(), "edm_loss": weighted.mean().detach(),
               "edm_loss_per_frame": weighted.detach().mean(dim=[1, 3, 4])}        # [B, T]: what the per-frame analysis reads
        return out, loss

    @torch.no_grad()
    def generate_samples_from_batch(self, data_batch: Dict, guidance: float = 1.5, seed: int = 1, state_shape=None,
                                    n_sample=None, is_negative_prompt: bool = False, num_steps: int = 35,
                                    solver_option: str = "2ab", x_sigma_max: Optional[torch.Tensor] = None,
                                    sigma_max: Optional[float] = None, **kw) -> torch.Tensor:
        """Latents (at the model's data scale) from noise: the multistep / Runge-Kutta sampler over Karras noise levels, or - with
        ``config.use_flowunipc_scheduler`` - the flow UniPC solver driven through ``denoise_with_velocity`` (text2world_model.py:
        519-640 of the reference). ``guided_image`` / ``guided_mask`` in the batch pin parts of every prediction."""
        from ..utils.misc import arch_invariant_rand
        self._normalize_video_databatch_inplace(data_batch)
        self._augment_image_dim_inplace(data_batch)
        is_image = self.is_image_batch(data_batch)
        cond, uncond = self._conditions_for_sampling(data_batch, is_negative_prompt)
        cfg = self.config
        key = cfg.input_image_key if is_image else (cfg.input_data_key if cfg.input_data_key in data_batch else cfg.input_latent_key)
        n_sample = n_sample or data_batch[key].shape[0]
        if state_shape is None:
            if key == cfg.input_latent_key:
                state_shape = tuple(data_batch[key].shape[1:])
            else:
                _T, _H, _W = data_batch[key].shape[-3:]
                tk = self.tokenizer
                state_shape = (cfg.state_ch, tk.get_latent_num_frames(_T), _H // tk.spatial_compression_factor, _W // tk.spatial_compression_factor)
        cond, uncond = self._prepare_sampling_conditions(data_batch, cond, uncond)
        noise = arch_invariant_rand((n_sample,) + tuple(state_shape), torch.float32, self.device_, seed)

        if getattr(cfg, "use_flowunipc_scheduler", False):
            solver = FlowUniPCSolver(1000, shift=1.0)
            solver.set_timesteps(num_steps, device="cpu", shift=5.0)
            x = noise
            for t in solver.timesteps.tolist():
                tt = torch.full((n_sample, 1), float(t) / 1000.0, device=x.device)
                c, u = self.denoise_with_velocity(x, tt, cond), self.denoise_with_velocity(x, tt, uncond)
                x = solver.step(u + guidance * (c - u), t, x)
            return x

        combine = self._guidance_combiner(data_batch, guidance)

        def x0_fn(x, sigma):
            x0 = combine(self.denoise_edm(x, sigma, cond), self.denoise_edm(x, sigma, uncond))
            if "guided_image" in data_batch:
                assert "guided_mask" in data_batch, "guided_mask should be in data_batch if guided_image is present"
                x0 = data_batch["guided_mask"] * data_batch["guided_image"] + (1 - data_batch["guided_mask"]) * x0
            return x0

        if x_sigma_max is None:
            x_sigma_max = noise * self.sde.sigma_max
        return self.sampler(x0_fn, x_sigma_max, num_steps=num_steps, sigma_max=self.sde.sigma_max if sigma_max is None else sigma_max,
                            sigma_min=self.sde.sigma_min, solver_option=solver_option)

    def _prepare_sampling_conditions(self, data_batch, cond, uncond):
        return cond, uncond

    def _guidance_combiner(self, data_batch: Dict, guidance: float) -> Callable:
        """(conditional, unconditional) clean-latent predictions -> the guided one."""
        return lambda c, u: c + guidance * (c - u)


class Video2WorldModel(DiffusionModel):
    """EDM Video2World: clean conditioning frames are fed at a tiny noise level ``sigma_conditional`` (per-frame sigma)
    and their x0 prediction is replaced by the ground truth."""

    condition_is_video2world = True

    def get_data_and_condition(self, batch: Dict):
        raw, latent, condition = super().get_data_and_condition(batch)
        c = self.config
        condition = condition.set_video_condition(latent.to(**self.tensor_kwargs), c.min_num_conditional_frames,
                                                  c.max_num_conditional_frames, batch.get(NUM_CONDITIONAL_FRAMES_KEY),
                                                  c.conditional_frames_probs)
        return raw, latent, condition

    def draw_training_sigma(self, B: int, is_video: bool) -> torch.Tensor:
        """Base levels, then for video batches the high-noise strategy (video2world_model.py:89-146 of the reference; draws in
        its order): ``uniform80_2000`` / ``loguniform200_100000``: a share ``high_sigma_ratio`` of the samples is re-drawn from
        that range; ``shift24``: every sample is re-drawn as t / (1 - t) with t = 24 u / (1 + 23 u), then the uniform re-draw;
        ``balanced_two_heads_v1``: the log-uniform re-draw, then a share ``low_sigma_ratio`` re-drawn uniformly in (1e-5, 2);
        ``hardcoded_20steps``: every sample from the 20-step sampling grid plus 100000."""
        sigma = super().draw_training_sigma(B, is_video)
        c = self.config
        strat = str(c.high_sigma_strategy).lower()
        if not is_video or strat == HighSigmaStrategy.NONE:
            return sigma
        rand = lambda: torch.rand(sigma.shape)
        log_lo, log_hi = math.log(200.0), math.log(100000.0)
        if strat == HighSigmaStrategy.UNIFORM80_2000.lower():
            pick = rand() < c.high_sigma_ratio
            sigma = torch.where(pick, rand().type_as(sigma) * 1920 + 80, sigma)
        elif strat == HighSigmaStrategy.LOGUNIFORM200_100000.lower():
            pick = rand() < c.high_sigma_ratio
            sigma = torch.where(pick, (rand().type_as(sigma) * (log_hi - log_lo) + log_lo).exp(), sigma)
        elif strat == HighSigmaStrategy.SHIFT24.lower():
            t = rand().double()
            t = 24 * t / (24 * t + 1 - t)
            sigma = (t / (1.0 - t)).float()
            pick = rand() < c.high_sigma_ratio
            sigma = torch.where(pick, rand().type_as(sigma) * 1920 + 80, sigma)
        elif strat == HighSigmaStrategy.BALANCED_TWO_HEADS_V1.lower():
            pick = rand() < c.high_sigma_ratio
            sigma = torch.where(pick, (rand().type_as(sigma) * (log_hi - log_lo) + log_lo).exp(), sigma)
            low = rand() < c.low_sigma_ratio
            sigma = torch.where(low, rand().type_as(sigma) * 2.0 + 0.00001, sigma)
        elif strat == HighSigmaStrategy.HARDCODED_20steps.lower():
            grid = torch.cat([torch.tensor([100000.0]), torch.as_tensor(get_rev_ts(self.sde.sigma_min, self.sde.sigma_max, 20, 7.0)).float()])
            sigma = grid[torch.randint(0, len(grid), sigma.shape)].type_as(sigma)
        else:
            raise ValueError(f"High sigma strategy {strat} is not supported")
        return sigma

    def denoise_edm(self, xt, sigma, condition):
        """x0 prediction with conditioning frames (video2world_model.py:168-247 of the reference): their clean latents, divided by
        sigma_data (and zeroed when the sample's video-condition flag is off), replace the scaled noisy input; their noise
        conditioning is c_noise(sigma_conditional); with ``denoise_replace_gt_frames`` their prediction is the clean latent."""
        if condition.data_type != DataType.VIDEO or getattr(condition, "gt_frames", None) is None:
            return super().denoise_edm(xt, sigma, condition)
        B, C, T = xt.shape[:3]
        xt = xt.float()
        sig = sigma.view(B, 1, -1, 1, 1).float() if sigma.ndim == 2 else sigma.view(B, 1, 1, 1, 1).float()
        c_skip, c_out, c_in, c_noise = self.scaling(sig)
        mask = condition.condition_video_input_mask_B_C_T_H_W.type_as(xt)
        gt = condition.gt_frames.type_as(xt)
        keep = gt / self.config.sigma_data * Video2WorldModelRectifiedFlow._use_flags(condition, B, xt)
        net_in = keep * mask + xt * c_in * (1 - mask)
        c_noise_cond = self.scaling(torch.ones_like(sig) * self.config.sigma_conditional)[3]
        m_T = mask.mean(dim=[1, 3, 4], keepdim=True)
        c_noise = c_noise_cond * m_T + c_noise * (1 - m_T)
        net_out = self.net(net_in.to(**self.tensor_kwargs), c_noise.expand(B, 1, T, 1, 1).reshape(B, T),
                           condition_video_input_mask_B_C_T_H_W=mask, **self._net_kwargs(condition)).float()
        x0 = c_skip * xt + c_out * net_out
        if self.config.denoise_replace_gt_frames:
            x0 = gt * mask + x0 * (1 - mask)
        return x0

    def _prepare_sampling_conditions(self, data_batch, cond, uncond):
        n = data_batch.get(NUM_CONDITIONAL_FRAMES_KEY, 1)
        _, x0, _ = DiffusionModel.get_data_and_condition(self, data_batch)
        x0 = x0.to(**self.tensor_kwargs)
        cond = cond.set_video_condition(x0, 0, 0, num_conditional_frames=n).edit_for_inference(True, n)
        uncond = uncond.set_video_condition(x0, 0, 0, num_conditional_frames=n).edit_for_inference(False, n)
        return cond, uncond

    def denoise_with_velocity(self, xt: torch.Tensor, t: torch.Tensor, condition) -> torch.Tensor:
        """Adapter that lets the flow solvers drive an EDM model: sigma = t / (1 - t), x_sigma = x_t (1 + sigma),
        velocity = eps_hat - x0_hat."""
        sigma = t / (1 - t).clamp_min(1e-6)
        x_sigma = xt * (1 + sigma.view(-1, 1, 1, 1, 1))
        x0 = self.denoise_edm(x_sigma, sigma, condition)
        eps = (x_sigma - x0) / sigma.view(-1, 1, 1, 1, 1)
        return eps - x0
