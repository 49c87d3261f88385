"""Continuous-time consistency distillation (sCM) with score regularisation (rCM) of the rectified-flow DiT.

The reference ships only the attention JVP kernel this needs (cosmos_predict2/_src/predict2/utils/flash_attention_jvp_triton.py)
and no trainer; the algorithm below follows the published methods (sCM: continuous-time consistency models with tangent
normalisation and warm-up; rCM: the same objective plus a distribution-matching term driven by a frozen teacher and an
online "fake score" network), written for the rectified-flow parameterisation used by this model family:

    x_t = (1 - t) x0 + t eps,   v = eps - x0,   student velocity F = v_theta(x_t, t),   f_theta(x_t, t) = x_t - t F  (-> x0)

* The time derivative of the consistency function along the teacher's probability-flow ODE (dx_t/dt = v_T) is
      df/dt = v_T - F - t dF/dt,      dF/dt = JVP of v_theta- at (x_t, t) with tangents (v_T, 1)
  and the gradient of the continuous-time consistency loss is <d_theta f, w df/dt> = -t <d_theta F, w df/dt>. It is
  realised by the surrogate  || F_theta - sg(F_theta- - g) ||^2  with  g = -t df/dt, tangent warm-up r on the dF/dt term
  and normalisation g / (||g|| + c).
* The JVP runs in forward mode through the whole network: plain torch operators carry the tangents and attention uses the
  sm_100a JVP kernel through a function with a JVP rule (``ops.functional._FlashAttentionJVP``).
* rCM: a few-step sample of the student is re-noised to a random time s; the difference between the fake-score network's
  and the teacher's velocity at (x_s, s) is the (stop-gradient) direction that moves the student's sample distribution
  towards the teacher's (reverse KL). The fake-score network is trained with the ordinary flow-matching loss on student
  samples, alternating with the student.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.autograd.forward_ad as fwAD
import torch.nn as nn

from ..ops import native
from .conditioner import DataType
from .rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig


def network_jvp(net: nn.Module, x: torch.Tensor, timesteps_B_T: torch.Tensor, tx: torch.Tensor, tt: torch.Tensor,
                **net_kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
    """(F, dF) = value and directional derivative of ``net(x, timesteps, ...)`` along (tx, tt). No parameter gradients."""
    with torch.no_grad(), native.forward_mode_ad(), fwAD.dual_level():
        xd = fwAD.make_dual(x, tx.to(x.dtype))
        td = fwAD.make_dual(timesteps_B_T, tt.to(timesteps_B_T.dtype))
        out = net(xd, td, **net_kwargs)
        F, dF = fwAD.unpack_dual(out)
        if dF is None:
            dF = torch.zeros_like(F)
    return F.detach(), dF.detach()


@dataclass
class DistillConfig(Video2WorldRFConfig):
    student_sample_steps: int = 4                # few-step sampler of the student (times t_max -> 0)
    t_max: float = 0.999
    t_min: float = 0.001
    teacher_guidance: float = 0.0                # classifier-free guidance folded into the teacher velocity (0 = conditional only)
    tangent_warmup_iters: int = 1000             # r ramps 0 -> 1
    tangent_norm_c: float = 0.1
    scm_weight: float = 1.0
    dmd_weight: float = 0.0                      # > 0 switches the rCM regulariser (and the fake-score network) on
    critic_every: int = 1                        # fake-score updates per student update
    p_mean: float = 0.0                          # logit-normal time sampling for the consistency loss
    p_std: float = 1.6
    use_jvp: bool = True                         # False: finite difference along the ODE (for tests / debugging)
    fd_eps: float = 1e-3


class ConsistencyDistillModel(Video2WorldModelRectifiedFlow):
    """Student = ``self.net`` (initialised from the teacher); ``self.teacher`` frozen; ``self.fake_score`` optional."""

    def __init__(self, config: DistillConfig, **kw):
        super().__init__(config, **kw)
        # the teacher is frozen and never enters the sharded engine: it is held in the compute precision
        self.teacher = copy.deepcopy(self.net).requires_grad_(False).eval().to(self.precision)
        self.fake_score = copy.deepcopy(self.net) if config.dmd_weight > 0 else None
        self._phase = "student"

    # the teacher never trains; keep it out of the sharded engine's view of trainable parameters
    def train(self, mode: bool = True):
        super().train(mode)
        self.teacher.eval()
        return self

    def load_teacher_state_dict(self, sd: Dict[str, torch.Tensor], also_student: bool = True):
        sd = {k[len("net."):] if k.startswith("net.") else k: v for k, v in sd.items() if not k.startswith("net_ema.")}
        self.teacher.load_state_dict(sd, strict=False)
        if also_student:
            self.net.load_state_dict(sd, strict=False)
            if self.fake_score is not None:
                self.fake_score.load_state_dict(sd, strict=False)

    # ---- pieces --------------------------------------------------------------------------------------------------
    def _net_call(self, net, xt, t_B1, condition, mask_gt: bool = True):
        """Velocity of ``net`` at (x_t, t in [0,1]) with the video conditioning of ``denoise`` (frame replacement, mask input)."""
        cfg = self.config
        kw = self._net_kwargs(condition)
        x_in = xt
        mask = None
        if condition.data_type == DataType.VIDEO and getattr(condition, "gt_frames", None) is not None:
            mask = condition.condition_video_input_mask_B_C_T_H_W.type_as(xt)
            x_in = condition.gt_frames.type_as(xt) * mask + xt * (1 - mask)
        return net(x_in.to(**self.tensor_kwargs), t_B1 * 1000.0, condition_video_input_mask_B_C_T_H_W=mask, **kw).float(), mask

    def teacher_velocity(self, xt, t_B1, condition, uncondition=None):
        with torch.no_grad():
            v, _ = self._net_call(self.teacher, xt, t_B1, condition)
            g = self.config.teacher_guidance
            if g > 0 and uncondition is not None:
                vu, _ = self._net_call(self.teacher, xt, t_B1, uncondition)
                v = v + g * (v - vu)
        return v

    def student_jvp(self, xt, t_B1, v_teacher, condition):
        """F- and dF-/dt along the teacher ODE, through the student network with stop-gradient weights."""
        kw = self._net_kwargs(condition)
        mask = None
        x_in, tx = xt, v_teacher
        if condition.data_type == DataType.VIDEO and getattr(condition, "gt_frames", None) is not None:
            mask = condition.condition_video_input_mask_B_C_T_H_W.type_as(xt)
            x_in = condition.gt_frames.type_as(xt) * mask + xt * (1 - mask)
            tx = v_teacher * (1 - mask)                    # conditioning frames do not move
        if self.config.use_jvp:
            F, dF = network_jvp(self.net, x_in.to(**self.tensor_kwargs), t_B1 * 1000.0, tx.to(**self.tensor_kwargs),
                                torch.full_like(t_B1, 1000.0), condition_video_input_mask_B_C_T_H_W=mask, **kw)
            return F.float(), dF.float()
        with torch.no_grad():                               # central difference along (v_T, 1)
            e = self.config.fd_eps
            call = lambda dx, dt: self.net((x_in + dx * tx).to(**self.tensor_kwargs), (t_B1 + dt) * 1000.0,
                                           condition_video_input_mask_B_C_T_H_W=mask, **kw).float()
            F = call(0.0, 0.0)
            dF = (call(e, e) - call(-e, -e)) / (2 * e)
        return F, dF

    def sample_consistency_time(self, B: int) -> torch.Tensor:
        c = self.config
        u = torch.randn(B) * c.p_std + c.p_mean
        return torch.sigmoid(u).clamp(c.t_min, c.t_max)

    def tangent_warmup(self, iteration: int) -> float:
        n = self.config.tangent_warmup_iters
        return 1.0 if n <= 0 else min(1.0, iteration / n)

    # ---- losses ------------------------------------------------------------------------------------------------------
    def scm_loss(self, x0, eps, t_B, condition, uncondition, iteration: int):
        B = x0.shape[0]
        t5 = t_B.view(B, 1, 1, 1, 1)
        t_B1 = t_B.view(B, 1)
        xt = (1 - t5) * x0 + t5 * eps
        v_T = self.teacher_velocity(xt, t_B1, condition, uncondition)
        F_minus, dF = self.student_jvp(xt, t_B1, v_T, condition)
        r = self.tangent_warmup(iteration)
        dfdt = v_T - F_minus - r * t5 * dF
        g = -t5 * dfdt
        norm = g.flatten(1).norm(dim=1).view(B, 1, 1, 1, 1) / math.sqrt(g[0].numel())     # RMS per sample
        g = g / (norm + self.config.tangent_norm_c)
        F, mask = self._net_call(self.net, xt, t_B1, condition)
        target = (F_minus - g).detach()
        w = 1.0 if mask is None else (1 - mask)
        per = ((F - target) ** 2 * w).mean(dim=list(range(1, F.ndim)))
        return per.mean(), {"scm/tangent_rms": norm.mean().detach(), "scm/warmup": torch.tensor(r)}

    @torch.no_grad()
    def student_times(self) -> List[float]:
        n = self.config.student_sample_steps
        return [self.config.t_max * (1 - i / n) for i in range(n)] + [0.0]

    def student_sample(self, noise, condition, grad_last: bool = False):
        """Few-step consistency sampling: x0 = f(x_t, t); re-noise to the next time with fresh noise."""
        ts = self.student_times()
        x = noise
        B = noise.shape[0]
        x0 = None
        for i, t in enumerate(ts[:-1]):
            last = i == len(ts) - 2
            t_B1 = torch.full((B, 1), t, device=noise.device, dtype=torch.float32)
            with torch.set_grad_enabled(grad_last and last):
                F, mask = self._net_call(self.net, x, t_B1, condition)
                x0 = x - t * F
                if mask is not None:
                    x0 = condition.gt_frames.type_as(x0) * mask + x0 * (1 - mask)
            if not last:
                tn = ts[i + 1]
                x = (1 - tn) * x0.detach() + tn * torch.randn_like(x0)
        return x0

    def dmd_loss(self, x_gen, condition, uncondition):
        """Distribution matching: gradient direction (v_fake - v_teacher) at a re-noised student sample, stop-gradient."""
        B = x_gen.shape[0]
        s = torch.rand(B, device=x_gen.device).clamp(0.02, 0.98)
        s5, s_B1 = s.view(B, 1, 1, 1, 1), s.view(B, 1)
        eps = torch.randn_like(x_gen)
        xs = (1 - s5) * x_gen.detach() + s5 * eps
        with torch.no_grad():
            v_real = self.teacher_velocity(xs, s_B1, condition, uncondition)
            v_fake, _ = self._net_call(self.fake_score, xs, s_B1, condition)
            # x0 estimates of both score models; their difference is the reverse-KL gradient w.r.t. the sample
            x0_real, x0_fake = xs - s5 * v_real, xs - s5 * v_fake
            grad = x0_fake - x0_real
            grad = grad / (x_gen.detach() - x0_real).abs().mean(dim=list(range(1, x_gen.ndim)), keepdim=True).clamp_min(1e-4)
        return 0.5 * ((x_gen - (x_gen - grad).detach()) ** 2).mean()

    def critic_loss(self, x_gen, condition):
        """Flow matching of the fake-score network on (detached) student samples."""
        B = x_gen.shape[0]
        s = torch.rand(B, device=x_gen.device).clamp(0.001, 0.999)
        s5 = s.view(B, 1, 1, 1, 1)
        eps = torch.randn_like(x_gen)
        xs = (1 - s5) * x_gen.detach() + s5 * eps
        v, mask = self._net_call(self.fake_score, xs, s.view(B, 1), condition)
        w = 1.0 if mask is None else (1 - mask)
        return (((v - (eps - x_gen.detach())) ** 2) * w).mean()

    # ---- training step -----------------------------------------------------------------------------------------------------
    def set_phase(self, phase: str):
        assert phase in ("student", "critic")
        self._phase = phase

    def training_step(self, data_batch: Dict, iteration: int):
        cfg = self.config
        _, x0, condition = self.get_data_and_condition(data_batch)
        uncondition = None
        if cfg.teacher_guidance > 0:
            _, uncondition = self._conditions_for_sampling(data_batch, is_negative_prompt=False)
            from dataclasses import replace
            uncondition = replace(uncondition, gt_frames=condition.gt_frames,
                                  condition_video_input_mask_B_C_T_H_W=condition.condition_video_input_mask_B_C_T_H_W)
        B = x0.shape[0]
        eps = torch.randn_like(x0)
        t_B = self.sample_consistency_time(B).to(**self.tensor_kwargs_fp32)
        x0, condition, eps, t_B = self.broadcast_split_for_model_parallelsim(x0, condition, eps, t_B)
        out: Dict[str, Any] = {}
        if self._phase == "critic" and self.fake_score is not None:
            with torch.no_grad():
                x_gen = self.student_sample(torch.randn_like(x0), condition)
            loss = self.critic_loss(x_gen, condition)
            out["critic_loss"] = loss.detach()
            return out, loss
        loss, info = self.scm_loss(x0, eps, t_B, condition, uncondition, iteration)
        out.update(info)
        out["scm_loss"] = loss.detach()
        loss = cfg.scm_weight * loss
        if self.fake_score is not None and cfg.dmd_weight > 0:
            x_gen = self.student_sample(torch.randn_like(x0), condition, grad_last=True)
            dmd = self.dmd_loss(x_gen, condition, uncondition)
            out["dmd_loss"] = dmd.detach()
            loss = loss + cfg.dmd_weight * dmd
        out["edm_loss"] = loss.detach()
        return out, loss

    # ---- few-step generation with the distilled student ------------------------------------------------------------------------
    @torch.no_grad()
    def generate_samples_from_batch(self, data_batch: Dict, guidance: float = 0.0, seed: int = 1, state_shape=None, n_sample=None,
                                    is_negative_prompt: bool = False, num_steps: Optional[int] = None, **kw) -> torch.Tensor:
        from ..utils.misc import arch_invariant_rand
        self._normalize_video_databatch_inplace(data_batch)
        self._augment_image_dim_inplace(data_batch)
        _, x0, condition = self.get_data_and_condition(data_batch)
        n = data_batch.get("num_conditional_frames", 1)
        condition = condition.set_video_condition(x0.to(**self.tensor_kwargs), 0, 0, num_conditional_frames=n)
        shape = (n_sample or x0.shape[0],) + tuple(state_shape or x0.shape[1:])
        noise = arch_invariant_rand(shape, torch.float32, self.device_, seed)
        if num_steps is not None:
            old, self.config.student_sample_steps = self.config.student_sample_steps, num_steps
        try:
            torch.manual_seed(seed)
            return self.student_sample(noise, condition)
        finally:
            if num_steps is not None:
                self.config.student_sample_steps = old


class DistillTrainerMixin:
    """Alternation schedule used by the training loop: ``critic_every`` fake-score steps after each student step. The two
    networks keep separate sharded engines / optimizers; the trainer calls ``model.set_phase`` before each step."""

    @staticmethod
    def phase_of(iteration: int, critic_every: int, has_critic: bool) -> str:
        if not has_critic or critic_every <= 0:
            return "student"
        return "student" if iteration % (critic_every + 1) == 0 else "critic"
