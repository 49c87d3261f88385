"""Plain-PyTorch oracle for every fused op of the framework.

Each function states the math of one kernel in the simplest possible form, in the
dtype of its inputs (tests call them in fp32). They are the CPU execution path and
the numerical reference the CUDA kernels are compared against.

Reference semantics these restate:
  * AdaLN layer-norm + modulate and the gated residual:
    cosmos_predict2/_src/predict2/networks/minimal_v4_dit.py:1166-1241
  * per-head RMSNorm followed by rotate-half RoPE on q and k:
    cosmos_predict2/_src/predict2/networks/minimal_v4_dit.py:395-419
  * attention contract ([B,S,H,D] in and out, non-causal):
    cosmos_predict2/_src/predict2/networks/attention.py:90-181
  * forward-mode (JVP) attention contract:
    cosmos_predict2/_src/predict2/utils/flash_attention_jvp_triton.py:176-378
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def ln_modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """LayerNorm over the last dim (no affine) then ``*(1+scale)+shift``.

    x: [B, T, L, D]; shift, scale: [B, T, D] (one vector per latent frame).
    """
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = xf.var(-1, unbiased=False, keepdim=True)
    xhat = (xf - mean) * torch.rsqrt(var + eps)
    out = xhat * (1.0 + scale.float().unsqueeze(2)) + shift.float().unsqueeze(2)
    return out.to(x.dtype)


def gate_residual(x: torch.Tensor, gate: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """``x + gate * y`` with gate [B, T, D] broadcast over the L tokens of each frame."""
    return (x.float() + gate.float().unsqueeze(2) * y.float()).to(x.dtype)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    out = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return out.to(x.dtype)


def rope_rotate_half(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """Non-interleaved rotary embedding. x: [B, S, H, D]; angles: [S, D] (fp32)."""
    xf = x.float()
    d = xf.shape[-1] // 2
    rot = torch.cat([-xf[..., d:], xf[..., :d]], dim=-1)
    cos = angles.cos()[None, :, None, :]
    sin = angles.sin()[None, :, None, :]
    return (xf * cos + rot * sin).to(x.dtype)


def rmsnorm_rope(x: torch.Tensor, weight: torch.Tensor, angles: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    """Per-head RMSNorm (learnable [D]) and, when ``angles`` is given, rotate-half RoPE.

    The norm output is kept in fp32 through the rotation (the q/k fp32 up-cast of the
    reference's ``use_wan_fp32_strategy``).
    """
    xf = x.float()
    out = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    if angles is not None:
        d = out.shape[-1] // 2
        rot = torch.cat([-out[..., d:], out[..., :d]], dim=-1)
        out = out * angles.cos()[None, :, None, :] + rot * angles.sin()[None, :, None, :]
    return out.to(x.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
              causal: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax(q k^T * scale) v with [B, S, H, D] layout. Returns (out, lse[B,H,Sq])."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        sq, sk = s.shape[-2:]
        mask = torch.ones(sq, sk, dtype=torch.bool, device=s.device).tril(sk - sq)
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.matmul(p, vf).transpose(1, 2)
    return o.to(q.dtype), lse


def attention_jvp(q, k, v, tq, tk, tv, scale: Optional[float] = None, causal: bool = False):
    """Primal and tangent of attention in closed form.

    With P = softmax(S), S = q k^T * scale and tS = (tq k^T + q tk^T) * scale:
    tO = P tV + (P * tS) V - rowsum(P * tS) * O.  Layout [B, S, H, D]. Returns (o, to, lse).
    """
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    qf, kf, vf, tqf, tkf, tvf = (t.float().transpose(1, 2) for t in (q, k, v, tq, tk, tv))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    ts = (torch.matmul(tqf, kf.transpose(-1, -2)) + torch.matmul(qf, tkf.transpose(-1, -2))) * scale
    if causal:
        sq, sk = s.shape[-2:]
        mask = torch.ones(sq, sk, dtype=torch.bool, device=s.device).tril(sk - sq)
        s = s.masked_fill(~mask, float("-inf"))
        ts = ts.masked_fill(~mask, 0.0)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.matmul(p, vf)
    pts = p * ts
    to = torch.matmul(p, tvf) + torch.matmul(pts, vf) - pts.sum(-1, keepdim=True) * o
    return o.transpose(1, 2).to(q.dtype), to.transpose(1, 2).to(q.dtype), lse


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none") -> torch.Tensor:
    """``act(x @ w.T + bias)`` with fp32 accumulation; act in {none, gelu}. GELU is the exact erf form."""
    y = F.linear(x.float(), w.float(), None if bias is None else bias.float())
    if act == "gelu":
        y = F.gelu(y)
    elif act != "none":
        raise ValueError(act)
    return y.to(x.dtype)


def adamw_step(param_master, grad, exp_avg, exp_avg_sq, *, lr, beta1, beta2, eps, weight_decay, step,
               grad_scale: float = 1.0):
    """One decoupled-weight-decay Adam step on fp32 tensors (in place). Mirrors torch.optim.AdamW."""
    g = torch.nan_to_num(grad.float() * grad_scale, nan=0.0, posinf=0.0, neginf=0.0)
    param_master.mul_(1.0 - lr * weight_decay)
    exp_avg.mul_(beta1).add_(g, alpha=1.0 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (exp_avg_sq.sqrt() / math.sqrt(bc2)).add_(eps)
    param_master.addcdiv_(exp_avg, denom, value=-lr / bc1)
    return param_master


def cfg_combine(cond: torch.Tensor, uncond: torch.Tensor, guidance: float) -> torch.Tensor:
    """Video2World guidance: ``cond + g * (cond - uncond)``."""
    return cond + guidance * (cond - uncond)


def lincomb(xs, coeffs) -> torch.Tensor:
    """``sum_k coeffs[k] * xs[k]`` in the dtype of ``xs[0]``."""
    out = coeffs[0] * xs[0]
    for c, x in zip(coeffs[1:], xs[1:]):
        out = out + c * x.to(out.dtype)
    return out


def frame_blend(x, gt, noise, mask, flag=None, out_dtype=None) -> torch.Tensor:
    """``keep * mask + x * (1 - mask)``; ``keep = gt * flag`` (``noise`` is None) or ``noise - gt``. ``mask`` broadcasts over the
    channels, ``flag`` ([B]) over everything but the batch."""
    if noise is not None:
        keep = noise - gt
    else:
        keep = gt if flag is None else gt * flag.view(-1, *([1] * (gt.dim() - 1))).to(gt.dtype)
    m = mask.to(x.dtype)
    out = keep.to(x.dtype) * m + x * (1 - m)
    return out if out_dtype is None else out.to(out_dtype)


def causal_conv3d(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], cache: Optional[torch.Tensor] = None):
    """3-D conv that pads (or prepends ``cache`` frames) on the past side of time only.

    x: [B, C, T, H, W]; w: [O, C, kt, kh, kw]; spatial padding is symmetric (k//2).
    """
    kt, kh, kw = w.shape[2:]
    pad_t = kt - 1
    if cache is not None and pad_t > 0:
        x = torch.cat([cache.to(x.dtype), x], dim=2)
        pad_t -= cache.shape[2]
    x = F.pad(x, (kw // 2, kw // 2, kh // 2, kh // 2, max(pad_t, 0), 0))
    return F.conv3d(x, w, b)
