"""Wan2.1 text-to-video / image-to-video DiT and its rectified-flow fine-tuning model.

Parity targets: ``WanModel`` and parts (cosmos_predict2/_src/predict2/networks/wan2pt1.py:104-1014: 3-D rotary table,
interleaved RoPE ``rope_apply`` :214, full-width q/k RMSNorm, ``WanSelfAttention`` :291, T2V / I2V cross-attention :387/:410,
six-way learned modulation added to the projected timestep, ``Head`` :579, ``MLPProj`` :616),
``WANDiffusionModel`` (cosmos_predict2/_src/predict2/models/text2world_wan2pt1_model.py:89-760) and ``I2VWan2pt1Model``
(cosmos_predict2/_src/predict2/models/video2world_wan2pt1_model.py:31-60). Parameter names follow the Wan checkpoints.

Attention runs through this package's attention front-end (tcgen05 flash attention on B200); the context-parallel path is
the same Ulysses exchange the Cosmos DiT uses (the reference's ring / a2a choice collapses to all-to-all).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from ..parallel import ulysses
from .conditioner import DataType
from .dit import register_training_stats
from .rectified_flow import Text2WorldModelRectifiedFlow, Text2WorldRFConfig

T5_CONTEXT_TOKEN_NUMBER = 512
FIRST_LAST_FRAME_CONTEXT_TOKEN_NUMBER = 257 * 2
WAN2PT1_I2V_COND_LATENT_KEY = "i2v_WAN2PT1_cond_latents"


@dataclass
class WanConfig:
    model_type: str = "t2v"            # t2v | i2v | flf2v
    patch_size: Tuple[int, int, int] = (1, 2, 2)
    text_len: int = 512
    in_dim: int = 16
    dim: int = 2048
    ffn_dim: int = 8192
    freq_dim: int = 256
    text_dim: int = 4096
    out_dim: int = 16
    num_heads: int = 16
    num_layers: int = 32
    qk_norm: bool = True
    cross_attn_norm: bool = True
    eps: float = 1e-6
    concat_padding_mask: bool = False
    checkpoint_mode: str = "none"

    @property
    def head_dim(self) -> int:
        return self.dim // self.num_heads


def sinusoidal_embedding_1d(dim: int, position: torch.Tensor) -> torch.Tensor:
    half = dim // 2
    pos = position.to(torch.float64)
    s = torch.outer(pos, torch.pow(10000, -torch.arange(half, device=pos.device, dtype=torch.float64) / half))
    return torch.cat([torch.cos(s), torch.sin(s)], dim=1)


class WanRope3D(nn.Module):
    """Angles [T*H*W, head_dim/2] = cat(t, h, w) with head_dim split (d - 2*(d//6*2), d//6*2, d//6*2)."""

    def __init__(self, head_dim: int, len_h: int = 128, len_w: int = 128, len_t: int = 32):
        super().__init__()
        self.max_h, self.max_w, self.max_t = len_h, len_w, len_t
        self.dim_h = head_dim // 6 * 2
        self.dim_t = head_dim - 2 * self.dim_h

    def generate(self, T: int, H: int, W: int, device, t_offset: int = 0) -> torch.Tensor:
        assert H <= self.max_h and W <= self.max_w, (H, W)
        sr = torch.arange(0, self.dim_h, 2, device=device)[: self.dim_h // 2].float() / self.dim_h
        tr = torch.arange(0, self.dim_t, 2, device=device)[: self.dim_t // 2].float() / self.dim_t
        fs, ft = 1.0 / (10000.0 ** sr), 1.0 / (10000.0 ** tr)
        seq = torch.arange(max(H, W, t_offset + T), device=device).float()
        e_t = torch.outer(seq[t_offset:t_offset + T], ft)[:, None, None, :].expand(T, H, W, -1)
        e_h = torch.outer(seq[:H], fs)[None, :, None, :].expand(T, H, W, -1)
        e_w = torch.outer(seq[:W], fs)[None, None, :, :].expand(T, H, W, -1)
        return torch.cat([e_t, e_h, e_w], dim=-1).reshape(T * H * W, -1).float()


def rope_apply_interleaved(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """Rotate pairs (2i, 2i+1) of the head dim by ``angles[s, i]``; x [B,S,H,D], fp32 math."""
    B, S, H, D = x.shape
    xf = x.float().view(B, S, H, D // 2, 2)
    c, s = angles.cos()[None, :, None, :], angles.sin()[None, :, None, :]
    a, b = xf[..., 0], xf[..., 1]
    return torch.stack([a * c - b * s, a * s + b * c], dim=-1).view(B, S, H, D).to(x.dtype)


class WanRMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def reset_parameters(self):
        nn.init.ones_(self.weight)

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x) * self.weight.to(x.dtype)


class WanLayerNorm(nn.LayerNorm):
    def __init__(self, dim, eps=1e-6, elementwise_affine=False):
        super().__init__(dim, elementwise_affine=elementwise_affine, eps=eps)

    def forward(self, x):
        w = None if self.weight is None else self.weight.float()
        b = None if self.bias is None else self.bias.float()
        return F.layer_norm(x.float(), self.normalized_shape, w, b, self.eps).type_as(x)


def _lin(x: torch.Tensor, m: nn.Linear, act: str = "none") -> torch.Tensor:
    return ops.linear(x, m.weight, m.bias, act)


class WanSelfAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, qk_norm: bool = True, eps: float = 1e-6):
        super().__init__()
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.q, self.k, self.v, self.o = (nn.Linear(dim, dim) for _ in range(4))
        self.norm_q = WanRMSNorm(dim, eps) if qk_norm else nn.Identity()
        self.norm_k = WanRMSNorm(dim, eps) if qk_norm else nn.Identity()
        self.cp_group = None

    def init_weights(self):
        std = 1.0 / math.sqrt(self.dim)
        for m in (self.q, self.k, self.v, self.o):
            nn.init.trunc_normal_(m.weight, std=std)
            nn.init.zeros_(m.bias)
        for n in (self.norm_q, self.norm_k):
            if isinstance(n, WanRMSNorm):
                n.reset_parameters()

    def forward(self, x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
        B, S, _ = x.shape
        n, d = self.num_heads, self.head_dim
        q = rope_apply_interleaved(self.norm_q(_lin(x, self.q)).view(B, S, n, d), angles)
        k = rope_apply_interleaved(self.norm_k(_lin(x, self.k)).view(B, S, n, d), angles)
        v = _lin(x, self.v).view(B, S, n, d)
        if self.cp_group is not None:
            o = ulysses.ulysses_attention(q, k, v, self.cp_group)
        else:
            o = ops.attention(q, k, v)
        return _lin(o.reshape(B, S, n * d), self.o)


class WanT2VCrossAttention(WanSelfAttention):
    def forward(self, x: torch.Tensor, context: torch.Tensor) -> torch.Tensor:
        B, n, d = x.shape[0], self.num_heads, self.head_dim
        q = self.norm_q(_lin(x, self.q)).view(B, -1, n, d)
        k = self.norm_k(_lin(context, self.k)).view(B, -1, n, d)
        v = _lin(context, self.v).view(B, -1, n, d)
        return _lin(ops.attention(q, k, v).flatten(2), self.o)


class WanI2VCrossAttention(WanSelfAttention):
    """Text and CLIP-image contexts attend separately (own K/V projections for the image tokens) and are summed."""

    def __init__(self, dim, num_heads, qk_norm=True, eps=1e-6):
        super().__init__(dim, num_heads, qk_norm, eps)
        self.k_img, self.v_img = nn.Linear(dim, dim), nn.Linear(dim, dim)
        self.norm_k_img = WanRMSNorm(dim, eps) if qk_norm else nn.Identity()

    def init_weights(self):
        super().init_weights()
        std = 1.0 / math.sqrt(self.dim)
        for m in (self.k_img, self.v_img):
            nn.init.trunc_normal_(m.weight, std=std)
            nn.init.zeros_(m.bias)
        if isinstance(self.norm_k_img, WanRMSNorm):
            self.norm_k_img.reset_parameters()

    def forward(self, x: torch.Tensor, context: torch.Tensor) -> torch.Tensor:
        n_img = context.shape[1] - T5_CONTEXT_TOKEN_NUMBER
        ctx_img, ctx = context[:, :n_img], context[:, n_img:]
        B, n, d = x.shape[0], self.num_heads, self.head_dim
        q = self.norm_q(_lin(x, self.q)).view(B, -1, n, d)
        k = self.norm_k(_lin(ctx, self.k)).view(B, -1, n, d)
        v = _lin(ctx, self.v).view(B, -1, n, d)
        k_img = self.norm_k_img(_lin(ctx_img, self.k_img)).view(B, -1, n, d)
        v_img = _lin(ctx_img, self.v_img).view(B, -1, n, d)
        out = ops.attention(q, k, v).flatten(2) + ops.attention(q, k_img, v_img).flatten(2)
        return _lin(out, self.o)


class WanAttentionBlock(nn.Module):
    def __init__(self, cfg: WanConfig):
        super().__init__()
        dim = cfg.dim
        self.dim = dim
        self.norm1 = WanLayerNorm(dim, cfg.eps)
        self.self_attn = WanSelfAttention(dim, cfg.num_heads, cfg.qk_norm, cfg.eps)
        self.norm3 = WanLayerNorm(dim, cfg.eps, elementwise_affine=True) if cfg.cross_attn_norm else nn.Identity()
        cross = WanT2VCrossAttention if cfg.model_type == "t2v" else WanI2VCrossAttention
        self.cross_attn = cross(dim, cfg.num_heads, cfg.qk_norm, cfg.eps)
        self.norm2 = WanLayerNorm(dim, cfg.eps)
        self.ffn = nn.Sequential(nn.Linear(dim, cfg.ffn_dim), nn.GELU(approximate="tanh"), nn.Linear(cfg.ffn_dim, dim))
        self.modulation = nn.Parameter(torch.randn(1, 6, dim) / dim ** 0.5)

    def init_weights(self):
        self.self_attn.init_weights()
        self.cross_attn.init_weights()
        for n in (self.norm1, self.norm2, self.norm3):
            if isinstance(n, nn.LayerNorm) and n.elementwise_affine:
                n.reset_parameters()
        nn.init.trunc_normal_(self.modulation, std=1.0 / math.sqrt(self.dim))
        for m in (self.ffn[0], self.ffn[2]):
            nn.init.trunc_normal_(m.weight, std=1.0 / math.sqrt(m.in_features))
            nn.init.zeros_(m.bias)

    def forward(self, x: torch.Tensor, e: torch.Tensor, angles: torch.Tensor, context: torch.Tensor) -> torch.Tensor:
        """x [B,L,C]; e [B,6,C] fp32."""
        e0, e1, e2, e3, e4, e5 = (self.modulation.float() + e.float()).chunk(6, dim=1)
        y = self.self_attn((self.norm1(x).float() * (1 + e1) + e0).type_as(x), angles)
        x = (x.float() + y.float() * e2).type_as(x)
        x = x + self.cross_attn(self.norm3(x), context)
        h = (self.norm2(x).float() * (1 + e4) + e3).type_as(x)
        y = self.ffn[2](F.gelu(self.ffn[0](h), approximate="tanh"))
        return (x.float() + y.float() * e5).type_as(x)


class WanHead(nn.Module):
    def __init__(self, dim: int, out_dim: int, patch_size, eps: float = 1e-6):
        super().__init__()
        self.dim = dim
        self.norm = WanLayerNorm(dim, eps)
        self.head = nn.Linear(dim, math.prod(patch_size) * out_dim)
        self.modulation = nn.Parameter(torch.randn(1, 2, dim) / dim ** 0.5)

    def init_weights(self):
        std = 1.0 / math.sqrt(self.dim)
        nn.init.trunc_normal_(self.modulation, std=std)
        nn.init.trunc_normal_(self.head.weight, std=std)
        nn.init.zeros_(self.head.bias)

    def forward(self, x, e):
        e0, e1 = (self.modulation.float() + e.float().unsqueeze(1)).chunk(2, dim=1)
        h = self.norm(x).float() * (1 + e1) + e0
        return F.linear(h, self.head.weight.float(), self.head.bias.float())


class MLPProj(nn.Module):
    """CLIP image tokens (1280 wide) -> model width."""

    def __init__(self, in_dim: int, out_dim: int, flf_pos_emb: bool = False):
        super().__init__()
        self.proj = nn.Sequential(nn.LayerNorm(in_dim), nn.Linear(in_dim, in_dim), nn.GELU(), nn.Linear(in_dim, out_dim),
                                  nn.LayerNorm(out_dim))
        if flf_pos_emb:
            self.emb_pos = nn.Parameter(torch.zeros(1, FIRST_LAST_FRAME_CONTEXT_TOKEN_NUMBER, 1280))

    def init_weights(self):
        for i in (0, 1, 3, 4):
            self.proj[i].reset_parameters()
        if hasattr(self, "emb_pos"):
            self.emb_pos.data.zero_()

    def forward(self, image_embeds):
        if hasattr(self, "emb_pos"):
            bs, n, d = image_embeds.shape
            image_embeds = image_embeds.view(-1, 2 * n, d) + self.emb_pos
        return self.proj(image_embeds)


class WanModel(nn.Module):
    def __init__(self, cfg: WanConfig):
        super().__init__()
        assert cfg.model_type in ("t2v", "i2v", "flf2v")
        assert cfg.dim % cfg.num_heads == 0 and cfg.head_dim % 2 == 0
        self.cfg = cfg
        in_dim = cfg.in_dim + (1 if cfg.concat_padding_mask else 0)
        self.patch_embedding = nn.Linear(in_dim * math.prod(cfg.patch_size), cfg.dim)
        self.text_embedding = nn.Sequential(nn.Linear(cfg.text_dim, cfg.dim), nn.GELU(approximate="tanh"), nn.Linear(cfg.dim, cfg.dim))
        self.time_embedding = nn.Sequential(nn.Linear(cfg.freq_dim, cfg.dim), nn.SiLU(), nn.Linear(cfg.dim, cfg.dim))
        self.time_projection = nn.Sequential(nn.SiLU(), nn.Linear(cfg.dim, cfg.dim * 6))
        self.blocks = nn.ModuleList([WanAttentionBlock(cfg) for _ in range(cfg.num_layers)])
        self.head = WanHead(cfg.dim, cfg.out_dim, cfg.patch_size, cfg.eps)
        register_training_stats(self)
        self.rope_position_embedding = WanRope3D(cfg.head_dim)
        if cfg.model_type in ("i2v", "flf2v"):
            self.img_emb = MLPProj(1280, cfg.dim, flf_pos_emb=cfg.model_type == "flf2v")
        self.cp_group = None

    def init_weights(self):
        for m in (self.patch_embedding, self.text_embedding[0], self.text_embedding[2], self.time_embedding[0],
                  self.time_embedding[2], self.time_projection[1]):
            nn.init.trunc_normal_(m.weight, std=1.0 / math.sqrt(m.in_features))
            nn.init.zeros_(m.bias)
        for b in self.blocks:
            b.init_weights()
        self.head.init_weights()
        if hasattr(self, "img_emb"):
            self.img_emb.init_weights()

    def enable_context_parallel(self, group):
        self.cp_group = group
        for b in self.blocks:
            b.self_attn.cp_group = group

    def disable_context_parallel(self):
        self.enable_context_parallel(None)

    @property
    def is_context_parallel_enabled(self) -> bool:
        return self.cp_group is not None

    def fsdp_units(self):
        return list(self.blocks) + [self.head]

    def build_context_cache(self, crossattn_emb):     # interface parity with the Cosmos DiT; Wan re-projects each step
        return None

    def forward(self, x_B_C_T_H_W, timesteps_B_T, crossattn_emb, frame_cond_crossattn_emb_B_L_D=None, y_B_C_T_H_W=None,
                padding_mask=None, is_uncond: bool = False, slg_layers=None, **_unused):
        cfg = self.cfg
        t_B = timesteps_B_T.reshape(timesteps_B_T.shape[0], -1)[:, 0]
        if cfg.model_type in ("i2v", "flf2v"):
            assert frame_cond_crossattn_emb_B_L_D is not None and y_B_C_T_H_W is not None
        x = x_B_C_T_H_W
        if y_B_C_T_H_W is not None:
            x = torch.cat([x, y_B_C_T_H_W.to(x.dtype)], dim=1)
        if cfg.concat_padding_mask:
            B, _, T, H, W = x.shape
            pm = padding_mask.to(x.dtype)
            if pm.shape[-2:] != (H, W):
                pm = F.interpolate(pm, size=(H, W), mode="nearest")
            x = torch.cat([x, pm.view(B, 1, 1, H, W).expand(B, 1, T, H, W)], dim=1)
        B, C, T, H, W = x.shape
        kt, kh, kw = cfg.patch_size
        x = x.view(B, C, T // kt, kt, H // kh, kh, W // kw, kw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        Tt, Hh, Ww = T // kt, H // kh, W // kw
        x = x.reshape(B, Tt * Hh * Ww, C * kt * kh * kw)
        w = self.patch_embedding.weight
        x = F.linear(x.to(w.dtype), w, self.patch_embedding.bias)
        e = self.time_embedding(sinusoidal_embedding_1d(cfg.freq_dim, t_B).float().to(x.device).to(self.time_embedding[0].weight.dtype)).float()
        e0 = self.time_projection(e.to(self.time_projection[1].weight.dtype)).float().unflatten(1, (6, cfg.dim))
        ctx = self.text_embedding(crossattn_emb.to(w.dtype))
        if frame_cond_crossattn_emb_B_L_D is not None:
            ctx = torch.cat([self.img_emb(frame_cond_crossattn_emb_B_L_D.to(w.dtype)), ctx], dim=1)
        _, cp_rank = ulysses.group_size_rank(self.cp_group)
        angles = self.rope_position_embedding.generate(Tt, Hh, Ww, x.device, t_offset=cp_rank * Tt)
        from .checkpointing import run_block
        for i, block in enumerate(self.blocks):
            if slg_layers is not None and i in slg_layers and is_uncond:
                continue
            x = run_block(block, cfg.checkpoint_mode if self.training else "none", x, e0, angles, ctx)
        out = self.head(x, e)
        out = out.view(B, Tt, Hh, Ww, kt, kh, kw, cfg.out_dim).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return out.reshape(B, cfg.out_dim, Tt * kt, Hh * kh, Ww * kw)


# ---- size presets (Wan2.1 release configs) ---------------------------------------------------------------------------------
def wan_t2v_1p3b(**kw) -> WanConfig:
    return WanConfig(**{**dict(model_type="t2v", dim=1536, ffn_dim=8960, num_heads=12, num_layers=30), **kw})


def wan_t2v_14b(**kw) -> WanConfig:
    return WanConfig(**{**dict(model_type="t2v", dim=5120, ffn_dim=13824, num_heads=40, num_layers=40), **kw})


def wan_i2v_14b(**kw) -> WanConfig:
    return WanConfig(**{**dict(model_type="i2v", in_dim=36, dim=5120, ffn_dim=13824, num_heads=40, num_layers=40), **kw})


def wan_tiny(**kw) -> WanConfig:
    return WanConfig(**{**dict(dim=128, ffn_dim=256, num_heads=4, num_layers=2, text_dim=64, freq_dim=32), **kw})


# ---- models ---------------------------------------------------------------------------------------------------------------------
@dataclass
class WanRFConfig(Text2WorldRFConfig):
    net: WanConfig = field(default_factory=WanConfig)
    shift: float = 3.0


class WANDiffusionModel(Text2WorldModelRectifiedFlow):
    """Rectified-flow fine-tuning of Wan2.1: same schedule / loss / sampler as the Cosmos RF model, Wan network."""

    def build_net(self):
        net = WanModel(self.config.net).to(self.device_)
        net.init_weights()
        return net

    def _net_kwargs(self, condition) -> Dict:
        kw = {"crossattn_emb": condition.crossattn_emb.to(self.precision), "padding_mask": condition.padding_mask}
        for k in ("frame_cond_crossattn_emb_B_L_D", "y_B_C_T_H_W"):
            if getattr(condition, k, None) is not None:
                kw[k] = getattr(condition, k)
        return kw

    def _batched_cfg_fn(self, condition, uncondition, guidance: float, t2w_formula: bool):
        def velocity_fn(noise, noise_x, timestep):
            c = self.denoise(noise, noise_x, timestep, condition)
            u = self.denoise(noise, noise_x, timestep, uncondition)
            return u + guidance * (c - u)
        return velocity_fn


class I2VWan2pt1Model(WANDiffusionModel):
    """Image-to-video: the latent of (first frame, zeros...) plus a 4-channel frame mask enters as ``y``; CLIP tokens of
    the first frame enter the cross-attention."""

    def get_data_and_condition(self, batch: Dict):
        self._normalize_video_databatch_inplace(batch)
        self._augment_image_dim_inplace(batch)
        is_image = self.is_image_batch(batch)
        raw = batch[self.config.input_image_key if is_image else self.config.input_data_key]
        latent = self.encode(raw.to(**self.tensor_kwargs)).contiguous().float()
        if WAN2PT1_I2V_COND_LATENT_KEY not in batch:
            cond = torch.zeros_like(raw, **self.tensor_kwargs)
            if not is_image:
                cond[:, :, 0] = raw[:, :, 0]
            batch[WAN2PT1_I2V_COND_LATENT_KEY] = self.encode(cond).contiguous()
        from dataclasses import replace
        condition = self.conditioner(batch)
        condition = replace(condition, data_type=DataType.IMAGE if is_image else DataType.VIDEO)
        return raw, latent, condition
